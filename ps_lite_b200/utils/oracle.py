"""Plain PyTorch fp32 statements of the server-side updates, used as test oracles.

The sum handle restates the reference's ``KVServerDefaultHandle`` (include/ps/kv_app.h:
440-463).  SGD, momentum, Adam and FTRL-proximal have no counterpart in the reference; the
formulas are the ones the device kernels implement.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch


def dense_update(w: torch.Tensor, grads: Sequence[torch.Tensor], kind: str, *, lr=0.01,
                 momentum=0.9, weight_decay=0.0, beta1=0.9, beta2=0.999, eps=1e-8, scale=1.0,
                 step=1, s1: Optional[torch.Tensor] = None, s2: Optional[torch.Tensor] = None):
    """Apply one push of ``grads`` (one tensor per worker) to fp32 ``w`` in place.

    Gradients are summed in worker-rank order in fp32, like the kernels do.
    """
    g = torch.zeros_like(w, dtype=torch.float32)
    for x in grads:
        g += x.to(torch.float32)
    g *= scale
    if kind == "sum":
        w += g
    elif kind == "assign":
        w.copy_(g)
    elif kind == "sgd":
        g = g + weight_decay * w
        w -= lr * g
    elif kind == "momentum":
        g = g + weight_decay * w
        s1.mul_(momentum).add_(g)
        w -= lr * s1
    elif kind in ("adam", "adamw"):
        if kind == "adamw":
            w *= (1.0 - lr * weight_decay)
        else:
            g = g + weight_decay * w
        s1.mul_(beta1).add_((1.0 - beta1) * g)
        s2.mul_(beta2).add_((1.0 - beta2) * g * g)
        bias1 = 1.0 - beta1 ** step
        bias2 = math.sqrt(1.0 - beta2 ** step)
        denom = s2.sqrt() / bias2 + eps
        w -= (lr / bias1) * (s1 / denom)
    else:
        raise ValueError(kind)
    return w


def ftrl_update(z: torch.Tensor, n: torch.Tensor, w: torch.Tensor, g: torch.Tensor, *,
                alpha=0.1, beta=1.0, l1=1.0, l2=1.0):
    """FTRL-proximal on the touched coordinates (all tensors same shape, fp32, in place)."""
    sigma = ((n + g * g).sqrt() - n.sqrt()) / alpha
    z += g - sigma * w
    n += g * g
    shrink = torch.sign(z) * l1 - z
    denom = (beta + n.sqrt()) / alpha + l2
    w.copy_(torch.where(z.abs() <= l1, torch.zeros_like(z), shrink / denom))
    return w
