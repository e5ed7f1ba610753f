"""Communication filters on the device: cast/scale and int8 block-scale compression."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

GROUP = 256


def _s(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def cast_scale(x: torch.Tensor, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """fp32 -> bf16 or bf16 -> fp32 with a scale factor."""
    x = x.contiguous()
    out = torch.empty_like(x, dtype=dtype)
    if x.dtype == torch.float32 and dtype == torch.bfloat16:
        d = 0
    elif x.dtype == torch.bfloat16 and dtype == torch.float32:
        d = 1
    else:
        raise ValueError("cast_scale handles fp32<->bf16")
    _lib.check(_lib.device_lib().psdev_filter_cast(x.data_ptr(), out.data_ptr(), x.numel(),
                                                   float(scale), d, _s(x.device)), "filter_cast")
    return out


def int8_pack(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 -> (int8 values, fp32 scales per 256 values)."""
    x = x.contiguous().view(-1)
    q = torch.empty(x.numel(), dtype=torch.int8, device=x.device)
    scales = torch.empty((x.numel() + GROUP - 1) // GROUP, dtype=torch.float32, device=x.device)
    _lib.check(_lib.device_lib().psdev_filter_int8_pack(x.data_ptr(), q.data_ptr(),
                                                        scales.data_ptr(), x.numel(),
                                                        _s(x.device)), "int8_pack")
    return q, scales


def int8_unpack(q: torch.Tensor, scales: torch.Tensor, out: Optional[torch.Tensor] = None,
                accumulate: bool = False) -> torch.Tensor:
    if out is None:
        out = torch.zeros(q.numel(), dtype=torch.float32, device=q.device)
    _lib.check(_lib.device_lib().psdev_filter_int8_unpack(q.data_ptr(), scales.data_ptr(),
                                                          out.data_ptr(), q.numel(),
                                                          1 if accumulate else 0, _s(q.device)),
               "int8_unpack")
    return out
