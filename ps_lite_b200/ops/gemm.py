"""bf16 GEMM on the tcgen05 tensor cores, alone or fused with the pull of its weights."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _lib


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def gemm_status(device) -> int:
    """Error word of the last GEMM launches on ``device`` (0 = none); synchronises."""
    st = C.c_int32()
    with torch.cuda.device(device):
        _lib.check(_lib.device_lib().psdev_gemm_status(C.byref(st)), "psdev_gemm_status")
    return st.value


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                num_ctas: int = 0, timeout_s: float = 2.0) -> torch.Tensor:
    """``out[M,N] = x[M,K] @ w[N,K]^T`` (bf16 in, fp32 accumulate, bf16 out)."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.is_contiguous() and w.is_contiguous() and x.shape[-1] == w.shape[-1]
    M, K = x.numel() // x.shape[-1], x.shape[-1]
    N = w.shape[0]
    if out is None:
        out = torch.empty(*x.shape[:-1], N, dtype=torch.bfloat16, device=x.device)
    rc = _lib.device_lib().psdev_gemm_bf16(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K,
                                           num_ctas, int(timeout_s * 1e9), _stream(x.device))
    _lib.check(rc, "psdev_gemm_bf16")
    return out


def pull_linear_bf16(table, w_offset: int, n_out: int, x: torch.Tensor,
                     out: Optional[torch.Tensor] = None, num_copy_ctas: int = 0,
                     num_ctas: int = 0, timeout_s: float = 2.0) -> torch.Tensor:
    """Pull ``W = table.weight[w_offset : w_offset + n_out*K]`` (viewed ``[n_out, K]``) from its
    owners and compute ``x @ W^T`` in the same kernel.

    Must follow, on the same stream, a ``table.push(..., publish=True)`` covering that range.
    Afterwards ``table.weight`` holds the complete W locally (for the backward pass).
    """
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    assert table.out_dtype == torch.bfloat16
    K = x.shape[-1]
    M = x.numel() // K
    if out is None:
        out = torch.empty(*x.shape[:-1], n_out, dtype=torch.bfloat16, device=x.device)
    rc = _lib.device_lib().psdev_pull_gemm_bf16(
        C.byref(table._world), C.byref(table._table), int(w_offset), x.data_ptr(), out.data_ptr(),
        M, n_out, K, num_copy_ctas, num_ctas, int(timeout_s * 1e9), _stream(x.device))
    _lib.check(rc, "psdev_pull_gemm_bf16")
    return out


def fusion_pays(weight_bytes: int, world: int) -> bool:
    """Whether pulling a weight inside the GEMM that consumes it beats push+pull followed by
    the GEMM.  Measured (benchmarks/pull_gemm_bench.py): with a 128 MiB weight the fused form
    is 1.12-1.16x faster; with the 6 MiB QKV weight of BERT-large it is slower (0.96x on 2 GPUs,
    0.91x on 4: the cooperative launch and the per-panel waits cost more than the pull they
    hide).  The switch-over lies between; ``PSB200_FUSE_MIN_MB`` (default 32) sets it."""
    import os
    if world < 2:
        return False
    return weight_bytes >= int(os.environ.get("PSB200_FUSE_MIN_MB", "32")) << 20


class _PullLinearFn(torch.autograd.Function):
    """``x @ W^T`` where W is pulled from its owners inside the GEMM kernel.

    ``weight`` is the parameter whose storage is the table's weight slice: the kernel fills
    it while multiplying, so the backward pass can use it as an ordinary local tensor."""

    @staticmethod
    def forward(ctx, x, weight, table, w_offset):
        n_out, k = weight.shape
        x2 = x.reshape(-1, k).contiguous()
        out = pull_linear_bf16(table, w_offset, n_out, x2)
        ctx.save_for_backward(x2, weight)
        ctx.x_shape = x.shape
        return out.view(*x.shape[:-1], n_out)

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, weight.shape[0])
        dx = (dy2 @ weight).view(ctx.x_shape)
        dw = dy2.t() @ x2
        return dx, dw, None, None


def pull_linear(x: torch.Tensor, weight: torch.nn.Parameter, table, w_offset: int) -> torch.Tensor:
    """Differentiable form of :func:`pull_linear_bf16` for a parameter stored in ``table``."""
    return _PullLinearFn.apply(x, weight, table, w_offset)
