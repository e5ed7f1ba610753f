"""The GEMM entry point that allocates nothing, called through its exported C symbol.

Some users of this library run where device allocation is off limits after start-up (the
whole GPU belongs to a framework's memory pool, or a latency-critical thread may not enter
the driver's allocator).  ``psdev_gemm_bf16_noalloc`` keeps its counters in a fixed array
inside the library instead of a ``cudaMalloc`` block.  Here it must give the same product as
the ordinary entry point, twice in a row (the second call finds the array as the first left
it), and must refuse an output wider than its array can track.

This file sorts last on purpose: a run that stops at the first failure has by then run
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ps_lite_b200 import _build
    lib = C.CDLL(str(_build.build_device()))
    vp, i64, u64 = C.c_void_p, C.c_int64, C.c_uint64
    lib.psdev_gemm_bf16.restype = C.c_int
    lib.psdev_gemm_bf16.argtypes = [vp, vp, vp, i64, i64, i64, C.c_int, u64, vp]
    lib.psdev_gemm_bf16_noalloc.restype = C.c_int
    lib.psdev_gemm_bf16_noalloc.argtypes = [vp, vp, vp, i64, i64, i64, C.c_int, u64, vp, vp]
    return lib


def test_no_alloc_gemm_matches_regular_entry_point_twice(cuda_device):
    lib = _lib()
    torch.cuda.set_device(cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.full((1,), 123, dtype=torch.int32, device=cuda_device)
    for call, (M, N, K) in enumerate([(512, 768, 256), (1000, 392, 520)]):
        torch.manual_seed(call)
        x = torch.randn(M, K, device=cuda_device).to(torch.bfloat16)
        w = (torch.randn(N, K, device=cuda_device) / K ** 0.5).to(torch.bfloat16)
        ref = torch.empty(M, N, device=cuda_device, dtype=torch.bfloat16)
        out = torch.full((M, N), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        assert lib.psdev_gemm_bf16(x.data_ptr(), w.data_ptr(), ref.data_ptr(), M, N, K, 0,
                                   2_000_000_000, stream) == 0
        assert lib.psdev_gemm_bf16_noalloc(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K,
                                           0, 2_000_000_000, status.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(out.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-2)


def test_no_alloc_gemm_rejects_outputs_beyond_its_limit(cuda_device):
    lib = _lib()
    torch.cuda.set_device(cuda_device)
    dummy = torch.zeros(64, device=cuda_device, dtype=torch.bfloat16)
    n_too_wide = 1023 * 256 + 256   # 1024 panels of 256 columns
    rc = lib.psdev_gemm_bf16_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 8,
                                     n_too_wide, 8, 0, 0, None,
                                     torch.cuda.current_stream().cuda_stream)
    assert rc == -7   # PSDEV_ERR_TOO_LARGE; nothing was launched
    torch.cuda.synchronize()
