"""A server handle written by the application runs inside the fused push kernel: the example
``tests/cuda/user_handle_clip.cu`` is compiled into its own shared object, loaded, and checked
against the same update in plain PyTorch fp32 (1 rank and 4 ranks emulated on one GPU)."""
import ctypes
import os
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def clip_handle(cuda_device):
    from ps_lite_b200 import _build, _lib
    lib = _build.build_device()
    _lib.device_lib()
    out = os.path.join(ROOT, "build", "tests", "libuser_handle_clip.so")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [_build.NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3",
           "-shared", "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cuda", "user_handle_clip.cu"), "-o", out, str(lib),
           "-Xlinker", f"-rpath={os.path.dirname(str(lib))}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    return ctypes.CDLL(out, mode=ctypes.RTLD_GLOBAL)   # static constructor registers kind 100


@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_clipped_sgd_handle(cuda_device, clip_handle, world, dt):
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    assert _lib.device_lib().psdev_handle_states(100) == 0
    assert _lib.device_lib().psdev_handle_states(101) == -1
    torch.manual_seed(3)
    n, clip, lr = 100_000, 0.25, 0.5
    opt = ServerOptimizer("user", lr=lr, user_kind=100, user=(clip,))
    heaps = SymmetricHeap.emulated(64 << 20, world, device=cuda_device)
    tables = [DenseTable(h, n, dt, dt, blk=1024, optimizer=opt) for h in heaps]
    w0 = torch.randn(tables[0].n, device=cuda_device)
    grads = [torch.randn(tables[0].n, device=cuda_device).to(dt) for _ in range(world)]
    for t, g in zip(tables, grads):
        t.load_master(w0)
        t.grad.copy_(g)
    ref = w0.clone()
    for step in range(2):
        for t in tables:           # every rank's server role, back to back on one GPU
            t.push_pull(sync=False)
        torch.cuda.synchronize()
        gsum = sum(g.float() for g in grads)
        ref -= lr * gsum.clamp(-clip, clip)
    tol = dict(rtol=1e-2, atol=1e-2) if dt == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)
    for t in tables:
        torch.testing.assert_close(t.weight[:n].float(), ref[:n].to(dt).float(), **tol)
    for h in heaps:
        h.close()


def test_unregistered_kind_is_refused(cuda_device):
    from ps_lite_b200.parallel import ServerOptimizer
    with pytest.raises(ValueError):
        ServerOptimizer("user", user_kind=177).num_states
