"""Heap arenas from the virtual-memory-management API (src/device/vmm_heap.cu): export as a file
descriptor, second mapping through the descriptor, and the fused dense kernel on such arenas
against the fp32 PyTorch statement of the update."""
import ctypes as C
import os

import pytest
import torch

from ps_lite_b200.utils.oracle import dense_update

pytestmark = pytest.mark.gpu


@pytest.fixture()
def lib(cuda_device):
    from ps_lite_b200 import _lib
    torch.cuda.set_device(cuda_device)
    torch.zeros(1, device=cuda_device)
    lib = _lib.device_lib()
    if not lib.psdev_vmm_supported():
        pytest.skip("device cannot export allocations as file descriptors")
    return lib


def test_arena_is_shared_through_its_descriptor(cuda_device, lib):
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel.heap import tensor_from_ptr
    nbytes = 8 << 20
    base, fd, mapped = C.c_void_p(), C.c_int(-1), C.c_size_t(0)
    _lib.check(lib.psdev_vmm_create(nbytes, C.byref(base), C.byref(fd), C.byref(mapped)), "create")
    assert mapped.value >= nbytes and fd.value >= 0
    other = C.c_void_p()
    _lib.check(lib.psdev_vmm_import(fd.value, mapped.value, C.byref(other)), "import")
    os.close(fd.value)
    assert other.value != base.value
    a = tensor_from_ptr(base.value, nbytes, cuda_device)
    b = tensor_from_ptr(other.value, nbytes, cuda_device)
    assert int(a[:_lib.CTRL_BYTES].max()) == 0          # control region starts cleared
    pattern = torch.arange(nbytes, device=cuda_device, dtype=torch.int64).to(torch.uint8)
    a.copy_(pattern)
    torch.cuda.synchronize()
    assert torch.equal(b, pattern)                       # same physical memory
    b[123] = 77
    torch.cuda.synchronize()
    assert int(a[123]) == 77
    del a, b
    assert lib.psdev_vmm_release(other) == 0
    assert lib.psdev_vmm_release(base) == 0
    assert lib.psdev_vmm_release(base) != 0              # unknown by now


@pytest.mark.parametrize("world", [1, 4])
def test_dense_push_pull_on_vmm_arenas(cuda_device, lib, world):
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    torch.manual_seed(7)
    n = 50_000
    nbytes = 65536 + 4 * (n + 64) * 8 + (1 << 20)
    opt = ServerOptimizer("momentum", lr=0.05, momentum=0.9, scale=1.0 / world)
    if world == 1:
        heaps = [SymmetricHeap(nbytes, 0, 1, device=cuda_device, backend="vmm")]
    else:
        heaps = SymmetricHeap.emulated(nbytes, world, device=cuda_device, backend="vmm")
    assert heaps[0].backend == "vmm" or world > 1
    tables = [DenseTable(h, n, torch.float32, torch.float32, blk=1024, optimizer=opt)
              for h in heaps]
    npad = tables[0].n
    w0 = torch.randn(npad, device=cuda_device)
    w0[n:] = 0
    for t in tables:
        t.load_master(w0)
    ref_w, s1, s2 = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
    for step in range(1, 3):
        grads = []
        for t in tables:
            g = torch.randn(npad, device=cuda_device)
            g[n:] = 0
            t.grad.copy_(g)
            grads.append(g)
        for t in tables:
            t.push_pull(sync=False)
        torch.cuda.synchronize()
        dense_update(ref_w, grads, "momentum", lr=0.05, momentum=0.9, scale=1.0 / world, step=step,
                     s1=s1, s2=s2)
        for t in tables:
            torch.testing.assert_close(t.weight[:n], ref_w[:n], rtol=2e-5, atol=2e-5)
    del tables
    for h in heaps:
        for o in getattr(h, "_siblings", []):
            o.close()
        h.close()
