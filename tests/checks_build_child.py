"""Child of test_device_checks_gpu.py: runs in a process that loaded the checks variant of the
device library (PSB200_DEVICE_CHECKS=1).  Prints CHECKS_OK when everything held."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ps_lite_b200 import _lib  # noqa: E402
from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap  # noqa: E402
from ps_lite_b200.utils.oracle import dense_update  # noqa: E402


def main():
    assert os.environ.get("PSB200_DEVICE_CHECKS") == "1"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    world, n, blk = 2, 40_000, 1024
    opt = ServerOptimizer("sgd", lr=0.1, scale=1.0 / world)
    heaps = SymmetricHeap.emulated(65536 + 4 * (n + 64) * 8 + (1 << 20), world, device=dev)
    tables = [DenseTable(h, n, torch.float32, torch.float32, blk=blk, optimizer=opt)
              for h in heaps]
    npad = tables[0].n
    torch.manual_seed(3)
    w0 = torch.randn(npad, device=dev)
    for t in tables:
        t.load_master(w0)
    grads = [torch.randn(npad, device=dev) for _ in range(world)]

    # 1. consistent arguments: the checks stay silent and the result is the oracle's
    for t, g in zip(tables, grads):
        t.grad.copy_(g)
    for t in tables:
        t.push_pull(sync=False)
    torch.cuda.synchronize()
    ref = w0.clone()
    dense_update(ref, grads, "sgd", lr=0.1, scale=1.0 / world)
    for t in tables:
        t.check()
        torch.testing.assert_close(t.weight[:n], ref[:n], rtol=2e-5, atol=2e-5)

    # 2. the kernel is told that the table is 4096 elements shorter than it is: vectors in the
    #    tail are refused (status PSDEV_ERR_BOUNDS) and left alone, the rest is updated
    os.environ["PSDEV_CHECKS_TEST_SHRINK"] = "4096"
    before = [t.weight.clone() for t in tables]
    for t, g in zip(tables, grads):
        t.grad.copy_(g)
    for t in tables:
        t.push_pull(sync=False)
    torch.cuda.synchronize()
    del os.environ["PSDEV_CHECKS_TEST_SHRINK"]
    ref2 = ref.clone()
    dense_update(ref2, grads, "sgd", lr=0.1, scale=1.0 / world)
    cut = npad - 4096
    refused = 0
    for t, b in zip(tables, before):
        try:
            t.check()
        except _lib.PsdevError as exc:
            assert exc.code == -8, exc
            refused += 1
        torch.testing.assert_close(t.weight[:cut], ref2[:cut], rtol=2e-5, atol=2e-5)
        assert torch.equal(t.weight[cut:], b[cut:]), "refused vectors must not be written"
    assert refused >= 1, "the tail belongs to at least one rank"
    for h in heaps:
        h.close()

    # 3. sparse kernels: silent on a consistent table; told that the store has fewer slots
    #    than it has, they refuse the keys beyond (status PSDEV_ERR_BOUNDS on the table's
    #    channel) and leave them alone -- no address outside an allocation is formed
    from ps_lite_b200.parallel import SparseTable
    key_space, nk = 1 << 14, 2000
    heap = SymmetricHeap(65536 + 64 * nk + 4 * key_space + (1 << 20), 0, 1, device=dev)
    st = SparseTable(heap, key_space, nk, kind="sum")
    keys = torch.sort(torch.randperm(key_space, device=dev)[:nk]).values
    vals = torch.randn(nk, device=dev)
    out = st.push_pull(keys, vals).clone()
    torch.cuda.synchronize()
    st.check()
    torch.testing.assert_close(out, vals)
    st._t.slots = key_space // 2          # the lie: every address still lies inside the store
    out = st.push_pull(keys, vals).clone()
    torch.cuda.synchronize()
    try:
        st.check()
        raise AssertionError("the sparse kernels accepted slots beyond the stated capacity")
    except _lib.PsdevError as exc:
        assert exc.code == -8, exc
    low = keys < key_space // 2
    torch.testing.assert_close(out[low], 2 * vals[low])
    assert torch.equal(st.w[key_space // 2:][keys[~low] - key_space // 2], vals[~low]), \
        "refused keys must keep their old values"
    heap.close()
    print("CHECKS_OK", refused, flush=True)


if __name__ == "__main__":
    main()
