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
    print("CHECKS_OK", refused, flush=True)


if __name__ == "__main__":
    main()
