"""Training through the server-side optimizer equals plain PyTorch training (one rank)."""
import copy

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


def _model(dev):
    torch.manual_seed(3)
    return nn.Sequential(nn.Linear(64, 200), nn.ReLU(), nn.Linear(200, 33), nn.ReLU(),
                         nn.Linear(33, 10)).to(dev)


@pytest.mark.parametrize("kind", ["momentum", "adam"])
@pytest.mark.parametrize("overlap", [False, True])
def test_matches_torch_optimizer(cuda_device, kind, overlap):
    from ps_lite_b200.parallel import ServerOptimizer, SymmetricHeap
    from ps_lite_b200.parallel.optimizer import DistributedOptimizer
    ref = _model(cuda_device)
    mine = copy.deepcopy(ref)
    heap = SymmetricHeap(8 << 20, 0, 1, device=cuda_device)
    if kind == "momentum":
        topt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
        sopt = ServerOptimizer("momentum", lr=0.05, momentum=0.9)
    else:
        topt = torch.optim.Adam(ref.parameters(), lr=0.01, eps=1e-6)
        sopt = ServerOptimizer("adam", lr=0.01, eps=1e-6)
    # tiny slices so that every tensor is cut and the priority queue is exercised
    dopt = DistributedOptimizer(mine.parameters(), heap, sopt, grad_dtype=torch.float32, blk=64,
                                slice_bytes=1024, overlap=overlap)
    for step in range(5):
        x = torch.randn(32, 64, device=cuda_device)
        y = torch.randint(0, 10, (32,), device=cuda_device)
        for m, o in ((ref, topt), (mine, dopt)):
            o.zero_grad()
            nn.functional.cross_entropy(m(x), y).backward()
            o.step()
        torch.cuda.synchronize()
        dopt.check()
        for a, b in zip(ref.parameters(), mine.parameters()):
            torch.testing.assert_close(b, a, rtol=1e-4, atol=1e-5)
    assert dopt.launched_slices > 5 * len(dopt.params)
