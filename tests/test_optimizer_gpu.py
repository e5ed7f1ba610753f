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


def test_training_with_pull_fused_into_first_gemm(cuda_device):
    """The first layer's weight is pushed with publish and pulled by the GEMM that consumes it;
    training must follow an fp32-master SGD reference within bf16 tolerance."""
    from ps_lite_b200.ops.gemm import gemm_status, pull_linear
    from ps_lite_b200.parallel import ServerOptimizer, SymmetricHeap
    from ps_lite_b200.parallel.optimizer import DistributedOptimizer
    torch.manual_seed(11)
    K, H, O, B = 256, 512, 16, 384
    w1 = nn.Parameter((torch.randn(H, K, device=cuda_device) * 0.05).to(torch.bfloat16))
    w2 = nn.Parameter((torch.randn(O, H, device=cuda_device) * 0.05).to(torch.bfloat16))
    m1, m2 = w1.detach().float().clone(), w2.detach().float().clone()  # fp32 masters of the reference
    heap = SymmetricHeap(16 << 20, 0, 1, device=cuda_device)
    dopt = DistributedOptimizer([w1, w2], heap, ServerOptimizer("sgd", lr=0.05),
                                grad_dtype=torch.bfloat16, blk=1024, slice_bytes=64 << 10,
                                publish_first=1)
    off = dopt.offset_of(w1)
    for step in range(4):
        x = torch.randn(B, K, device=cuda_device).to(torch.bfloat16)
        y = torch.randn(B, O, device=cuda_device)
        # reference step on bf16 copies of the fp32 masters
        r1 = m1.to(torch.bfloat16).requires_grad_(True)
        r2 = m2.to(torch.bfloat16).requires_grad_(True)
        ((torch.relu(x @ r1.t()) @ r2.t()).float() - y).pow(2).mean().backward()
        m1 -= 0.05 * r1.grad.float()
        m2 -= 0.05 * r2.grad.float()
        dopt.zero_grad()
        h = torch.relu(pull_linear(x, w1, dopt.table, off))
        ((h @ w2.t()).float() - y).pow(2).mean().backward()
        dopt.step()
        torch.cuda.synchronize()
        dopt.check()
        assert gemm_status(cuda_device) == 0
        torch.testing.assert_close(w2.float(), m2.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-3)
    # w1's storage is refreshed by the fused pull of the next forward pass
    x = torch.randn(B, K, device=cuda_device).to(torch.bfloat16)
    pull_linear(x, w1, dopt.table, off)
    torch.cuda.synchronize()
    torch.testing.assert_close(w1.float(), m1.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-3)
