"""Multi-GPU checks run as joint processes of a parameter-server job (``python -m
ps_lite_b200.launch.local --joint N python
tests/mp_fused_check.py``): (1) push with publish followed by the pull fused with
the tcgen05 GEMM, (2) sparse push/pull with FTRL across ranks, (3) a small model trained
through the server-side optimizer on different data per rank equals single-process training
on the averaged gradient.  Rank 0 prints MP_FUSED_OK when every rank agreed."""
import copy
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.ops.gemm import gemm_status, pull_linear_bf16  # noqa: E402
from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SparseTable  # noqa: E402
from ps_lite_b200.parallel.optimizer import DistributedOptimizer  # noqa: E402
from ps_lite_b200.utils.oracle import ftrl_update  # noqa: E402


def seeded(seed, n, dev, scale=1.0):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randn(n, device=dev, generator=g) * scale


def main():
    ctx = kvstore.init(heap_bytes=512 << 20)
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    ok = True

    def expect(cond, what):
        nonlocal ok
        if not cond:
            ok = False
            print(f"rank {rank}: FAILED {what}", flush=True)

    # (1) fused pull + GEMM
    M, N, K, pad = 2048, 1536, 1024, 4096
    n = pad + N * K + 1024
    t = DenseTable(ctx.heap, n, torch.bfloat16, torch.bfloat16, blk=4096,
                   optimizer=ServerOptimizer("sgd", lr=0.5), channel=ctx.new_channel())
    w0 = seeded(1, t.n, dev, 0.05)
    t.load_master(w0)
    for step in range(1, 3):
        grads = [seeded(100 * step + r, t.n, dev, 0.01).to(torch.bfloat16) for r in range(world)]
        t.grad.copy_(grads[rank])
        t.weight.fill_(float("nan"))
        t.push(publish=True)
        x = seeded(7 + step, M * K, dev).to(torch.bfloat16).view(M, K)
        out = pull_linear_bf16(t, pad, N, x)
        torch.cuda.synchronize()
        t.check()
        expect(gemm_status(dev) == 0, "gemm status")
        w0 = w0 - 0.5 * sum(g.float() for g in grads)
        W = w0[pad:pad + N * K].to(torch.bfloat16).view(N, K)
        ref = x.float() @ W.float().t()
        expect(torch.allclose(out.float(), ref, rtol=3e-2, atol=3e-2), f"fused gemm step {step}")
        expect(torch.allclose(t.weight[pad:pad + N * K].float(), W.reshape(-1).float(),
                              rtol=1e-2, atol=1e-2), f"pulled W step {step}")

    # (2) sparse FTRL
    key_space, nk = 1 << 22, 50000
    st = SparseTable(ctx.heap, key_space, nk, kind="ftrl")
    Wt = torch.zeros(key_space, device=dev)
    Z, Nn = torch.zeros_like(Wt), torch.zeros_like(Wt)
    for step in range(3):
        reqs = []
        for r in range(world):
            g = torch.Generator(device=dev)
            g.manual_seed(1000 * step + r)
            u = torch.rand(3 * nk, generator=g, device=dev, dtype=torch.float64)
            keys = torch.unique(((key_space ** u).to(torch.int64) - 1).clamp_(0, key_space - 1))[:nk]
            grads = torch.randn(keys.numel(), generator=g, device=dev) * 0.5
            reqs.append((keys, grads))
        out = st.push_pull(*reqs[rank])
        torch.cuda.synchronize()
        st.check()
        G = torch.zeros_like(Wt)
        touched = torch.zeros(key_space, dtype=torch.bool, device=dev)
        for keys, grads in reqs:
            G.index_add_(0, keys, grads)
            touched[keys] = True
        idx = touched.nonzero().squeeze(1)
        z, nn_, w = Z[idx], Nn[idx], Wt[idx]
        ftrl_update(z, nn_, w, G[idx])
        Z[idx], Nn[idx], Wt[idx] = z, nn_, w
        expect(torch.allclose(out, Wt[reqs[rank][0]], rtol=1e-3, atol=1e-4), f"sparse step {step}")

    # (2b) the same kind of table through KVWorker requests (KeyedStore): FTRL, width 2, and a
    # table with per-key lengths whose pull returns the lengths the owners hold
    ks = kvstore.KeyedStore(ctx, 11, key_space, nk, width=2, kind="ftrl", alpha=0.1, beta=1.0,
                            l1=1.0, l2=1.0)
    W2 = torch.zeros(key_space, 2, device=dev)
    Z2, N2 = torch.zeros_like(W2), torch.zeros_like(W2)
    for step in range(2):
        reqs = []
        for r in range(world):
            g = torch.Generator(device=dev)
            g.manual_seed(7000 * step + r)
            keys = torch.unique(torch.randint(0, key_space, (nk // 2,), device=dev, generator=g))
            vals = torch.randn(keys.numel(), 2, generator=g, device=dev) * 0.5
            reqs.append((keys, vals))
        keys, vals = reqs[rank]
        out = torch.empty_like(vals)
        ks.wait(ks.push_pull(keys, vals.reshape(-1).contiguous(), out.view(-1)))
        G = torch.zeros_like(W2)
        touched = torch.zeros(key_space, dtype=torch.bool, device=dev)
        for k, v in reqs:
            G.index_add_(0, k, v)
            touched[k] = True
        idx = touched.nonzero().squeeze(1)
        z, nn_, w = Z2[idx], N2[idx], W2[idx]
        ftrl_update(z, nn_, w, G[idx])
        Z2[idx], N2[idx], W2[idx] = z, nn_, w
        expect(torch.allclose(out, W2[keys], rtol=1e-3, atol=1e-4), f"keyed store step {step}")
    kl = kvstore.KeyedStore(ctx, 12, 1 << 16, 4000, width=3, kind="sum", var_len=True)
    g = torch.Generator(device=dev)
    g.manual_seed(99)      # every rank pushes the same keys: the sum is world x the values
    keys = torch.unique(torch.randint(0, 1 << 16, (3000,), device=dev, generator=g))
    lens = (keys % 3 + 1).int()
    vals = torch.randn(int(lens.sum()), device=dev, generator=g)
    kl.wait(kl.push(keys, vals, lens))
    ask = keys[rank::2].contiguous()       # a different request on every rank
    out = torch.zeros(ask.numel() * 3, device=dev)
    lens_back = torch.full((ask.numel(),), -1, device=dev, dtype=torch.int32)
    kl.wait(kl.pull(ask, out, lens_back))
    expect(torch.equal(lens_back, (ask % 3 + 1).int()), "lengths returned by a keyed pull")
    offs = torch.cumsum(lens.long(), 0) - lens.long()
    pos = torch.searchsorted(keys, ask)
    got_offs = torch.cumsum(lens_back.long(), 0) - lens_back.long()
    good = True
    for j in range(3):
        m = lens[pos] > j
        good = good and torch.allclose(out[(got_offs + j)[m]], world * vals[(offs[pos] + j)[m]],
                                       rtol=1e-5, atol=1e-5)
    expect(good, "values returned by a keyed pull with lengths")

    # (3) data-parallel training through the server-side optimizer
    torch.manual_seed(5)
    ref = nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 8)).to(dev)
    mine = copy.deepcopy(ref)
    topt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    dopt = DistributedOptimizer(mine.parameters(), ctx.heap,
                                ServerOptimizer("momentum", lr=0.1, momentum=0.9, scale=1.0 / world),
                                grad_dtype=torch.float32, blk=64, slice_bytes=2048,
                                channel=ctx.new_channel())
    for step in range(4):
        xs = [seeded(50 * step + r, 16 * 32, dev).view(16, 32) for r in range(world)]
        ys = [seeded(900 + 50 * step + r, 16 * 8, dev).view(16, 8) for r in range(world)]
        topt.zero_grad()
        sum(nn.functional.mse_loss(ref(x), y) for x, y in zip(xs, ys)).div(world).backward()
        topt.step()
        dopt.zero_grad()
        nn.functional.mse_loss(mine(xs[rank]), ys[rank]).backward()
        dopt.step()
        torch.cuda.synchronize()
        dopt.check()
        for a, b in zip(ref.parameters(), mine.parameters()):
            expect(torch.allclose(a, b, rtol=1e-4, atol=1e-5), f"training step {step}")

    ctx.heap.barrier()
    torch.cuda.synchronize()
    all_ok = all(b == b"1" for b in ctx.allgather(b"1" if ok else b"0"))
    if rank == 0 and all_ok:
        print(f"MP_FUSED_OK world={world} heap={ctx.heap.backend}", flush=True)
    kvstore.finalize()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
