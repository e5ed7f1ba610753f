"""Sparse logistic-regression push/pull benchmark: key space 2^30, per worker and step 2^20
unique keys drawn from a Zipf(1.1) law, sorted, one fp32 gradient ~N(0, 0.01) each; the
server handle is FTRL-proximal (alpha 0.1, beta 1, l1 1, l2 1); the pull returns the weights
of the same keys.  Reports keys per second (whole job) and checks one step against the fp32
PyTorch statement of FTRL.

    python benchmarks/sparse_lr.py                       # one GPU
    python -m ps_lite_b200.launch.local --joint 8 python benchmarks/sparse_lr.py   # 8 GPUs
    python benchmarks/sparse_lr.py --cpu-oracle [--workers 8]   # timed CPU baseline, no GPU needed
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.parallel import SparseTable  # noqa: E402
from ps_lite_b200.utils.oracle import ftrl_update  # noqa: E402
from ps_lite_b200.utils.timing import max_over_ranks  # noqa: E402


def zipf_keys(n, key_space, s, gen, dev):
    """n unique keys, sorted; rank r drawn with P(r) ~ r^-s by inverting the Pareto CDF."""
    keys = torch.empty(0, dtype=torch.int64, device=dev)
    while keys.numel() < n:
        u = torch.rand(2 * n, generator=gen, device=dev, dtype=torch.float64).clamp_(1e-300, 1.0)
        r = torch.floor(u.pow(-1.0 / (s - 1.0))).clamp_(1, key_space).to(torch.int64) - 1
        # spread the ranks over the key space so that hot keys land on every server
        r = (r * 2654435761) % key_space
        keys = torch.unique(torch.cat([keys, r]))
    idx = torch.randperm(keys.numel(), generator=gen, device=dev)[:n]
    picked = keys[idx].contiguous()
    if picked.is_cuda:
        # unsorted keys become the sorted list a push needs with the library's own radix sort
        from ps_lite_b200.ops.keys import sort_keys
        return sort_keys(picked, max(1, (key_space - 1).bit_length()))[0]
    return torch.sort(picked).values


def cpu_oracle(args):
    """The same step as plain PyTorch on the host CPUs: the requests of `workers` workers are
    merged (sort + sum of duplicate keys, the server's view), FTRL runs on the touched
    coordinates of direct-indexed fp32 state, and every worker reads its keys back."""
    import time
    dev = torch.device("cpu")
    key_space, n, W = 1 << args.log2_key_space, 1 << args.log2_keys, args.workers
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234)
    batches = [[(zipf_keys(n, key_space, 1.1, gen, dev), torch.randn(n, generator=gen) * 0.1)
                for _ in range(W)] for _ in range(2)]
    z = torch.zeros(key_space)
    nn_ = torch.zeros(key_space)
    w = torch.zeros(key_space)

    def step(reqs):
        uk, inv = torch.unique(torch.cat([k for k, _ in reqs]), return_inverse=True)
        G = torch.zeros(uk.numel()).index_add_(0, inv, torch.cat([g for _, g in reqs]))
        zs, ns, ws = z[uk], nn_[uk], w[uk]
        ftrl_update(zs, ns, ws, G)
        z[uk], nn_[uk], w[uk] = zs, ns, ws
        return [w[k] for k, _ in reqs]

    for i in range(min(args.warmup, 2)):
        step(batches[i % 2])
    steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for i in range(steps):
        step(batches[i % 2])
    ms = (time.perf_counter() - t0) * 1e3 / steps
    print(json.dumps({"metric": "sparse_lr_keys_per_s", "impl": "cpu oracle (PyTorch, host CPUs)",
                      "value": round(W * n / (ms * 1e-3)), "unit": "keys/s", "workers": W,
                      "ms_per_step": round(ms, 2), "keys_per_worker_per_step": n,
                      "key_space": key_space, "threads": torch.get_num_threads(),
                      "handle": "FTRL-proximal"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2-key-space", type=int, default=30)
    ap.add_argument("--log2-keys", type=int, default=20)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cpu-oracle", action="store_true")
    ap.add_argument("--workers", type=int, default=1, help="workers merged by the CPU oracle")
    args = ap.parse_args()
    if args.cpu_oracle:
        return cpu_oracle(args)
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("DMLC_NUM_WORKER", "1")))
    key_space, n = 1 << args.log2_key_space, 1 << args.log2_keys
    per_rank = (key_space + world - 1) // world
    ctx = kvstore.init(heap_bytes=4 * per_rank + 20 * n + (64 << 20))
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    table = SparseTable(ctx.heap, key_space, n, kind="ftrl")
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    batches = [(zipf_keys(n, key_space, 1.1, gen, dev),
                torch.randn(n, generator=gen, device=dev) * 0.1) for _ in range(4)]

    # correctness of one step on a fresh table (rank-local oracle needs every rank's request)
    keys0, g0 = batches[0]
    all_k, all_g = [keys0], [g0]
    if world > 1:  # every rank's first request, over the control plane
        all_k = [torch.from_numpy(np.frombuffer(b, dtype=np.int64).copy()).to(dev)
                 for b in ctx.allgather(keys0.cpu().numpy().tobytes())]
        all_g = [torch.from_numpy(np.frombuffer(b, dtype=np.float32).copy()).to(dev)
                 for b in ctx.allgather(g0.cpu().numpy().tobytes())]
    out = table.push_pull(keys0, g0).clone()
    torch.cuda.synchronize()
    cat_k, cat_g = torch.cat(all_k), torch.cat(all_g)
    uk, inv = torch.unique(cat_k, return_inverse=True)
    G = torch.zeros(uk.numel(), device=dev).index_add_(0, inv, cat_g)
    z, nn_, w = torch.zeros_like(G), torch.zeros_like(G), torch.zeros_like(G)
    ftrl_update(z, nn_, w, G)
    ref = w[torch.searchsorted(uk, keys0)]
    ok = bool(torch.allclose(out, ref, rtol=1e-4, atol=1e-5))

    for i in range(args.warmup):
        table.push_pull(*batches[i % 4])
    torch.cuda.synchronize()
    ctx.host_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        table.push_pull(*batches[i % 4])
    e1.record()
    torch.cuda.synchronize()
    table.check()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    if rank == 0:
        print(json.dumps({"metric": "sparse_lr_keys_per_s", "value": round(world * n / (ms * 1e-3)),
                          "unit": "keys/s", "n_gpus": world, "ms_per_step": round(ms, 4),
                          "keys_per_worker_per_step": n, "key_space": key_space,
                          "handle": "FTRL-proximal", "first_step_matches_oracle": ok,
                          "timing": "device, CUDA events, max over ranks; includes staging the "
                                    "request into the heap, push, FTRL, pull"}), flush=True)
    kvstore.finalize()


if __name__ == "__main__":
    main()
