"""Extra records that bench.py appends to its one JSON line, so that a driver-run record holds
more than the headline point: the size sweep of the dense push+pull, the sparse logistic-
regression step, and the two model workloads (data-parallel ResNet-50 and BERT-large through
the server-side optimizer).  Every record is measured on the job that bench.py has already
started (same ranks, same heap); each is skipped once the run is older than the budget, and a
failure of one is reported in its place instead of ending the run."""
from __future__ import annotations

import json
import os
import time

import torch


def _baselines():
    """Library baselines measured with this repository's own baseline programs (NCCL
    reduce-scatter + SGD + all-gather; torch DDP + torch.optim) and kept beside the profiles."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "profiles",
                        "baselines_measured.json")
    try:
        with open(path) as fh:
            return json.load(fh)
    except (OSError, ValueError):
        return {}


def _sweep(ctx, rounds=30):
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    out = []
    ch = ctx.new_channel()
    nbytes = 4 << 10
    while nbytes <= 1 << 30:
        n = max(8 * world, nbytes // 4 // (8 * world) * (8 * world))
        t = DenseTable(ctx.heap, n, torch.float32, torch.float32,
                       optimizer=ServerOptimizer("sgd", lr=0.01), channel=ch)
        t.grad.copy_(torch.randn(n, device=dev))
        for _ in range(5):
            t.push_pull()
        torch.cuda.synchronize()
        ctx.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(rounds):
            t.push_pull()
        e1.record()
        torch.cuda.synchronize()
        ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / rounds
        t.check()
        out.append({"bytes": n * 4, "us_per_round": round(ms * 1e3, 2),
                    "goodput_GBps_per_gpu": round(2 * n * 4 / (ms * 1e-3) / 1e9, 2),
                    "path": "low-latency" if t.ll_cap >= n and world > 1 else
                            ("multicast" if t.nvls and t._multicast_pays(n * 4) else "peer")})
        t.free()
        nbytes *= 4
    return out


def _sparse(ctx, steps=10):
    import numpy as np
    from benchmarks.sparse_lr import zipf_keys
    from ps_lite_b200.parallel import SparseTable
    from ps_lite_b200.utils.oracle import ftrl_update
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    key_space, n = 1 << 30, 1 << 20
    table = SparseTable(ctx.heap, key_space, n, kind="ftrl")
    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)
    batches = [(zipf_keys(n, key_space, 1.1, gen, dev),
                torch.randn(n, generator=gen, device=dev) * 0.1) for _ in range(2)]
    keys0, g0 = batches[0]
    all_k, all_g = [keys0], [g0]
    if world > 1:
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
    ok = bool(torch.allclose(out, w[torch.searchsorted(uk, keys0)], rtol=1e-4, atol=1e-5))
    shared = 1.0 - uk.numel() / cat_k.numel()   # share of requests that hit a key of another worker
    for i in range(3):
        table.push_pull(*batches[i % 2])
    torch.cuda.synchronize()
    ctx.host_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        table.push_pull(*batches[i % 2])
    e1.record()
    torch.cuda.synchronize()
    table.check()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / steps
    all_ok = all(b == b"1" for b in ctx.allgather(b"1" if ok else b"0"))
    return {"metric": "sparse_lr_keys_per_s", "value": round(world * n / (ms * 1e-3)),
            "unit": "keys/s", "ms_per_step": round(ms, 4), "keys_per_worker_per_step": n,
            "key_space": key_space, "handle": "FTRL-proximal", "launches_per_step": 3,
            "first_step_matches_oracle": all_ok,
            "requests_on_keys_shared_between_workers": round(shared, 4)}


def run(ctx, kv, args, elapsed_s):
    """Returns {"sweep": [...], "sparse": {...}, "resnet50": {...}, "bert": {...}}; entries
    that were skipped for time say so."""
    t0 = time.time() - elapsed_s
    budget = args.extras_budget_s
    base = _baselines().get(str(ctx.world), {})
    out = {}

    def attempt(name, need_s, fn):
        # every rank takes the same decision: rank 0's clock decides
        mine = b"1" if time.time() - t0 + need_s < budget else b"0"
        go = ctx.allgather(mine)[0] == b"1"
        if not go:
            out[name] = {"skipped": f"run older than {budget:.0f} s"}
            return
        try:
            rec = fn()
        except Exception as exc:  # report instead of losing the headline record
            rec = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        if isinstance(rec, dict) and name in base:
            rec["baseline"] = base[name]
        out[name] = rec

    attempt("sweep", 15, lambda: _sweep(ctx))
    if "sweep" in base and isinstance(out.get("sweep"), list):
        out["sweep_baseline_nccl"] = base["sweep"]
    attempt("sparse", 25, lambda: _sparse(ctx))
    from benchmarks import workloads
    attempt("resnet50", 60, lambda: workloads.measure_ps(ctx, "resnet50", 8, 3))
    attempt("bert", 60, lambda: workloads.measure_ps(ctx, "bert", 6, 3))
    return out
