"""Small single-GPU cases of the kernels that have no benchmark of their own, for profiling.

    python benchmarks/kernel_cases.py --case sparse|filters|sort|p3|barrier [--iters 3]

Each case builds its inputs (larger than the 126 MB L2 where DRAM figures matter, a few GB at
most), runs the kernels `--iters` times and prints CUDA-event times per launch group as one JSON
line.  The ncu summaries under ``profiles/`` were captured on these commands.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import _lib  # noqa: E402
from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SparseTable, SymmetricHeap  # noqa: E402


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return round(e0.elapsed_time(e1) / iters * 1e3, 1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["sparse", "filters", "sort", "p3", "barrier"])
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    out = {"case": args.case}
    if args.case == "sparse":
        key_space, n = 1 << 28, 1 << 22
        heap = SymmetricHeap(4 * key_space + 24 * n + (64 << 20), 0, 1, device=dev)
        t = SparseTable(heap, key_space, n, kind="ftrl")
        keys = torch.sort(torch.randperm(key_space, device=dev)[:n]).values
        grads = torch.randn(n, device=dev) * 0.1
        t.stage(keys, grads)
        # whole steps (an apply without a scatter before it finds nothing to do); the phases are
        # timed inside the steps
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.iters)]
        for _ in range(2):
            t.scatter(), t.apply(), t.respond()
        torch.cuda.synchronize()
        for e in ev:
            e[0].record()
            t.scatter()
            e[1].record()
            t.apply()
            e[2].record()
            t.respond()
            e[3].record()
        torch.cuda.synchronize()
        for j, name in enumerate(("scatter_us", "apply_us", "respond_us")):
            out[name] = round(sum(e[j].elapsed_time(e[j + 1]) for e in ev) / len(ev) * 1e3, 1)
        out["keys"] = n
        t.check()
    elif args.case == "filters":
        from ps_lite_b200.ops import filters as F
        x = torch.randn(64 << 20, device=dev)
        out["cast_scale_256MiB_us"] = timed(lambda: F.cast_scale(x, torch.bfloat16, 0.5), args.iters)
        q, sc = F.int8_pack(x)
        out["int8_pack_256MiB_us"] = timed(lambda: F.int8_pack(x), args.iters)
        y = torch.empty_like(x)
        out["int8_unpack_us"] = timed(lambda: F.int8_unpack(q, sc, out=y), args.iters)
    elif args.case == "sort":
        from ps_lite_b200.ops.keys import sort_keys
        keys = torch.randint(0, 1 << 30, (1 << 24,), device=dev, dtype=torch.int64)
        out["sort_2^24_30bit_perm_us"] = timed(lambda: sort_keys(keys.clone(), 30, return_perm=True),
                                               args.iters)
    elif args.case == "p3":
        n = 64 << 20
        heap = SymmetricHeap(8 * n + (64 << 20), 0, 1, device=dev)
        t = DenseTable(heap, n, torch.float32, torch.float32, blk=4096,
                       optimizer=ServerOptimizer("sgd", lr=0.01))
        t.grad.normal_()
        segs = [(i * (n // 256), (i + 1) * (n // 256), i % 17) for i in range(256)]
        out["push_pull_256_slices_one_launch_us"] = timed(
            lambda: t.run_multi(_lib.OP_PUSHPULL, segs), args.iters)
        t.check()
    else:
        heap = SymmetricHeap(1 << 20, 0, 1, device=dev)
        out["device_barrier_us"] = timed(lambda: heap.barrier(), max(args.iters, 10))
    print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
