"""Radix sort of 64-bit keys (src/kernels/sort_match.cu) against torch.sort (CUB) on one GPU.

    python benchmarks/sort_bench.py

Keys are uniform below 2^30 (the key space of the sparse workload), uniform over 64 bits, and
Zipf-distributed below 2^30; 2^20 and 2^24 keys; with and without the permutation payload.
Each case: 3 warm-up and 10 timed runs on fresh copies of the input, CUDA events.  One JSON
line per case; `ratio` = this library's time / torch.sort's time.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200.ops.keys import sort_keys  # noqa: E402


def timed(fn, make, reps=10):
    for _ in range(3):
        fn(make())
    inputs = [make() for _ in range(reps)]
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for x in inputs:
        fn(x)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def main():
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    for log2n in (20, 24):
        n = 1 << log2n
        cases = {
            "uniform30": (torch.randint(0, 1 << 30, (n,), device=dev, dtype=torch.int64, generator=g), 30),
            "uniform64": (torch.randint(-(1 << 62), 1 << 62, (n,), device=dev, dtype=torch.int64,
                                        generator=g), 64),
            "zipf30": ((torch.rand(n, device=dev, dtype=torch.float64, generator=g).clamp_(1e-12)
                        .pow(-10.0).clamp_(max=float(1 << 30)).to(torch.int64) - 1), 30),
        }
        for name, (keys, bits) in cases.items():
            for payload in (False, True):
                ours = timed(lambda x: sort_keys(x, bits, return_perm=payload), keys.clone)
                ref = timed((lambda x: torch.sort(x, stable=True)) if payload
                            else (lambda x: torch.sort(x).values), keys.clone)
                print(json.dumps({"keys": n, "dist": name, "key_bits": bits, "payload": payload,
                                  "ours_us": round(ours, 1), "torch_sort_us": round(ref, 1),
                                  "ratio": round(ours / ref, 2),
                                  "ours_Gkeys_per_s": round(n / ours / 1e3, 2)}), flush=True)


if __name__ == "__main__":
    main()
