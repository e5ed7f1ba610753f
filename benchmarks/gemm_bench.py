"""Times the tcgen05 GEMM of this package against torch.matmul (cuBLAS) on one GPU.

    python benchmarks/gemm_bench.py [--shapes 16384x3072x1024,...] [--iters 20]

Each timed iteration is preceded by an L2 flush (a 256 MB memset); times are CUDA-event
times of the kernel alone; one JSON line per shape.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200.ops.gemm import gemm_status, linear_bf16  # noqa: E402
from ps_lite_b200.utils.timing import flush_l2  # noqa: E402


def timed(fn, iters, dev):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        flush_l2(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="16384x3072x1024,16384x1024x1024,16384x4096x1024,8192x8192x8192,2048x3072x1024")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--tile", type=int, default=0, help="output tile height: 128, 256, 0 = auto")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from ps_lite_b200 import _lib
    _lib.check(_lib.device_lib().psdev_gemm_config(args.tile), "psdev_gemm_config")
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak = peaks.get("bf16_tflops", 1590.0)
    for shape in args.shapes.split(","):
        M, N, K = (int(v) for v in shape.split("x"))
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ours = timed(lambda: linear_bf16(x, w, out, num_ctas=args.ctas), args.iters, dev)
        assert gemm_status(dev) == 0
        ref_out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        lib = timed(lambda: torch.matmul(x, w.t(), out=ref_out), args.iters, dev)
        err = (out.float() - ref_out.float()).abs().max().item()
        fl = 2.0 * M * N * K
        print(json.dumps({"shape": [M, N, K], "tile": args.tile, "ours_us": round(ours * 1e3, 1),
                          "cublas_us": round(lib * 1e3, 1),
                          "ours_tflops": round(fl / ours / 1e9, 1),
                          "cublas_tflops": round(fl / lib / 1e9, 1),
                          "ours_frac_of_measured_peak": round(fl / ours / 1e9 / peak, 3),
                          "max_abs_diff_vs_cublas": err}), flush=True)


if __name__ == "__main__":
    main()
