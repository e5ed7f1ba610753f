"""Host path head to head: the reference library over its ZMQ van versus this package's host
runtime over its TCP / Unix-socket van, same program, same machine.

The program is ``baseline/ref_bench.cc``, written against the reference's public API
(``ps::Start``, ``KVWorker::ZPush/ZPull/Wait``, ``KVServer`` with a request handle;
include/ps/kv_app.h of the reference).  The same source file is compiled twice: against the
unmodified reference (``baseline/build_ref.py``) and against ``include/`` +
``libpsb200_core`` of this package.  W workers + W servers + the scheduler run on localhost;
every worker pushes one fp32 tensor and pulls it back per step (shape of the reference's
tests/test_kv_app_benchmark.cc, with a sum + SGD server handle).  Wall-clock time inside the
workers, max over workers.

    python benchmarks/host_kv_bench.py [--workers 1 2] [--mb 1 16 64] [--steps 5]
"""
from __future__ import annotations

import argparse
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ps_lite_b200 import _build  # noqa: E402
from ps_lite_b200.launch.local import LocalJob  # noqa: E402


def build_ours() -> str:
    libs = _build.build_all()
    libdir = os.path.dirname(libs["core"])
    out_dir = os.path.join(ROOT, "build", "hostbench")
    os.makedirs(out_dir, exist_ok=True)
    exe = os.path.join(out_dir, "kv_bench_ours")
    src = os.path.join(ROOT, "baseline", "ref_bench.cc")
    if not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(src),
                                                              os.path.getmtime(libs["core"])):
        subprocess.check_call(["g++", "-std=c++17", "-O3", "-I", os.path.join(ROOT, "include"), src,
                               "-o", exe, "-L", libdir, "-lpsb200_core", f"-Wl,-rpath,{libdir}",
                               "-lpthread"])
    return exe


def run(exe: str, n: int, workers: int, steps: int, warmup: int, env: dict):
    saved = dict(os.environ)
    os.environ.update(env)
    try:
        job = LocalJob([exe, str(n), str(steps), str(warmup)], num_workers=workers,
                       num_servers=workers, capture=True)
        job.start()
        rc = job.wait(timeout=900)
        out = job.output()
    finally:
        os.environ.clear()
        os.environ.update(saved)
    secs = [float(m.group(1)) for m in re.finditer(r"REF_SECONDS ([0-9.]+)", out)]
    if rc != 0 or len(secs) != workers:
        return None
    return max(secs) * 1e3 / steps


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workers", type=int, nargs="+", default=[1, 2])
    ap.add_argument("--mb", type=float, nargs="+", default=[1, 16, 64])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    args = ap.parse_args()
    ours = build_ours()
    ref = os.path.join(ROOT, "baseline", "_ref", "ref_bench")
    arms = [("ours_tcp", ours, {}), ("ours_unix", ours, {"DMLC_LOCAL": "1"})]
    if os.path.exists(ref):
        arms += [("reference_zmq_tcp", ref, {}), ("reference_zmq_ipc", ref, {"DMLC_LOCAL": "1"})]
    for w in args.workers:
        for mb in args.mb:
            n = int(mb * (1 << 20)) // 4 // w * w
            row = {"workers": w, "servers": w, "tensor_mib": mb}
            for name, exe, env in arms:
                ms = run(exe, n, w, args.steps, args.warmup, env)
                row[name] = None if ms is None else {
                    "ms_per_step": round(ms, 3),
                    "GBps_per_worker": round(2.0 * n * 4 / (ms * 1e-3) / 1e9, 3)}
            print(json.dumps(row), flush=True)


if __name__ == "__main__":
    main()
