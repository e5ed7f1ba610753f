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

``--kv-app-benchmark`` runs the reference's own benchmark program instead
(tests/test_kv_app_benchmark.cc: 10 M keys with one float each, one push and one pull through a
server handle that stores nothing), again compiled unchanged against both libraries, and
reports its "Push/Pull average time cost".
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


def build_kv_app_benchmark():
    """The reference's tests/test_kv_app_benchmark.cc against this runtime and, when the
    reference has been built (baseline/build_ref.py), against the reference."""
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    src = os.path.join(ref_root, "ps-lite", "tests", "test_kv_app_benchmark.cc")
    if not os.path.exists(src):
        from baseline import reference_source
        if reference_source() is None:
            raise FileNotFoundError("set PS_REFERENCE_SRC to the reference sources")
        src = os.path.join(reference_source(), "tests", "test_kv_app_benchmark.cc")
    libs = _build.build_all()
    libdir = os.path.dirname(libs["core"])
    out_dir = os.path.join(ROOT, "build", "hostbench")
    os.makedirs(out_dir, exist_ok=True)
    ours = os.path.join(out_dir, "kv_app_benchmark_ours")
    subprocess.check_call(["g++", "-std=c++17", "-O3", "-I", os.path.join(ROOT, "include"), src,
                           "-o", ours, "-L", libdir, "-lpsb200_core", f"-Wl,-rpath,{libdir}",
                           "-lpthread"])
    ref = None
    if os.path.exists(os.path.join(ref_root, "libps.a")):
        from baseline.build_ref import find_libzmq
        zmq = find_libzmq()
        ref = os.path.join(out_dir, "kv_app_benchmark_ref")
        subprocess.check_call(
            ["g++", "-std=c++11", "-msse2", "-fPIC", "-O3", "-I", os.path.join(ref_root, "ps-lite", "src"),
             "-I", os.path.join(ref_root, "ps-lite", "include"), "-I", os.path.join(ref_root, "deps", "include"),
             "-Wno-unused-function", "-Wno-deprecated-declarations", src,
             os.path.join(ref_root, "libps.a"), zmq, f"-Wl,-rpath,{os.path.dirname(zmq)}", "-pthread",
             "-o", ref])
    return ours, ref


def run_kv_app_benchmark(exe: str, workers: int, env: dict):
    saved = dict(os.environ)
    os.environ.update(env)
    try:
        job = LocalJob([exe], num_workers=workers, num_servers=workers, capture=True)
        job.start()
        rc = job.wait(timeout=900)
        out = job.output()
    finally:
        os.environ.clear()
        os.environ.update(saved)
    push = [float(x) for x in re.findall(r"Push average time cost: ([0-9.]+)ms", out)]
    pull = [float(x) for x in re.findall(r"Pull average time cost: ([0-9.]+)ms", out)]
    if rc != 0 or len(push) != workers or len(pull) != workers:
        return None
    return {"push_ms": round(max(push), 1), "pull_ms": round(max(pull), 1)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workers", type=int, nargs="+", default=[1, 2])
    ap.add_argument("--mb", type=float, nargs="+", default=[1, 16, 64])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--kv-app-benchmark", action="store_true")
    args = ap.parse_args()
    if args.kv_app_benchmark:
        ours, ref = build_kv_app_benchmark()
        arms = [("ours_tcp", ours, {}), ("ours_unix_shm", ours, {"DMLC_LOCAL": "1"}),
                ("ours_unix_no_shm", ours, {"DMLC_LOCAL": "1", "PS_SHM": "0"})]
        if ref:
            arms += [("reference_zmq_tcp", ref, {}), ("reference_zmq_ipc", ref, {"DMLC_LOCAL": "1"})]
        for w in args.workers:
            row = {"program": "test_kv_app_benchmark", "workers": w, "servers": w,
                   "keys_per_worker": 10000000}
            for name, exe, env in arms:
                row[name] = run_kv_app_benchmark(exe, w, env)
            print(json.dumps(row), flush=True)
        return
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
