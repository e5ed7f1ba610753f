"""Reference arm of bench.py: the unmodified reference library on the same metric and shape.

N workers and N servers (plus the scheduler) of the reference run on this host's CPUs over
its ZMQ van on localhost; every worker pushes one fp32 tensor of the configured size per step
and pulls it back (``baseline/ref_bench.cc``).  The reference has no GPU path, so nothing of it
runs on a GPU; its time is the wall-clock time its workers measure around the K timed steps,
maximum over workers.  Rank 0 starts all processes and prints the JSON line.
"""
from __future__ import annotations

import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
EXE = os.path.join(HERE, "_ref", "ref_bench")


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why[:300]}), flush=True)


def main(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if rank != 0:
        return
    if args.workload != "pushpull":
        _unavailable("the reference library has no model or training code; only the dense "
                     "push+pull workload exists for it")
        return
    if not os.path.exists(EXE):
        try:
            sys.path.insert(0, ROOT)
            from baseline import build_ref, reference_source
            src = reference_source()
            if src is None:
                raise FileNotFoundError("set PS_REFERENCE_SRC to the reference sources")
            build_ref.build(src)
        except Exception as exc:
            _unavailable(f"reference build not present and cannot be built here: {exc}")
            return
    sys.path.insert(0, ROOT)
    from ps_lite_b200.launch.local import LocalJob
    isz = 4
    n = int(args.size_mb * (1 << 20)) // isz
    n = max(8 * world, n // (8 * world) * (8 * world))
    nbytes = n * isz
    steps, warmup = args.steps, max(args.warmup, 1)
    job = LocalJob([EXE, str(n), str(steps), str(warmup)], num_workers=world, num_servers=world,
                   capture=True)
    job.start()
    rc = job.wait(timeout=3600)
    out = job.output()
    secs = [float(m.group(1)) for m in re.finditer(r"REF_SECONDS ([0-9.]+)", out)]
    if rc != 0 or len(secs) != world:
        _unavailable(f"reference run failed (rc={rc}, {len(secs)}/{world} workers reported): "
                     + out[-160:].replace("\n", " "))
        return
    sec = max(secs)
    ms = sec * 1e3 / steps
    per_gpu = 2.0 * nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "push_pull_goodput_GBps", "value": round(per_gpu * world, 4), "unit": "GB/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "impl": "reference",
        "config": {"model": "dense push+pull (test_kv_app_benchmark shape)",
                   "tensor_bytes_per_worker": nbytes, "global_bytes": nbytes * world,
                   "parallelism": f"{world} workers x {world} servers + scheduler, ZMQ van, "
                                  "TCP localhost, CPU memory",
                   "server_handle": "sum over workers + SGD lr=0.01",
                   "timing": "wall clock inside the reference's workers, max over workers",
                   "per_gpu_goodput_GBps": round(per_gpu, 4)},
        "e2e": {"value": round(per_gpu * world, 4), "unit": "GB/s",
                "note": "the reference works on host memory; its number is end to end already",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}), flush=True)
