#!/usr/bin/env python
"""Headline benchmark: dense push+pull goodput (the reference's test_kv_app_benchmark shape).

Every GPU is a worker and a server shard.  One step = every worker pushes one fp32 tensor
(values ~N(0,1)) to the key-range-sharded servers, the server handle sums the workers'
tensors and applies SGD (lr 0.01) to its fp32 master weights, and every worker pulls the
updated tensor.  Goodput per GPU = (bytes pushed + bytes pulled by that worker) / time;
``value`` is the sum over all GPUs.  Per-GPU work is fixed as N grows (weak scaling).

    python bench.py --gpus 1 --steps 50 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 50 --warmup 5

``--impl reference`` runs the unmodified reference library (baseline/_ref) on the same
shape through its own KVWorker/KVServer API over its ZMQ van.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "push_pull_goodput_GBps"
T_START = time.time()


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="pushpull", choices=["pushpull", "resnet50", "bert"])
    ap.add_argument("--size-mb", type=float, default=256.0, help="tensor bytes per worker (MiB)")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--ctas", type=int, default=0)
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the extra records (size sweep, sparse LR, model workloads)")
    ap.add_argument("--extras-budget-s", type=float, default=240.0,
                    help="the extra records stop being started once the run is this old")
    ap.add_argument("--slice-mb", type=float, default=16.0,
                    help="slice size of the end-to-end staging pipeline (MiB)")
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--trainer", default="ps", choices=["ps", "ddp"],
                    help="model workloads: this package's server-side optimizer, or the "
                         "torch DistributedDataParallel + torch.optim baseline over NCCL")
    return ap.parse_args()


def run_pushpull(args):
    import torch

    from ps_lite_b200 import kvstore
    from ps_lite_b200.launch import bootstrap
    from ps_lite_b200.parallel import ServerOptimizer
    from ps_lite_b200.utils.timing import ClockSampler

    gdt = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    isz = 4 if args.dtype == "fp32" else 2
    world_hint = int(os.environ.get("WORLD_SIZE", os.environ.get("DMLC_NUM_WORKER", "1")))
    n = int(args.size_mb * (1 << 20)) // isz
    n = max(8 * world_hint, n // (8 * world_hint) * (8 * world_hint))
    nbytes = n * isz
    # ps::Start from the launcher's environment, then the device plane: arena handles and
    # barriers travel over the parameter server's own control plane (no collective library)
    heap_bytes = 2 * nbytes + (64 << 20)
    if not args.no_extras:
        # room for the extra records: the 1 GiB point of the sweep, the sparse table's
        # accumulator (4 bytes per key of the rank's range) and the models' buffers
        heap_bytes += (2 << 30) + (4 << 30) // world_hint + (4 << 30)
    ctx = kvstore.init(heap_bytes=heap_bytes, slice_bytes=int(args.slice_mb * (1 << 20)))
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    local = dev.index or 0
    reporter = bootstrap.launcher_rank() == 0
    kv = kvstore.KVStore(ctx)
    # sum over workers + SGD lr 0.01; contiguous key ranges, one per server
    opt = ServerOptimizer("sgd", lr=0.01, scale=1.0)
    table = kv.declare(0, n, grad_dtype=gdt, out_dtype=gdt, optimizer=opt, num_ctas=args.ctas)
    g = torch.Generator(device=dev)
    g.manual_seed(1234 + rank)
    table.grad.copy_(torch.randn(n, device=dev, generator=g).to(gdt))
    from ps_lite_b200 import host
    L = host.lib()

    # ---- device-timed: K fused push+pull rounds on resident gradients, each one a
    # KVWorker::ZPushPull on the tensor's keys with values that already sit in the arena ------
    warmup = max(3, args.warmup)
    for _ in range(warmup):
        kv.push_pull(0)
    kv.wait_all()
    torch.cuda.synchronize()
    ctx.host_barrier()
    sampler = ClockSampler(local, period_ms=50)
    if reporter:
        sampler.start()
        time.sleep(0.3)
    ctx.host_barrier()
    torch.cuda.synchronize()
    launches0 = L.psnvl_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        kv.push_pull(0)
    e1.record()
    kv.wait_all()          # raises if a device-side wait ran out
    torch.cuda.synchronize()
    launches = L.psnvl_launches() - launches0
    ctx.host_barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = ms / args.steps
    per_gpu = 2.0 * nbytes / (ms_per_step * 1e-3) / 1e9
    value = per_gpu * world

    # ---- end to end: pinned host gradients in, pulled weights back to pinned host ---------
    e2e = None
    if not args.skip_e2e:
        hin = torch.randn(n, dtype=torch.float32).to(gdt).pin_memory()
        hout = torch.empty(n, dtype=gdt).pin_memory()
        for _ in range(max(3, min(warmup, 5))):
            kv.wait(kv.push_pull(0, hin, hout))
        torch.cuda.synchronize()
        ctx.host_barrier()
        torch.cuda.synchronize()
        k2 = max(3, min(args.steps, 20))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(k2):
            kv.wait(kv.push_pull(0, hin, hout))
        s1.record()
        torch.cuda.synchronize()
        ctx.host_barrier()
        ms2 = ctx.max_over_ranks(s0.elapsed_time(s1)) / k2
        # what the same bytes take as plain copies on this box, all ranks at once, no kernel
        from benchmarks.host_copy_ceiling import both_directions_ms
        ceiling_ms = both_directions_ms(ctx, hin, hout)
        e2e = {"value": round(world * 2.0 * nbytes / (ms2 * 1e-3) / 1e9, 3), "unit": "GB/s",
               "ms_per_step": round(ms2, 4), "steps": k2,
               "plain_copies_ms": round(ceiling_ms, 4),
               "ms_over_plain_copies": round(ms2 / ceiling_ms, 3),
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "slice_mib": args.slice_mb,
               "api": "KVStore.push_pull(pinned host tensor, out=pinned host tensor); wait(ts) "
                      "= KVWorker::ZPushPull + Wait through ps::Start and the device plane"}
    # the sampler ran through both timed regions (device-timed and end-to-end)
    clocks = sampler.stop() if reporter else None

    def headline():
        return {
            "metric": METRIC, "value": round(value, 3), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic N(0,1) gradients, random-init weights",
            "impl": "ours",
            "config": {"model": "dense push+pull (test_kv_app_benchmark shape)",
                       "tensor_bytes_per_worker": nbytes, "global_bytes": nbytes * world,
                       "global_batch": world, "seq_len": n,
                       "parallelism": f"dp{world} workers x {world} key-range server shards",
                       "server_handle": "sum over workers + SGD lr=0.01 on fp32 master",
                       "per_gpu_goodput_GBps": round(per_gpu, 3),
                       "value_is": "kernel goodput on device-resident gradients; e2e.value is "
                                   "the same metric from pinned host memory and back",
                       "control_plane": f"ps::Start ({ctx.launch_mode} launch), heap "
                                        f"{ctx.heap.backend}, multicast {bool(ctx.heap.mc_base)}",
                       "l2": "inputs larger than L2 (gradient+weight+master per step > 126 MB)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": int(launches),
        }

    def record(extras):
        return dict(headline(), **extras)

    extras = {}
    if not args.no_extras:
        from benchmarks import extras as extras_mod
        # the extra records must never cost the headline: if they are still running long after
        # their budget (a rank that left one of them early leaves the others waiting for it),
        # the headline is printed without them and the process ends
        import threading

        def give_up():
            if reporter:
                print(json.dumps(record({"extras": "abandoned: still running "
                                         f"{time.time() - T_START:.0f} s after start"})),
                      flush=True)
            from ps_lite_b200.launch import bootstrap
            bootstrap.abandon()
            os._exit(0)

        watchdog = threading.Timer(max(60.0, args.extras_budget_s + 180.0 -
                                       (time.time() - T_START)), give_up)
        watchdog.daemon = True
        watchdog.start()
        extras = extras_mod.run(ctx, kv, args, time.time() - T_START)
        watchdog.cancel()

    if reporter:
        print(json.dumps(record(extras)), flush=True)
    kvstore.finalize()


def run_reference(args):
    from baseline import ref_arm
    ref_arm.main(args)


def main():
    args = parse_args()
    if args.impl == "reference":
        try:
            run_reference(args)
        except Exception as exc:  # the arm must always answer with one JSON line
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference",
                                  "unavailable": f"{type(exc).__name__}: {exc}"[:300]}))
        return
    if args.workload == "pushpull":
        run_pushpull(args)
    else:
        from benchmarks import workloads
        workloads.run(args)


if __name__ == "__main__":
    main()
