"""Dense push+pull bandwidth sweep: one tensor per round, 4 KB ... 1 GB in powers of 4.

``--impl ours``  : the fused push+pull kernel of this package (sum over workers + SGD lr 0.01
                   on the owners' fp32 master weights, contiguous key ranges, one per rank).
``--impl nccl``  : the library baseline: ``reduce_scatter_tensor`` -> SGD step on the shard ->
                   ``all_gather_into_tensor`` through ``torch.distributed``.
Goodput per GPU = (bytes pushed + bytes pulled by the worker) / time, timed with CUDA events
over ``--rounds`` rounds after warm-up, max over ranks.  One JSON line per size on rank 0.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        benchmarks/dense_sweep.py --impl ours --dtype fp32
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "nccl"])
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--rounds", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--min-kb", type=int, default=4)
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--graph", action="store_true", help="replay the rounds from a CUDA graph")
    args = ap.parse_args()
    if args.graph and args.impl == "nccl":
        # capturing torch.distributed collectives together with the optimizer kernels did not
        # terminate on this setup (4 GPUs); the baseline is timed with ordinary launches
        print(json.dumps({"impl": "nccl", "graph": True,
                          "unavailable": "NCCL collectives are not graph-captured here"}))
        return
    dt = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    isz = 4 if args.dtype == "fp32" else 2
    sizes = []
    b = args.min_kb << 10
    while b <= args.max_mb << 20:
        sizes.append(b)
        b *= 4

    from ps_lite_b200.utils.timing import max_over_ranks
    if args.impl == "ours":
        # a parameter-server job: ps::Start + device plane, no collective library
        from ps_lite_b200 import kvstore
        from ps_lite_b200.parallel import ServerOptimizer
        ctx = kvstore.init(heap_bytes=2 * sizes[-1] + (64 << 20))
        rank, world, dev = ctx.rank, ctx.world, ctx.device
    else:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if args.impl == "ours":
            ctx.host_barrier()
        elif world > 1:
            dist.barrier()

    for nbytes in sizes:
        n = nbytes // isz
        n = max(8 * world, n // (8 * world) * (8 * world))
        torch.manual_seed(rank)
        if args.impl == "ours":
            from ps_lite_b200.parallel import DenseTable
            t = DenseTable(ctx.heap, n, dt, dt, optimizer=ServerOptimizer("sgd", lr=0.01),
                           channel=ctx.new_channel())
            t.grad.copy_(torch.randn(n, device=dev).to(dt))
            step = t.push_pull
        else:
            grad = torch.randn(n, device=dev).to(dt)
            shard = torch.empty(n // world, device=dev, dtype=dt)
            master = torch.zeros(n // world, device=dev, dtype=torch.float32)
            weights = torch.empty(n, device=dev, dtype=dt)
            out_shard = torch.empty(n // world, device=dev, dtype=dt)

            def step():
                if world > 1:
                    dist.reduce_scatter_tensor(shard, grad)
                else:
                    shard.copy_(grad)
                master.add_(shard.float(), alpha=-0.01)
                out_shard.copy_(master)
                if world > 1:
                    dist.all_gather_into_tensor(weights, out_shard)
                else:
                    weights.copy_(out_shard)
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.graph:
            # the rounds are captured once and replayed: launch cost leaves the measurement
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(args.rounds):
                    step()
            graph.replay()
            torch.cuda.synchronize()
            barrier()
            torch.cuda.synchronize()
            e0.record()
            graph.replay()
            e1.record()
        else:
            e0.record()
            for _ in range(args.rounds):
                step()
            e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1), dev) / args.rounds
        if rank == 0:
            print(json.dumps({"impl": args.impl, "dtype": args.dtype, "n_gpus": world, "graph": bool(args.graph),
                              "bytes": n * isz, "us_per_round": round(ms * 1e3, 2),
                              "goodput_GBps_per_gpu": round(2 * n * isz / (ms * 1e-3) / 1e9, 2)}),
                  flush=True)
        if args.impl == "ours":
            t.check()
            ctx.heap.free(t.grad_off)
            ctx.heap.free(t.weight_off)
    if args.impl == "ours":
        kvstore.finalize()
    elif world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
