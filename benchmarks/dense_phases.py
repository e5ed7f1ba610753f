"""Push-only, pull-only and fused push+pull of the dense kernel, peer path against NVSwitch
multicast path, over sizes and grid sizes: shows which half of a round limits it.

    python -m ps_lite_b200.launch.local --joint N python benchmarks/dense_phases.py

fp32 gradients and weights, sum + SGD handle.  Each case: 5 warm-up and 20 timed launches, CUDA
events on the launching stream, maximum over ranks; every launch rendezvouses with the other
ranks.  Bytes counted per launch and GPU: push = the tensor (its gradients are read once by
their owners), pull = the tensor (every value is written into this GPU's weight buffer),
push+pull = twice the tensor.  PHASES_MB selects the sizes (default "16,64,256,1024"),
PHASES_CTAS the grid sizes (default "0,148,296,592"; 0 = the library's default).
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import _lib, kvstore  # noqa: E402
from ps_lite_b200.parallel import DenseTable, ServerOptimizer  # noqa: E402


def main():
    sizes = [int(v) << 20 for v in os.environ.get("PHASES_MB", "16,64,256,1024").split(",")]
    ctas_list = [int(v) for v in os.environ.get("PHASES_CTAS", "0,148,296,592").split(",")]
    ctx = kvstore.init(heap_bytes=2 * max(sizes) + (64 << 20))
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    paths = [("peer", False)] + ([("multicast", True)] if ctx.heap.mc_base and world > 1 else [])
    ch = ctx.new_channel()
    for nbytes in sizes:
        n = nbytes // 4 // (8 * world) * (8 * world)
        for path, nvls in paths:
            t = DenseTable(ctx.heap, n, torch.float32, torch.float32,
                           optimizer=ServerOptimizer("sgd", lr=0.01), channel=ch, nvls=nvls)
            t.nvls_max_bytes = 1 << 62
            t.grad.copy_(torch.randn(n, device=dev))
            for ctas in ctas_list:
                t.num_ctas = ctas
                for name, op, factor in (("push", _lib.OP_PUSH, 1), ("pull", _lib.OP_PULL, 1),
                                         ("push_pull", _lib.OP_PUSHPULL, 2)):
                    for _ in range(5):
                        t._run(op, 0, None, True, None, None, False)
                    torch.cuda.synchronize()
                    ctx.host_barrier()
                    e0 = torch.cuda.Event(enable_timing=True)
                    e1 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(20):
                        t._run(op, 0, None, True, None, None, False)
                    e1.record()
                    torch.cuda.synchronize()
                    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / 20
                    t.check()
                    if rank == 0:
                        print(json.dumps({"path": path, "op": name, "bytes": n * 4, "ctas": ctas,
                                          "n_gpus": world, "us": round(ms * 1e3, 1),
                                          "GBps_per_gpu": round(factor * n * 4 / (ms * 1e-3) / 1e9, 1)}),
                              flush=True)
            ctx.heap.free(t.grad_off)
            ctx.heap.free(t.weight_off)
    kvstore.finalize()


if __name__ == "__main__":
    main()
