"""Where the time of an end-to-end push+pull on host tensors goes: the three legs of the staged
pipeline alone and together, over slice sizes, beside plain copies into the same memory.

    python -m ps_lite_b200.launch.local --joint N python benchmarks/e2e_phases.py
    (or plain ``python benchmarks/e2e_phases.py`` for one GPU)

256 MiB fp32 per worker (E2E_MB), sum + SGD handle.  Cases, each 3 warm-up + 10 timed requests,
CUDA events, maximum over ranks, every request waited for before the next one starts:

* ``push``       pinned host gradients -> device -> kernel (no pull)
* ``pull``       kernel -> device weights -> pinned host (no push)
* ``push_pull``  both, the three streams overlapping (what ``bench.py`` times end to end)
* ``copies``     plain ``cudaMemcpyAsync`` of the same bytes, host to the table's gradient
                 buffer in the arena and the table's weight buffer to host, on two streams,
                 whole buffers, no kernel: the floor of ``push_pull`` on this box.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import host, kvstore  # noqa: E402
from ps_lite_b200.parallel import ServerOptimizer  # noqa: E402


def main():
    nbytes = int(os.environ.get("E2E_MB", "256")) << 20
    slices = [int(v) for v in os.environ.get("E2E_SLICES_MB", "4,16,64").split(",")]
    n = nbytes // 4
    ctx = kvstore.init(heap_bytes=2 * nbytes + (64 << 20))
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    kv = kvstore.KVStore(ctx)
    t = kv.declare(0, n, optimizer=ServerOptimizer("sgd", lr=0.01))
    hin = torch.randn(n).pin_memory()
    hout = torch.empty(n).pin_memory()

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ctx.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return ctx.max_over_ranks(e0.elapsed_time(e1)) / reps

    def emit(**kw):
        if rank == 0:
            print(json.dumps(dict(kw, n_gpus=world, bytes_per_direction=nbytes)), flush=True)

    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def copies():
        cur = torch.cuda.current_stream()
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            t.grad[:n].copy_(hin, non_blocking=True)
        with torch.cuda.stream(s_out):
            hout.copy_(t.weight[:n], non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    emit(case="copies", ms=round(timed(copies), 3))
    for mb in slices:
        host._ck(host.lib().psnvl_set_slice_bytes(mb << 20))
        for name, fn in (("push", lambda: kv.wait(kv.push(0, hin))),
                         ("pull", lambda: kv.wait(kv.pull(0, hout))),
                         ("push_pull", lambda: kv.wait(kv.push_pull(0, hin, hout)))):
            emit(case=name, slice_mib=mb, ms=round(timed(fn), 3))
        # host time of the call that queues a whole request (copies, kernels, events)
        import time
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ts = kv.push_pull(0, hin, hout)
        t1 = time.perf_counter()
        kv.wait(ts)
        emit(case="push_pull: host time of the call", slice_mib=mb, ms=round((t1 - t0) * 1e3, 3))
    t.check()
    kvstore.finalize()


if __name__ == "__main__":
    main()
