"""Ceiling of the end-to-end push+pull path: what plain copies between pinned host memory and
the GPUs reach on this box when N ranks copy at once.

    python -m ps_lite_b200.launch.local --joint N python benchmarks/host_copy_ceiling.py

Every rank owns COPY_MB MiB (default 256) of pinned input and output and a device buffer, and
times ``cudaMemcpyAsync`` alone -- no kernel: host-to-device only, device-to-host only, and
both directions at once on two streams (what one step of ``KVStore.push_pull`` on host tensors
must move), as whole-buffer copies and in slices of 16 MiB.  All ranks start together after a
barrier; CUDA events, 3 warm-up and 10 timed repetitions, maximum over ranks.  Rank 0 prints
one JSON line per case with GB/s per direction per GPU and the step time that the bytes of one
push+pull would need.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import kvstore  # noqa: E402


def both_directions_ms(ctx, hin, hout, reps=5):
    """Milliseconds (maximum over ranks) that one whole-buffer copy of ``hin`` to the device
    and, at the same time, one of the same size from the device into ``hout`` take when every
    rank copies at once: the floor of a step that moves these bytes, whatever runs between."""
    dev = ctx.device
    din = torch.empty(hin.numel(), dtype=hin.dtype, device=dev)
    dout = torch.zeros(hout.numel(), dtype=hout.dtype, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def once():
        with torch.cuda.stream(s_in):
            din.copy_(hin, non_blocking=True)
        with torch.cuda.stream(s_out):
            hout.copy_(dout, non_blocking=True)

    for _ in range(2):
        once()
    torch.cuda.synchronize()
    ctx.host_barrier()
    cur = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    for _ in range(reps):
        once()
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    e1.record()
    torch.cuda.synchronize()
    return ctx.max_over_ranks(e0.elapsed_time(e1)) / reps


def main():
    nbytes = int(os.environ.get("COPY_MB", "256")) << 20
    ctx = kvstore.init(heap_bytes=64 << 20)
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    hin = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    hout = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    hin.fill_(1)
    din = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    dout = torch.ones(nbytes, dtype=torch.uint8, device=dev)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def copies(h2d, d2h, slice_bytes):
        for b in range(0, nbytes, slice_bytes):
            e = min(b + slice_bytes, nbytes)
            if h2d:
                with torch.cuda.stream(s_in):
                    din[b:e].copy_(hin[b:e], non_blocking=True)
            if d2h:
                with torch.cuda.stream(s_out):
                    hout[b:e].copy_(dout[b:e], non_blocking=True)

    for name, h2d, d2h in (("h2d", True, False), ("d2h", False, True), ("both", True, True)):
        for slice_mb in (0, 16):
            sl = nbytes if slice_mb == 0 else slice_mb << 20
            for _ in range(3):
                copies(h2d, d2h, sl)
            torch.cuda.synchronize()
            ctx.host_barrier()
            cur = torch.cuda.current_stream()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            for _ in range(10):
                copies(h2d, d2h, sl)
            cur.wait_stream(s_in)
            cur.wait_stream(s_out)
            e1.record()
            torch.cuda.synchronize()
            ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / 10
            if rank == 0:
                print(json.dumps({"case": name, "slice_mib": slice_mb or nbytes >> 20,
                                  "n_gpus": world, "bytes_per_direction": nbytes,
                                  "ms": round(ms, 3),
                                  "GBps_per_direction_per_gpu": round(nbytes / (ms * 1e-3) / 1e9, 2),
                                  "GBps_all_gpus_all_directions": round(
                                      world * nbytes * (int(h2d) + int(d2h)) / (ms * 1e-3) / 1e9, 1)}),
                      flush=True)
    kvstore.finalize()


if __name__ == "__main__":
    main()
