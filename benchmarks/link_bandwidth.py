"""NVLink peer-memory bandwidth of the box, the denominator of the fused kernels' rooflines.

Run as a parameter-server job with at least two joint processes:

    python -m ps_lite_b200.launch.local --joint 2 python benchmarks/link_bandwidth.py

Times the library's 16-byte load/store copy kernel (``psdev_link_copy``) between arenas of
the symmetric heap: local -> local, peer -> local (remote loads) and local -> peer (remote
stores), with one active rank and with all ranks at once, for several grid sizes.  CUDA
events on the launching stream, 3 warm-up launches, 10 timed, maximum over ranks (gathered
over the control plane).  Rank 0 prints one JSON line per measurement; the table kept in
``profiles/`` is made from them.  Buffers of LINK_MB MiB (default 256: larger than L2).
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import _lib, kvstore  # noqa: E402


def main():
    nbytes = int(os.environ.get("LINK_MB", "256")) << 20
    ctx = kvstore.init(heap_bytes=2 * nbytes + (8 << 20))
    rank, world = ctx.rank, ctx.world
    heap = ctx.heap
    a, b = heap.alloc(nbytes), heap.alloc(nbytes)
    lib = _lib.device_lib()
    peer = (rank + 1) % world
    stream = torch.cuda.current_stream()

    def run(dst, src, ctas, everyone):
        active = everyone or rank == 0
        ctx.host_barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if active:
            for _ in range(3):
                lib.psdev_link_copy(dst, src, nbytes, ctas, stream.cuda_stream)
            e0.record()
            for _ in range(10):
                lib.psdev_link_copy(dst, src, nbytes, ctas, stream.cuda_stream)
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10 if active else 0.0
        return nbytes / (ctx.max_over_ranks(ms) * 1e-3) / 1e9

    me, pr = heap.bases[rank], heap.bases[peer]
    for ctas in (74, 148, 296, 592):
        for name, dst, src in (("local", me + b, me + a), ("peer_read", me + b, pr + a),
                               ("peer_write", pr + b, me + a)):
            if world == 1 and name != "local":
                continue
            for everyone in (False, True):
                gbs = run(dst, src, ctas, everyone)
                if rank == 0:
                    print(json.dumps({"link": name, "ctas": ctas, "all_ranks": everyone,
                                      "n_gpus": world, "heap": heap.backend,
                                      "GBps_per_gpu": round(gbs, 1), "bytes": nbytes}), flush=True)
    kvstore.finalize()


if __name__ == "__main__":
    main()
