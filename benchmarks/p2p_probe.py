"""NVLink peer-memory bandwidth probe (run under torchrun with >= 2 ranks).

Times the library's 16-byte load/store copy kernel for: local->local, peer->local (remote
loads) and local->peer (remote stores), one active rank at a time and all ranks together.
Rank 0 prints one JSON line per measurement.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import _lib, kvstore  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    nbytes = int(os.environ.get("PROBE_MB", "256")) << 20
    ctx = kvstore.init(heap_bytes=2 * nbytes + (8 << 20), device=dev)
    heap = ctx.heap
    a, b = heap.alloc(nbytes), heap.alloc(nbytes)
    lib = _lib.device_lib()
    peer = (rank + 1) % world
    stream = torch.cuda.current_stream()

    def run(dst, src, ctas, everyone):
        active = everyone or rank == 0
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if active:
            for _ in range(3):
                lib.psdev_copy_probe(dst, src, nbytes, ctas, stream.cuda_stream)
            e0.record()
            for _ in range(10):
                lib.psdev_copy_probe(dst, src, nbytes, ctas, stream.cuda_stream)
            e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / 10 if active else 0.0
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return nbytes / (t.item() * 1e-3) / 1e9

    me, pr = heap.bases[rank], heap.bases[peer]
    for ctas in (32, 74, 148, 296, 592):
        for name, dst, src in (("local", me + b, me + a), ("peer_read", me + b, pr + a),
                               ("peer_write", pr + b, me + a)):
            for everyone in (False, True):
                gbs = run(dst, src, ctas, everyone)
                if rank == 0:
                    print(json.dumps({"probe": name, "ctas": ctas, "all_ranks": everyone,
                                      "GBps_per_gpu": round(gbs, 1), "bytes": nbytes}), flush=True)
    kvstore.finalize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
