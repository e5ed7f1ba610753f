"""Multi-GPU check of the fused dense kernel, run as one process per GPU under torchrun.

Every rank regenerates all ranks' gradients from their seeds, so each can compute the fp32
PyTorch statement of the update locally and compare its pulled weights and owned master
values with it.  Prints "MP_DENSE_OK" on rank 0 when every rank agreed.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.parallel import ServerOptimizer  # noqa: E402
from ps_lite_b200.utils.oracle import dense_update  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    ctx = kvstore.init(heap_bytes=256 << 20, device=dev)
    kv = kvstore.KVStore(ctx, slice_bytes=1 << 20)
    ok = True
    cases = [("momentum", torch.bfloat16, torch.bfloat16, 1_000_003, 4096),
             ("adam", torch.float32, torch.float32, 300_000, None),
             ("sum", torch.float32, torch.float32, 4096, 8),
             ("sgd", torch.bfloat16, torch.float32, 2_000_000, 1 << 16)]
    for key, (kind, gdt, odt, n, blk) in enumerate(cases):
        opt = ServerOptimizer(kind, lr=0.05, momentum=0.9, eps=1e-6, scale=1.0 / world)
        g0 = torch.Generator(device=dev)
        g0.manual_seed(99)
        t = kv.declare(key, n, grad_dtype=gdt, out_dtype=odt, optimizer=opt, blk=blk)
        w0 = torch.randn(t.n, device=dev, generator=g0)
        w0[n:] = 0
        t.load_master(w0)
        ref, s1, s2 = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
        for step in range(1, 5):
            grads = []
            for r in range(world):
                g = torch.Generator(device=dev)
                g.manual_seed(1000 * step + r)
                grads.append(torch.randn(t.n, device=dev, generator=g).to(gdt))
            if step % 2:   # fused
                kv.wait(kv.push_pull(key, grads[rank]))
            else:          # separate push and pull, host-staged in slices
                hin = grads[rank].cpu().pin_memory()
                hout = torch.empty(t.n, dtype=odt).pin_memory()
                kv.wait(kv.push(key, hin))
                kv.wait(kv.pull(key, hout))
                torch.cuda.synchronize()
                if not torch.equal(hout.to(dev), t.weight):
                    ok = False
                    print(f"rank {rank}: host copy of pulled weights differs", flush=True)
            dense_update(ref, grads, kind, lr=0.05, momentum=0.9, eps=1e-6, scale=1.0 / world,
                         step=step, s1=s1, s2=s2)
            tol = dict(rtol=1e-2, atol=1e-2) if odt == torch.bfloat16 else dict(rtol=3e-5, atol=3e-5)
            if t.nvls and gdt == torch.bfloat16 and odt == torch.float32:
                # the switch returns the bf16 sum rounded to bf16 (fp32 accumulation inside)
                tol = dict(rtol=3e-3, atol=3e-3)
            try:
                torch.testing.assert_close(t.weight[:n].float(), ref[:n].to(odt).float(), **tol)
            except AssertionError as e:
                ok = False
                print(f"rank {rank} case {kind} step {step}: {str(e)[:300]}", flush=True)
    ctx.heap.barrier()
    torch.cuda.synchronize()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print(f"MP_DENSE_OK heap={ctx.heap.backend} multicast={bool(ctx.heap.mc_base)} "
              f"nvls_used={kv.tables[0].nvls}", flush=True)
    kvstore.finalize()
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 1 else 1)


if __name__ == "__main__":
    main()
