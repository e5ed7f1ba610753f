"""Multi-GPU check of the fused dense kernel, run as one joint process per GPU under this
package's launcher (``python -m ps_lite_b200.launch.local --joint N python tests/mp_dense_check.py``);
the job is an ordinary parameter-server job: no collective library is involved.

Every rank regenerates all ranks' gradients from their seeds, so each can compute the fp32
PyTorch statement of the update locally and compare its pulled weights and owned master
values with it.  Prints "MP_DENSE_OK" on rank 0 when every rank agreed.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.parallel import ServerOptimizer  # noqa: E402
from ps_lite_b200.utils.oracle import dense_update  # noqa: E402


def main():
    ctx = kvstore.init(heap_bytes=256 << 20)
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    kv = kvstore.KVStore(ctx, slice_bytes=1 << 20)
    ok = True
    cases = [("momentum", torch.bfloat16, torch.bfloat16, 1_000_003, 4096),
             ("adam", torch.float32, torch.float32, 300_000, None),
             ("sum", torch.float32, torch.float32, 4096, 8),
             ("sgd", torch.bfloat16, torch.float32, 2_000_000, 1 << 16),
             # small enough for the low-latency exchange (values next to sequence numbers)
             ("momentum", torch.bfloat16, torch.bfloat16, 50_003, 64),
             ("adam", torch.float32, torch.bfloat16, 8, None)]
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
                kv.wait(kv.push_pull(key, grads[rank][:n]))
            else:          # separate push and pull, host-staged in slices
                hin = grads[rank][:n].cpu().pin_memory()
                hout = torch.empty(n, dtype=odt).pin_memory()
                kv.wait(kv.push(key, hin))
                kv.wait(kv.pull(key, hout))
                torch.cuda.synchronize()
                if not torch.equal(hout.to(dev), t.weight[:n]):
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
    all_ok = all(b == b"1" for b in ctx.allgather(b"1" if ok else b"0"))
    if rank == 0 and all_ok:
        print(f"MP_DENSE_OK world={world} heap={ctx.heap.backend} "
              f"multicast={bool(ctx.heap.mc_base)} nvls_used={kv.tables[0].nvls}", flush=True)
    kvstore.finalize()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
