"""Large-model parity of the server-side optimizer, run as joint processes of a parameter-server
job (``python -m ps_lite_b200.launch.local --joint N python tests/mp_bert_parity.py``).

BERT-large (bf16) is trained for 10 steps through ``DistributedOptimizer`` (bf16 gradients pushed
in slices, Adam on fp32 master weights on the servers, pull), every rank on its own sequences.
On every rank a second copy of the model is trained in one process on the global batch with
``torch.optim.Adam`` on fp32 master weights -- the same update written with library calls --
and the loss of every step is compared: the job's loss (mean over ranks) against the single-process
loss, within bf16 tolerance.  Prints MP_BERT_PARITY_OK on rank 0 when every rank agreed.
"""
import copy
import os
import struct
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.models.bert import BertLarge  # noqa: E402
from ps_lite_b200.parallel import ServerOptimizer  # noqa: E402
from ps_lite_b200.parallel.optimizer import DistributedOptimizer  # noqa: E402


def main():
    steps = int(os.environ.get("PARITY_STEPS", "10"))
    per_rank, seq = int(os.environ.get("PARITY_BATCH", "2")), 128
    ctx = kvstore.init(heap_bytes=6 << 30)
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    torch.manual_seed(11)
    mine = BertLarge().to(dev).to(torch.bfloat16)
    ref = copy.deepcopy(mine)
    lr, eps = 1e-4, 1e-6
    # reference: fp32 master weights updated by torch's Adam, bf16 working copy
    master = [p.detach().float().clone().requires_grad_(True) for p in ref.parameters()]
    topt = torch.optim.Adam(master, lr=lr, eps=eps)
    dopt = DistributedOptimizer(mine.parameters(), ctx.heap,
                                ServerOptimizer("adam", lr=lr, eps=eps, scale=1.0 / world),
                                grad_dtype=torch.bfloat16, channel=ctx.new_channel())
    gen = torch.Generator(device=dev)
    ok, worst = True, 0.0
    for step in range(steps):
        gen.manual_seed(1000 + step)   # the same global batch on every rank
        ids = torch.randint(0, 30522, (world * per_rank, seq), device=dev, generator=gen)
        labels = torch.randint(0, 30522, (world * per_rank, seq), device=dev, generator=gen)
        lo, hi = rank * per_rank, (rank + 1) * per_rank
        dopt.zero_grad()
        loss = mine(ids[lo:hi], labels[lo:hi])
        loss.backward()
        dopt.step()
        torch.cuda.synchronize()
        dopt.check()
        job_loss = sum(struct.unpack("<d", b)[0]
                       for b in ctx.allgather(struct.pack("<d", float(loss.item())))) / world
        # single process, global batch
        for p in ref.parameters():
            p.grad = None
        ref_loss = ref(ids, labels)
        ref_loss.backward()
        for m, p in zip(master, ref.parameters()):
            m.grad = p.grad.float()
        topt.step()
        with torch.no_grad():
            for m, p in zip(master, ref.parameters()):
                p.copy_(m.to(torch.bfloat16))
        diff = abs(job_loss - float(ref_loss.item()))
        worst = max(worst, diff)
        if rank == 0:
            print(f"step {step}: job loss {job_loss:.4f}, single-process loss "
                  f"{float(ref_loss.item()):.4f}", flush=True)
        # bf16 forward passes of two copies whose weights agree to bf16 rounding
        if diff > 3e-2 * max(1.0, abs(float(ref_loss.item()))):
            ok = False
    # the weights themselves, after 10 steps
    num = den = 0.0
    with torch.no_grad():
        for a, b in zip(mine.parameters(), ref.parameters()):
            num += float((a.float() - b.float()).pow(2).sum())
            den += float(b.float().pow(2).sum())
    rel = (num / max(den, 1e-30)) ** 0.5
    if rel > 2e-2:
        ok = False
    all_ok = all(b == b"1" for b in ctx.allgather(b"1" if ok else b"0"))
    if rank == 0:
        print(f"worst loss difference {worst:.4f}, relative weight difference {rel:.2e}", flush=True)
        if all_ok:
            print(f"MP_BERT_PARITY_OK world={world} steps={steps}", flush=True)
    dopt.close()
    kvstore.finalize()
    sys.exit(0 if all_ok else 1)


if __name__ == "__main__":
    main()
