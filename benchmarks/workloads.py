"""Model workloads of bench.py: data-parallel ResNet-50 and BERT-large through the
server-side optimizer (synthetic data, random-init weights)."""
from __future__ import annotations

import json
import os

import torch
import torch.nn.functional as F


def _setup(args):
    """Rank, world and device as the launcher gives them; only the library baseline (DDP over
    NCCL) starts ``torch.distributed``."""
    world = int(os.environ.get("WORLD_SIZE", os.environ.get("DMLC_NUM_WORKER", "1")))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", os.environ.get("PSB200_LOCAL_INDEX", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1 and getattr(args, "trainer", "ps") == "ddp":
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def _build(workload, batch, world, dev):
    """Model, server-side optimizer, batch factory and forward function of a workload."""
    from ps_lite_b200.parallel import ServerOptimizer
    if workload == "resnet50":
        from ps_lite_b200.models.resnet import ResNet50
        batch = batch or 256
        model = ResNet50().to(dev).to(memory_format=torch.channels_last)
        sopt = ServerOptimizer("momentum", lr=0.01, momentum=0.9, scale=1.0 / world)
        make = lambda: (torch.randn(batch, 3, 224, 224).pin_memory(),
                        torch.randint(0, 1000, (batch,)).pin_memory())
        unit, metric = "img/s", "resnet50_train_img_per_s"

        def fwd(net, x, y):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                out = net(x.contiguous(memory_format=torch.channels_last))
            return F.cross_entropy(out.float(), y)
    else:
        from ps_lite_b200.models.bert import BertLarge
        batch, seq = batch or 32, 512
        model = BertLarge().to(dev).to(torch.bfloat16)
        sopt = ServerOptimizer("adam", lr=1e-4, eps=1e-6, scale=1.0 / world)
        make = lambda: (torch.randint(0, 30522, (batch, seq)).pin_memory(),
                        torch.randint(0, 30522, (batch, seq)).pin_memory())
        unit, metric = "seq/s", "bert_large_train_seq_per_s"

        def fwd(net, x, y):
            return net(x, y)
    return model, sopt, make, fwd, unit, metric, batch


def measure_ps(ctx, workload, steps, warmup, batch=0, ctas=0, sample_clocks=False):
    """Trains `workload` for `warmup` + `steps` steps through the server-side optimizer of an
    existing context; returns the record (a dict) on every rank.  One step = pinned-host batch
    copied in, forward, backward with gradient slices pushed as they appear, pull, loss read
    back."""
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel.optimizer import DistributedOptimizer
    from ps_lite_b200.utils.timing import ClockSampler
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    torch.manual_seed(0)
    torch.backends.cudnn.benchmark = True
    model, sopt, make, fwd, unit, metric, per_step = _build(workload, batch, world, dev)
    nparam = sum(p.numel() for p in model.parameters())
    # the pull of the first GEMM's weight is fused into that GEMM when the weight is large
    # enough for the fusion to pay (ops.gemm.fusion_pays; BERT-large's 6 MiB QKV weight is not)
    from ps_lite_b200.ops.gemm import fusion_pays
    fused = (workload == "bert" and
             fusion_pays(model.layers[0].qkv.weight.numel() * 2, world))
    dopt = DistributedOptimizer(model.parameters(), ctx.heap, sopt, grad_dtype=torch.bfloat16,
                                num_ctas=ctas or 32, channel=ctx.new_channel(),
                                publish_params=[model.layers[0].qkv.weight] if fused else ())
    if fused:
        # the first GEMM that consumes pulled weights (layer-0 QKV) pulls them itself
        from ps_lite_b200.ops.gemm import pull_linear
        qkv_w = model.layers[0].qkv.weight
        off = dopt.offset_of(qkv_w)
        model.layers[0].qkv_fn = lambda x: pull_linear(x, qkv_w, dopt.table, off)
    hx, hy = make()
    lib = _lib.device_lib()

    def step():
        x = hx.to(dev, non_blocking=True)   # host -> device copy of this step's inputs
        y = hy.to(dev, non_blocking=True)
        dopt.zero_grad()
        loss = fwd(model, x, y)
        loss.backward()
        dopt.step()
        return loss

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    ctx.host_barrier()
    sampler = ClockSampler(dev.index) if sample_clocks else None
    if sampler:
        sampler.start()
    l0 = lib.psdev_launch_count()
    slices0, launches0 = dopt.launched_slices, dopt.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    losses = []
    for _ in range(steps):
        losses.append(float(step().item()))   # device -> host read of the step's loss
    e1.record()
    torch.cuda.synchronize()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / steps
    clocks = sampler.stop() if sampler else None
    dopt.check()
    value = world * per_step / (ms * 1e-3)
    rec = {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(ms, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "impl": "ours",
        "config": {"model": workload, "global_batch": per_step * world,
                   "parameters": nparam, "parallelism": f"dp{world}, server-side optimizer",
                   "slices_per_step": (dopt.launched_slices - slices0) // max(1, steps),
                   "exchange_launches_per_step": (dopt.launches - launches0) // max(1, steps),
                   "batch_bytes": dopt.batch_bytes,
                   "pull_fused_with_first_gemm": bool(fused),
                   "timing": "end to end: pinned-host inputs copied in and loss read back "
                             "every step"},
        "loss_first_last": [losses[0], losses[-1]], "clocks": clocks,
        "gpu_launches": int(lib.psdev_launch_count() - l0)}
    dopt.close()
    del model, dopt
    torch.cuda.empty_cache()
    return rec


def run(args):
    from ps_lite_b200 import kvstore
    rank, world, dev = _setup(args)
    if getattr(args, "trainer", "ps") == "ddp":
        model, _sopt, make, fwd, unit, metric, per_step = _build(args.workload, args.batch,
                                                                 world, dev)
        nparam = sum(p.numel() for p in model.parameters())
        torch.manual_seed(0)
        torch.backends.cudnn.benchmark = True
        return _run_ddp(args, model, fwd, make, rank, world, dev, metric, unit, per_step, nparam)
    nparam_bound = 400_000_000 if args.workload == "bert" else 30_000_000
    ctx = kvstore.init(heap_bytes=nparam_bound * 8 + (256 << 20), device=dev)
    rec = measure_ps(ctx, args.workload, args.steps, args.warmup, args.batch, args.ctas,
                     sample_clocks=ctx.rank == 0)
    if ctx.rank == 0:
        print(json.dumps(rec), flush=True)
    kvstore.finalize()


def _run_ddp(args, model, fwd, make, rank, world, dev, metric, unit, per_step, nparam):
    """Library baseline: DistributedDataParallel (NCCL all-reduce in buckets, overlapped with
    backward) and the fused torch optimizers, same model, data path and timing."""
    import torch.distributed as dist
    from ps_lite_b200.utils.timing import max_over_ranks
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[dev.index],
                                                        gradient_as_bucket_view=True)
    if args.workload == "resnet50":
        opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    else:
        opt = torch.optim.Adam(model.parameters(), lr=1e-4, eps=1e-6, fused=True)
    hx, hy = make()
    # (the forward goes through the DDP wrapper so that its hooks fire)

    def step():
        x = hx.to(dev, non_blocking=True)
        y = hy.to(dev, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        loss = fwd(net, x, y)
        loss.backward()
        opt.step()
        return loss

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        float(step().item())
    e1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    if rank == 0:
        print(json.dumps({"metric": metric, "value": round(world * per_step / (ms * 1e-3), 2),
                          "unit": unit, "n_gpus": world, "steps": args.steps,
                          "ms_per_step": round(ms, 3), "impl": "torch DDP + torch.optim (NCCL)",
                          "dtype": "bf16", "data": "synthetic",
                          "config": {"model": args.workload, "global_batch": per_step * world,
                                     "parameters": nparam}}), flush=True)
    if world > 1:
        dist.destroy_process_group()
