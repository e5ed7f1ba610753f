"""Pull fused with the consuming GEMM versus pull followed by the GEMM (run as a parameter-server job:
``python -m ps_lite_b200.launch.local --joint N python benchmarks/pull_gemm_bench.py``, or under
``torch.distributed.run``, whose environment is mapped onto such a job).

Shape: the layer-0 QKV projection of BERT-large, X[16384,1024] * W[3072,1024]^T, W sharded
block-cyclically over the ranks.  Each timed iteration is one server update of W and one use:
  unfused: push+pull of W (fused dense kernel, all-gather included), then the tcgen05 GEMM;
  fused  : push with publish, then the GEMM kernel that pulls W panel by panel itself, with the
           spare warps of its GEMM CTAs (fused) or with 16 CTAs set aside (fused_copy_ctas).
PULL_GEMM_SHAPE=M,N,K selects another shape.  CUDA events, max over ranks, one JSON line on
rank 0.
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from ps_lite_b200 import kvstore  # noqa: E402
from ps_lite_b200.ops.gemm import gemm_status, linear_bf16, pull_linear_bf16  # noqa: E402
from ps_lite_b200.parallel import DenseTable, ServerOptimizer  # noqa: E402
from ps_lite_b200.utils.timing import max_over_ranks  # noqa: E402


def main():
    M, N, K = (int(v) for v in os.environ.get("PULL_GEMM_SHAPE", "16384,3072,1024").split(","))
    ctx = kvstore.init(heap_bytes=(64 << 20) + 8 * N * K)
    rank, world, dev = ctx.rank, ctx.world, ctx.device
    t = DenseTable(ctx.heap, N * K, torch.bfloat16, torch.bfloat16, blk=4096,
                   optimizer=ServerOptimizer("sgd", lr=0.01), channel=ctx.new_channel())
    t.load_master(torch.randn(N * K, device=dev) * 0.02)
    t.grad.copy_((torch.randn(N * K, device=dev) * 0.01).to(torch.bfloat16))
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    W = t.weight.view(N, K)

    def unfused():
        t.push_pull(opt_step=False)
        linear_bf16(x, W, out)

    def fused():
        t.push(opt_step=False, publish=True)
        pull_linear_bf16(t, 0, N, x, out)

    def fused_copy_ctas():
        t.push(opt_step=False, publish=True)
        pull_linear_bf16(t, 0, N, x, out, num_copy_ctas=16)

    def gemm_only():
        linear_bf16(x, W, out)

    def push_pull_only():
        t.push_pull(opt_step=False)

    def publish_only():
        t.push(opt_step=False, publish=True)

    res = {}
    for name, fn in (("gemm_only", gemm_only), ("push_pull_only", push_pull_only),
                     ("publish_only", publish_only), ("unfused", unfused), ("fused", fused),
                     ("fused_copy_ctas", fused_copy_ctas)):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        ctx.host_barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(30):
            fn()
        e1.record()
        torch.cuda.synchronize()
        res[name] = round(max_over_ranks(e0.elapsed_time(e1), dev) / 30 * 1e3, 1)
    t.check()
    assert gemm_status(dev) == 0
    if rank == 0:
        fl = 2.0 * M * N * K
        print(json.dumps({"n_gpus": world, "shape": [M, N, K], "us": res,
                          "gemm_tflops": round(fl / res["gemm_only"] / 1e6, 1),
                          "fused_step_speedup_vs_unfused": round(res["unfused"] / res["fused"], 3),
                          "w_bytes": N * K * 2,
                          "nvlink_bytes_in_per_gpu_pull": N * K * 2 * (world - 1) // world}), flush=True)
    kvstore.finalize()


if __name__ == "__main__":
    main()
