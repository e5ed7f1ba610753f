"""tcgen05 GEMM (alone and fused with pull) against fp32 PyTorch matmul."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(x, w):
    return (x.float() @ w.float().t())


@pytest.mark.parametrize("tile", [128, 256, 2])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 128, 192),
                                   (1000, 392, 520), (2048, 3072, 1024), (130, 264, 72),
                                   (4096, 1024, 512),
                                   # more tiles than CTA pairs with a short last round: the
                                   # pair kernel cuts that round's tiles in 4 / in 2 along N
                                   (2560, 2304, 128), (3328, 2048, 192), (2560, 2296, 128)])
def test_gemm_matches_fp32_matmul(cuda_device, M, N, K, tile):
    from ps_lite_b200 import _lib
    from ps_lite_b200.ops.gemm import gemm_status, linear_bf16
    assert _lib.device_lib().psdev_gemm_config(tile) == 0
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=cuda_device).to(torch.bfloat16)
    w = (torch.randn(N, K, device=cuda_device) / K ** 0.5).to(torch.bfloat16)
    out = linear_bf16(x, w)
    torch.cuda.synchronize()
    assert gemm_status(cuda_device) == 0
    torch.testing.assert_close(out.float(), _ref(x, w), rtol=2e-2, atol=2e-2)
    _lib.device_lib().psdev_gemm_config(0)
    _lib.device_lib().psdev_pull_ring_config(1, 0)


@pytest.mark.parametrize("tile", [128, 256, 2])
@pytest.mark.parametrize("copy_ctas", [0, -1, 16])
@pytest.mark.parametrize("world,blk", [(2, 4096), (4, 1024), (8, 4096)])
def test_pull_fused_gemm_emulated_ranks(cuda_device, world, blk, tile, copy_ctas):
    """All ranks' heaps on one GPU: rank r's kernel pulls the other ranks' blocks of W and
    multiplies; every rank must get x @ W^T and end with the complete W in its weight buffer."""
    from ps_lite_b200 import _lib
    from ps_lite_b200.ops.gemm import gemm_status, pull_linear_bf16
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    assert _lib.device_lib().psdev_gemm_config(tile) == 0
    # 0: ring of bulk loads (default); -1: ring on the load/store path; 16: copy CTAs
    assert _lib.device_lib().psdev_pull_ring_config(0 if copy_ctas < 0 else 1, 0) == 0
    torch.manual_seed(world)
    M, N, K = 512, 768, 256
    pad = 1024  # W does not start at the beginning of the table
    n = pad + N * K + 512
    heaps = SymmetricHeap.emulated(65536 + 8 * n + (1 << 20), world, device=cuda_device)
    opt = ServerOptimizer("sgd", lr=0.5)
    tables = [DenseTable(h, n, torch.bfloat16, torch.bfloat16, blk=blk, optimizer=opt)
              for h in heaps]
    w0 = torch.randn(n, device=cuda_device) * 0.05
    grads = [torch.randn(n, device=cuda_device).to(torch.bfloat16) * 0.01 for _ in range(world)]
    for t, g in zip(tables, grads):
        t.load_master(w0)
        t.grad.copy_(g)
        t.weight.fill_(float("nan"))  # anything not published or pulled would poison C
    for t in tables:
        t.push(sync=False, publish=True)
    torch.cuda.synchronize()
    w_new = w0 - 0.5 * sum(g.float() for g in grads)
    W = w_new[pad:pad + N * K].to(torch.bfloat16).view(N, K)
    x = torch.randn(M, K, device=cuda_device).to(torch.bfloat16)
    for t in tables:
        out = pull_linear_bf16(t, pad, N, x, num_copy_ctas=copy_ctas)
        torch.cuda.synchronize()
        assert gemm_status(cuda_device) == 0
        torch.testing.assert_close(out.float(), _ref(x, W), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(t.weight[pad:pad + N * K].float(), W.reshape(-1).float(),
                                   rtol=1e-2, atol=1e-2)
    _lib.device_lib().psdev_gemm_config(0)
    _lib.device_lib().psdev_pull_ring_config(1, 0)
