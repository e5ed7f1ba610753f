"""Device key utilities (radix sort, ordered match) against torch.sort / plain indexing."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,bits", [(1, 64), (1000, 64), (300_001, 64), (2_000_000, 30),
                                    (5000, 12), (4096 * 3, 64), (4096 * 3 + 1, 20),
                                    (5_000_000, 64)])
def test_sort_keys(cuda_device, n, bits):
    from ps_lite_b200.ops.keys import sort_keys
    g = torch.Generator(device=cuda_device)
    g.manual_seed(n)
    hi = (1 << 62) if bits == 64 else (1 << bits)
    keys = torch.randint(0, hi, (n,), device=cuda_device, dtype=torch.int64, generator=g)
    if bits == 64:
        keys[::7] |= torch.iinfo(torch.int64).min  # top bit set: large unsigned values
    orig = keys.clone()
    out, perm = sort_keys(keys, bits, return_perm=True, check=True)
    torch.cuda.synchronize()
    # unsigned order: compare through a sign flip
    flip = orig ^ torch.iinfo(torch.int64).min
    ref_sorted, ref_idx = torch.sort(flip, stable=True)
    assert torch.equal(out ^ torch.iinfo(torch.int64).min, ref_sorted)
    assert torch.equal(perm.long(), ref_idx)


@pytest.mark.parametrize("kind", ["equal", "two_values", "skewed", "sorted", "reversed"])
def test_sort_keys_hard_distributions(cuda_device, kind):
    """Inputs that stress the ranking and the look-back: one digit everywhere, long runs, a
    skewed distribution, and already ordered keys; keys only and with the permutation."""
    from ps_lite_b200.ops.keys import sort_keys
    n = 1_000_003
    g = torch.Generator(device=cuda_device)
    g.manual_seed(3)
    if kind == "equal":
        keys = torch.full((n,), 0x1234_5678_9ABC, device=cuda_device, dtype=torch.int64)
    elif kind == "two_values":
        keys = torch.randint(0, 2, (n,), device=cuda_device, dtype=torch.int64, generator=g) << 40
    elif kind == "skewed":
        u = torch.rand(n, device=cuda_device, generator=g)
        keys = (u.pow(8) * (1 << 40)).long()
    elif kind == "sorted":
        keys = torch.arange(n, device=cuda_device, dtype=torch.int64) * 977
    else:
        keys = torch.arange(n, 0, -1, device=cuda_device, dtype=torch.int64) * 977
    ref_sorted, ref_idx = torch.sort(keys, stable=True)
    only, none = sort_keys(keys.clone(), 48, check=True)
    assert none is None and torch.equal(only, ref_sorted)
    out, perm = sort_keys(keys.clone(), 48, return_perm=True, check=True)
    assert torch.equal(out, ref_sorted) and torch.equal(perm.long(), ref_idx)


def test_sort_unique_sum_and_ordered_match(cuda_device):
    from ps_lite_b200.ops import keys as K
    g = torch.Generator(device=cuda_device)
    g.manual_seed(0)
    raw = torch.randint(0, 5000, (40000,), device=cuda_device, dtype=torch.int64, generator=g)
    vals = torch.randn(40000, device=cuda_device, generator=g)
    uk, uv = K.sort_unique_sum(raw, vals, key_bits=13)
    ref = torch.zeros(5000, device=cuda_device).index_add_(0, raw, vals)
    assert torch.equal(uk, torch.unique(raw))
    torch.testing.assert_close(uv, ref[uk], rtol=1e-4, atol=1e-4)
    # match a subset of keys into a larger table, width 2
    dst_keys = torch.arange(0, 6000, 2, device=cuda_device, dtype=torch.int64)
    dst = torch.ones(dst_keys.numel(), 2, device=cuda_device)
    src_keys = torch.arange(0, 6000, 3, device=cuda_device, dtype=torch.int64)
    src = torch.full((src_keys.numel(), 2), 2.0, device=cuda_device)
    n = K.ordered_match(src_keys, src, dst_keys, dst, op=K.PLUS, k=2)
    assert n == 1000  # multiples of 6 below 6000
    hit = (dst_keys % 3 == 0)
    assert torch.all(dst[hit] == 3.0) and torch.all(dst[~hit] == 1.0)
    di = torch.full((dst_keys.numel(),), 0b1100, device=cuda_device, dtype=torch.int32)
    si = torch.full((src_keys.numel(),), 0b1010, device=cuda_device, dtype=torch.int32)
    assert K.ordered_match(src_keys, si, dst_keys, di, op=K.XOR) == 1000
    assert torch.all(di[hit] == 0b0110) and torch.all(di[~hit] == 0b1100)


def test_filters(cuda_device):
    from ps_lite_b200.ops import filters as F
    torch.manual_seed(0)
    x = torch.randn(100_003, device=cuda_device) * 3
    b = F.cast_scale(x, torch.bfloat16, 0.5)
    torch.testing.assert_close(b.float(), (x * 0.5).to(torch.bfloat16).float())
    torch.testing.assert_close(F.cast_scale(b, torch.float32, 2.0), b.float() * 2.0)
    q, sc = F.int8_pack(x)
    pad = torch.zeros(sc.numel() * 256, device=cuda_device)
    pad[: x.numel()] = x
    ref_scale = pad.view(-1, 256).abs().amax(dim=1) / 127
    torch.testing.assert_close(sc, ref_scale)
    y = F.int8_unpack(q, sc)
    assert (y - x).abs().max() <= ref_scale.max() * 0.5 + 1e-6
    z = F.int8_unpack(q, sc, out=y.clone(), accumulate=True)
    torch.testing.assert_close(z, 2 * y)
