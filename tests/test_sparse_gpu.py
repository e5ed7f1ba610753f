"""Sparse push/pull kernels against a plain PyTorch statement of the same update."""
import pytest
import torch

from ps_lite_b200.utils.oracle import ftrl_update

pytestmark = pytest.mark.gpu


def _zipf_keys(n, key_space, gen, dev):
    u = torch.rand(4 * n, generator=gen, device=dev, dtype=torch.float64)
    k = (key_space ** u).to(torch.int64) - 1   # log-uniform: heavy head like a Zipf law
    k = torch.unique(k.clamp_(0, key_space - 1))
    k = k[torch.randperm(k.numel(), generator=gen, device=dev)[:n]]
    return torch.sort(k).values


@pytest.mark.parametrize("store", ["direct", "hash"])
@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("kind", ["sum", "sgd", "ftrl"])
def test_sparse_push_pull_matches_oracle(cuda_device, world, kind, store):
    from ps_lite_b200.parallel import SparseTable, SymmetricHeap
    key_space, n = 1 << 20, 20000
    cap = (1 << 17) if store == "hash" else 0
    nbytes = 65536 + 20 * n + 4 * ((key_space + world - 1) // world) + 12 * cap + (1 << 20)
    heaps = (SymmetricHeap.emulated(nbytes, world, device=cuda_device) if world > 1
             else [SymmetricHeap(nbytes, 0, 1, device=cuda_device)])
    tables = [SparseTable(h, key_space, n, kind=kind, lr=0.1, hash_capacity=cap) for h in heaps]
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(11)
    W = torch.zeros(key_space, device=cuda_device)
    Z, N = torch.zeros_like(W), torch.zeros_like(W)
    for step in range(3):
        reqs = []
        for t in tables:
            keys = _zipf_keys(n - 100 * step, key_space, gen, cuda_device)
            grads = torch.randn(keys.numel(), generator=gen, device=cuda_device) * 0.5
            t.stage(keys, grads)
            reqs.append((keys, grads))
        for t in tables:
            t.scatter()
        for t in tables:
            t.apply()
        for t in tables:
            t.respond()
        torch.cuda.synchronize()
        # oracle: sum the workers' gradients per key, update the touched keys once
        G = torch.zeros_like(W)
        for keys, grads in reqs:
            G.index_add_(0, keys, grads)
        touched = torch.zeros(key_space, dtype=torch.bool, device=cuda_device)
        for keys, _ in reqs:
            touched[keys] = True
        idx = touched.nonzero().squeeze(1)
        if kind == "sum":
            W[idx] += G[idx]
        elif kind == "sgd":
            W[idx] -= 0.1 * G[idx]
        else:
            z, nn, w = Z[idx], N[idx], W[idx]
            ftrl_update(z, nn, w, G[idx])
            Z[idx], N[idx], W[idx] = z, nn, w
        for t, (keys, _) in zip(tables, reqs):
            torch.testing.assert_close(t.out[: keys.numel()], W[keys], rtol=1e-4, atol=1e-5)
            pos = t.pos[: world + 2].tolist()
            assert pos[0] == 0 and pos[world] == keys.numel() and pos[world + 1] == keys.numel()
            assert torch.all(t.acc == 0)  # accumulators are clean for the next step
            t.check()


@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("var_len", [False, True])
def test_sparse_wide_and_dynamic_length_values(cuda_device, world, var_len):
    """Values of width 5, and values of per-key length 1..5 packed back to back (the
    reference's `lens`): sum handle against index_add on a dense [key_space, width] table."""
    from ps_lite_b200.parallel import SparseTable, SymmetricHeap
    key_space, n, width = 1 << 16, 3000, 5
    nbytes = 65536 + 64 * n * width + 4 * width * ((key_space + world - 1) // world) + (1 << 20)
    heaps = (SymmetricHeap.emulated(nbytes, world, device=cuda_device) if world > 1
             else [SymmetricHeap(nbytes, 0, 1, device=cuda_device)])
    tables = [SparseTable(h, key_space, n, kind="sum", width=width, var_len=var_len)
              for h in heaps]
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(5)
    dense = torch.zeros(key_space, width, device=cuda_device)
    # a key always has the same length, whoever pushes it
    key_len = torch.randint(1, width + 1, (key_space,), generator=gen, device=cuda_device)
    for step in range(3):
        reqs = []
        for t in tables:
            keys = _zipf_keys(n - 7 * step, key_space, gen, cuda_device)
            if var_len:
                lens = key_len[keys]
                vals = torch.randn(int(lens.sum().item()), generator=gen, device=cuda_device)
                t.stage(keys, vals, lens)
            else:
                lens = torch.full_like(keys, width)
                vals = torch.randn(keys.numel() * width, generator=gen, device=cuda_device)
                t.stage(keys, vals)
            reqs.append((keys, vals, lens))
        for t in tables:
            t.scatter()
        for t in tables:
            t.apply()
        for t in tables:
            t.respond()
        torch.cuda.synchronize()
        for keys, vals, lens in reqs:
            offs = torch.cumsum(lens, 0) - lens
            for j in range(width):
                m = lens > j
                dense[keys[m], j] += vals[(offs + j)[m]]
        for t, (keys, vals, lens) in zip(tables, reqs):
            offs = torch.cumsum(lens, 0) - lens
            got = t.out[: vals.numel()]
            for j in range(width):
                m = lens > j
                torch.testing.assert_close(got[(offs + j)[m]], dense[keys[m], j],
                                           rtol=1e-5, atol=1e-5)
            if var_len:
                assert torch.equal(t.offs[: keys.numel()], offs)
            t.check()


@pytest.mark.parametrize("world", [1, 4])
def test_pull_learns_lengths_from_owners(cuda_device, world):
    """A pull on a table with lengths names none: the owners store the lengths they hold into
    the requester's array, the values come back packed; a key nobody pushed has length 0."""
    import ctypes as C
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel import SparseTable, SymmetricHeap
    key_space, n, width = 1 << 14, 2000, 4
    nbytes = 65536 + 64 * n * width + 4 * width * ((key_space + world - 1) // world) + (1 << 20)
    heaps = (SymmetricHeap.emulated(nbytes, world, device=cuda_device) if world > 1
             else [SymmetricHeap(nbytes, 0, 1, device=cuda_device)])
    tables = [SparseTable(h, key_space, n, kind="sum", width=width, var_len=True) for h in heaps]
    gen = torch.Generator(device=cuda_device)
    gen.manual_seed(9)
    key_len = torch.randint(1, width + 1, (key_space,), generator=gen, device=cuda_device)
    dense = torch.zeros(key_space, width, device=cuda_device)
    pushed = torch.zeros(key_space, dtype=torch.bool, device=cuda_device)
    for t in tables:   # one push per rank (phases of all ranks run one after the other)
        keys = _zipf_keys(n, key_space, gen, cuda_device)
        keys = keys[keys % 2 == 0]          # odd keys are never pushed
        lens = key_len[keys]
        vals = torch.randn(int(lens.sum().item()), generator=gen, device=cuda_device)
        t.stage(keys, vals, lens)
        offs = torch.cumsum(lens, 0) - lens
        for j in range(width):
            m = lens > j
            dense[keys[m], j] += vals[(offs + j)[m]]
        pushed[keys] = True
    for phase in ("scatter", "apply", "respond"):
        for t in tables:
            getattr(t, phase)()
    torch.cuda.synchronize()
    asks = [_zipf_keys(n - 11 * r, key_space, gen, cuda_device) for r in range(world)]
    if world == 1:
        got, lens = tables[0].pull(asks[0])
        results = [(got.clone(), lens.clone())]
    else:
        s = torch.cuda.current_stream().cuda_stream
        for t, keys in zip(tables, asks):
            k = keys.numel()
            t.keys[:k].copy_(keys)
            t.count = k
            t.lens[:k].zero_()
            assert t.heap.lib.psdev_key_shard_lookup(t.keys.data_ptr(), k, t.range, world,
                                                     t.pos.data_ptr(), s) == 0
        for t in tables:
            assert t.heap.lib.psdev_sparse_lens(C.byref(t._world), C.byref(t._t), 0, s) == 0
        for t, keys in zip(tables, asks):
            assert t.heap.lib.psdev_lens_to_offsets(t.lens.data_ptr(), keys.numel(),
                                                    t.offs.data_ptr(), s) == 0
        for phase in ("apply", "respond"):
            for t in tables:
                getattr(t, phase)()
        torch.cuda.synchronize()
        results = [(t.out[: int(t.offs[k.numel()].item())].clone(), t.lens[: k.numel()].clone())
                   for t, k in zip(tables, asks)]
    for keys, (got, lens) in zip(asks, results):
        want_lens = torch.where(pushed[keys], key_len[keys], torch.zeros_like(keys)).int()
        assert torch.equal(lens, want_lens)
        offs = torch.cumsum(want_lens.long(), 0) - want_lens.long()
        assert got.numel() == int(want_lens.sum().item())
        for j in range(width):
            m = want_lens > j
            torch.testing.assert_close(got[(offs + j)[m]], dense[keys[m], j], rtol=1e-5, atol=1e-5)
    for t in tables:
        t.check()


def test_key_shard_lookup(cuda_device):
    from ps_lite_b200 import _lib
    lib = _lib.device_lib()
    keys = torch.tensor([0, 5, 9, 10, 11, 29, 30, 31, 45], device=cuda_device, dtype=torch.int64)
    pos = torch.zeros(6, dtype=torch.int64, device=cuda_device)
    rc = lib.psdev_key_shard_lookup(keys.data_ptr(), keys.numel(), 10, 4, pos.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    # ranges [0,10) [10,20) [20,30) [30,40); key 45 is beyond the last range
    assert pos.tolist() == [0, 3, 5, 6, 8, 9]
