"""Fused dense push/pull kernel against a plain PyTorch fp32 statement of the same update."""

import pytest
import torch

from ps_lite_b200.utils.oracle import dense_update

pytestmark = pytest.mark.gpu


def _mk_tables(world, n, gdt, odt, blk, opt, dev):
    from ps_lite_b200.parallel import DenseTable, SymmetricHeap
    nbytes = 65536 + 4 * (n + 64) * 8 + (1 << 20)
    if world == 1:
        heaps = [SymmetricHeap(nbytes, 0, 1, device=dev)]
    else:
        heaps = SymmetricHeap.emulated(nbytes, world, device=dev)
    tables = [DenseTable(h, n, gdt, odt, blk=blk, optimizer=opt) for h in heaps]
    return heaps, tables


def _tol(gdt, odt):
    if odt == torch.bfloat16:
        return dict(rtol=1e-2, atol=1e-2)
    return dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("kind", ["sum", "sgd", "momentum", "adam", "adamw"])
@pytest.mark.parametrize("gdt,odt", [(torch.float32, torch.float32),
                                     (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32),
                                     (torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("world,n,blk", [(1, 100_000, None), (4, 70_000, 1024),
                                         (8, 33_333, None), (8, 262_144 + 8, 4096)])
def test_push_pull_matches_oracle(cuda_device, kind, gdt, odt, world, n, blk):
    from ps_lite_b200.parallel import ServerOptimizer
    torch.manual_seed(1234)
    opt = ServerOptimizer(kind, lr=0.05, momentum=0.9, weight_decay=0.01, eps=1e-6,
                          scale=1.0 / world)
    heaps, tables = _mk_tables(world, n, gdt, odt, blk, opt, cuda_device)
    npad = tables[0].n
    w0 = torch.randn(npad, device=cuda_device)
    w0[n:] = 0
    for t in tables:
        t.load_master(w0)
    ref_w = w0.clone()
    s1 = torch.zeros_like(ref_w)
    s2 = torch.zeros_like(ref_w)
    for step in range(1, 4):
        grads = []
        for t in tables:
            g = torch.randn(npad, device=cuda_device).to(gdt)
            g[n:] = 0
            t.grad.copy_(g)
            grads.append(g)
        for t in tables:  # every rank's server role, one after the other
            t.push_pull(sync=False)
        torch.cuda.synchronize()
        dense_update(ref_w, grads, kind, lr=0.05, momentum=0.9, weight_decay=0.01, eps=1e-6,
                     scale=1.0 / world, step=step, s1=s1, s2=s2)
        for t in tables:
            torch.testing.assert_close(t.weight[:n].float(), ref_w[:n].to(odt).float(),
                                       **_tol(gdt, odt))
    full = torch.zeros(npad, device=cuda_device)
    for t in tables:
        t.gather_master(full)
    torch.testing.assert_close(full[:n], ref_w[:n], rtol=2e-5, atol=2e-5)
    for h in heaps:
        h.close()


@pytest.mark.parametrize("world", [1, 8])
def test_push_then_pull_and_subranges(cuda_device, world):
    """Separate Push and Pull, issued slice by slice, equal one whole-table PushPull."""
    from ps_lite_b200.parallel import ServerOptimizer
    torch.manual_seed(7)
    n = 50_000
    opt = ServerOptimizer("momentum", lr=0.1, momentum=0.9)
    heaps, tables = _mk_tables(world, n, torch.bfloat16, torch.bfloat16, 2048, opt, cuda_device)
    npad = tables[0].n
    w0 = torch.randn(npad, device=cuda_device)
    for t in tables:
        t.load_master(w0)
    ref_w, s1 = w0.clone(), torch.zeros(npad, device=cuda_device)
    grads = []
    for t in tables:
        g = torch.randn(npad, device=cuda_device).to(torch.bfloat16)
        t.grad.copy_(g)
        grads.append(g)
    cuts = [0, 8, 4096 + 16, 20_000, 20_008, npad]
    for b, e in zip(cuts[:-1], cuts[1:]):
        for t in tables:
            t.push(b, e, sync=False, opt_step=(b == 0))
    for b, e in zip(cuts[:-1], cuts[1:]):
        for t in tables:
            t.pull(b, e, sync=False)
    torch.cuda.synchronize()
    dense_update(ref_w, grads, "momentum", lr=0.1, momentum=0.9, s1=s1)
    for t in tables:
        torch.testing.assert_close(t.weight.float(), ref_w.to(torch.bfloat16).float(),
                                   rtol=1e-2, atol=1e-2)
    for h in heaps:
        h.close()


def test_entry_wait_runs_out_and_reports(cuda_device):
    """A rank whose peer never announces itself gives up after the limit and says who was late."""
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    heaps = SymmetricHeap.emulated(1 << 21, 2, device=cuda_device)
    t0 = DenseTable(heaps[0], 4096, optimizer=ServerOptimizer("sum"), channel=3)
    t0.grad.fill_(1.0)
    t0.push_pull(sync=True, timeout_s=0.2)   # rank 1 never launches: its flag is never set
    torch.cuda.synchronize()
    status, epoch = heaps[0].channel_status(3)
    assert status == -2
    assert torch.all(t0.master == 0)  # the data was not touched
    with pytest.raises(_lib.PsdevError):
        t0.check()
    heaps[0].clear_channel(3)
    assert heaps[0].channel_status(3)[0] == 0
    # the context is still usable
    t1 = DenseTable(heaps[0], 4096, optimizer=ServerOptimizer("sum"), channel=4)
    t1.grad.fill_(2.0)
    heaps[1].tensor(t1.grad_off, 4096, torch.float32).fill_(3.0)
    t1.push_pull(sync=False)
    torch.cuda.synchronize()
    assert torch.all(t1.master[:2048] == 5.0)


def test_world1_has_nobody_to_meet(cuda_device):
    """One rank: a synchronising request runs no flag round (the channel's epoch stays where it
    is); the device barrier, which is its own kernel, still counts its rounds."""
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    heap = SymmetricHeap(1 << 22, 0, 1, device=cuda_device)
    t = DenseTable(heap, 100_000, optimizer=ServerOptimizer("sum"), channel=1)
    t.grad.fill_(1.0)
    for _ in range(5):
        t.push_pull(sync=True)
    heap.barrier(channel=2)
    heap.barrier(channel=2)
    torch.cuda.synchronize()
    assert heap.channel_status(1) == (0, 0)
    assert heap.channel_status(2) == (0, 2)
    assert torch.all(t.weight[:100_000] == 5.0)
    heap.close()


@pytest.mark.parametrize("world", [1, 8])
def test_multi_slice_launch_with_device_schedule(cuda_device, world):
    """Many slices with priorities in one launch equal one whole-table push+pull."""
    from ps_lite_b200 import _lib
    from ps_lite_b200.parallel import ServerOptimizer
    torch.manual_seed(21)
    n = 300_000
    opt = ServerOptimizer("adam", lr=0.01, eps=1e-6)
    heaps, tables = _mk_tables(world, n, torch.bfloat16, torch.float32, 1024, opt, cuda_device)
    npad = tables[0].n
    w0 = torch.randn(npad, device=cuda_device)
    grads = []
    for t in tables:
        t.load_master(w0)
        g = torch.randn(npad, device=cuda_device).to(torch.bfloat16)
        t.grad.copy_(g)
        grads.append(g)
    # uneven slices, some empty of owned blocks for some ranks, shuffled priorities
    cuts = sorted(set([0, npad] + [int(x) & ~7 for x in torch.randint(0, npad, (60,)).tolist()]))
    segs = [(b, e, (i * 7) % 13) for i, (b, e) in enumerate(zip(cuts[:-1], cuts[1:]))]
    for t in tables:
        t.step = 1
        t.run_multi(_lib.OP_PUSHPULL, segs, sync=False)
    torch.cuda.synchronize()
    ref = dense_update(w0.clone(), grads, "adam", lr=0.01, eps=1e-6, step=1,
                       s1=torch.zeros_like(w0), s2=torch.zeros_like(w0))
    for t in tables:
        torch.testing.assert_close(t.weight[:n], ref[:n], rtol=2e-5, atol=2e-5)
    for h in heaps:
        h.close()


def test_shard_checkpoint_round_trip(cuda_device, tmp_path):
    """Saving a shard, training on, then loading puts the server back to the saved state."""
    from ps_lite_b200.parallel import DenseTable, ServerOptimizer, SymmetricHeap
    heap = SymmetricHeap(8 << 20, 0, 1, device=cuda_device)
    t = DenseTable(heap, 50_000, optimizer=ServerOptimizer("adam", lr=0.1), blk=1024)
    t.load_master(torch.randn(50_000, device=cuda_device))
    t.grad.copy_(torch.randn(t.n, device=cuda_device))
    t.push_pull()
    path = str(tmp_path / "shard0.pt")
    t.save(path)
    saved = (t.master.clone(), t.state1.clone(), t.state2.clone(), t.step)
    t.push_pull()
    t.push_pull()
    t.load(path)
    assert t.step == saved[3]
    for a, b in zip((t.master, t.state1, t.state2), saved[:3]):
        assert torch.equal(a, b)
    t.pull()
    torch.cuda.synchronize()
    torch.testing.assert_close(t.weight[:50_000], saved[0][:50_000])
    heap.close()


def test_cpp_device_kv_worker(cuda_device):
    """C++ DeviceKVWorker (timestamps, callbacks, Wait, error on a missing peer)."""
    import os
    import subprocess
    from ps_lite_b200 import _build
    root = str(_build.ROOT)
    lib = _build.build_device()
    core = _build.build_core()
    out = os.path.join(root, "build", "tests", "device_kv")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = [_build.NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O1",
           "-I", os.path.join(root, "include"), os.path.join(root, "tests", "cuda", "device_kv.cu"),
           "-o", out, str(lib), str(core), "-Xlinker", f"-rpath={os.path.dirname(str(lib))}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([out], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "DEVICE_KV_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("odt", [torch.float32, torch.bfloat16])
def test_int8_block_scale_gradients(cuda_device, world, odt):
    """Gradients travel as int8 + one scale per 256 values; the push kernel dequantises while
    it reduces.  The reference is the same update applied to the dequantised gradients."""
    from ps_lite_b200.ops.filters import int8_pack, int8_unpack
    from ps_lite_b200.parallel import ServerOptimizer
    torch.manual_seed(5)
    n = 100_000
    opt = ServerOptimizer("momentum", lr=0.1, momentum=0.9)
    heaps, tables = _mk_tables(world, n, torch.int8, odt, 1024, opt, cuda_device)
    npad = tables[0].n
    assert npad % 256 == 0
    w0 = torch.randn(npad, device=cuda_device)
    ref_w, s1 = w0.clone(), torch.zeros(npad, device=cuda_device)
    for t in tables:
        t.load_master(w0)
    for step in range(2):
        deq = []
        for t in tables:
            g = torch.randn(npad, device=cuda_device) * (1 + step)
            t.stage_int8(g)
            q, sc = int8_pack(g)
            deq.append(int8_unpack(q, sc))
        for t in tables:
            t.push_pull(sync=False)
        torch.cuda.synchronize()
        dense_update(ref_w, deq, "momentum", lr=0.1, momentum=0.9, s1=s1)
        for t in tables:
            torch.testing.assert_close(t.weight[:n].float(), ref_w[:n].to(odt).float(),
                                       **_tol(torch.float32, odt))
    for h in heaps:
        h.close()
