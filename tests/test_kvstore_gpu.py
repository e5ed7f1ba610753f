"""The public path on a GPU: ``kvstore.init`` = ``ps::Start`` + device plane, ``KVStore`` requests
= ``KVWorker::ZPush/ZPull/ZPushPull`` on a registered tensor, completion through the worker's
request tracker.  One process (the loop van); the multi-process form is tests/test_multi_gpu.py.
Each test body runs in a child process: the host runtime is a process-wide singleton."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(body, env=None, timeout=300):
    code = "import sys; sys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body)
    e = dict(os.environ)
    e.pop("DMLC_ROLE", None)
    e.update(env or {})
    return subprocess.run([sys.executable, "-c", code], capture_output=True, text=True,
                          timeout=timeout, env=e)


@pytest.mark.parametrize("heap", ["ipc", "vmm"])
def test_push_pull_device_and_host_tensors(cuda_device, heap):
    r = _run("""
        import torch
        from ps_lite_b200 import kvstore, host
        from ps_lite_b200.parallel import ServerOptimizer
        from ps_lite_b200.utils.oracle import dense_update
        ctx = kvstore.init(heap_bytes=128 << 20)
        assert ctx.world == 1 and ctx.heap.backend == "%s", ctx.heap.backend
        dev = ctx.device
        kv = kvstore.KVStore(ctx, slice_bytes=1 << 20)
        n = 3_000_003
        for key, (kind, gdt, odt) in enumerate([("momentum", torch.bfloat16, torch.bfloat16),
                                                ("adam", torch.float32, torch.float32)]):
            opt = ServerOptimizer(kind, lr=0.05, momentum=0.9, eps=1e-6)
            t = kv.declare(key, n, grad_dtype=gdt, out_dtype=odt, optimizer=opt)
            keys = kv.keys_of(key)
            assert keys.size == 1 and int(keys[0]) == key
            w0 = torch.randn(t.n, device=dev); w0[n:] = 0
            t.load_master(w0)
            ref, s1, s2 = w0.clone(), torch.zeros_like(w0), torch.zeros_like(w0)
            last = -1
            for step in range(1, 5):
                g = torch.randn(t.n, device=dev).to(gdt); g[n:] = 0
                if step == 1:       # device tensors, one fused pass
                    out = torch.empty(n, device=dev, dtype=odt)
                    ts = kv.push_pull(key, g[:n].contiguous(), out)
                elif step == 2:     # pinned host tensors, sliced pipeline
                    hin = g[:n].cpu().pin_memory(); hout = torch.empty(n, dtype=odt).pin_memory()
                    ts = kv.push_pull(key, hin, hout)
                elif step == 3:     # separate push and pull
                    kv.wait(kv.push(key, g[:n].contiguous()))
                    hout = torch.empty(n, dtype=odt).pin_memory()
                    ts = kv.pull(key, hout)
                else:               # values already in the arena: zero copy
                    t.grad.copy_(g)
                    ts = kv.push_pull(key)
                assert ts > last; last = ts
                kv.wait(ts)
                torch.cuda.synchronize()
                dense_update(ref, [g], kind, lr=0.05, momentum=0.9, eps=1e-6, step=step,
                             s1=s1, s2=s2)
                tol = dict(rtol=1e-2, atol=1e-2) if odt == torch.bfloat16 else dict(rtol=3e-5, atol=3e-5)
                torch.testing.assert_close(t.weight[:n].float(), ref[:n].to(odt).float(), **tol)
                if step == 1:
                    torch.testing.assert_close(out, t.weight[:n])
                if step in (2, 3):
                    torch.testing.assert_close(hout.to(dev), t.weight[:n])
        assert host.lib().psnvl_launches() > 0
        kvstore.finalize()
        print("KVSTORE_OK")
    """ % heap, env={"PSB200_HEAP": heap})
    assert r.returncode == 0 and "KVSTORE_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_channels_run_out_with_an_error(cuda_device):
    r = _run("""
        import torch
        from ps_lite_b200 import kvstore, host
        ctx = kvstore.init(heap_bytes=64 << 20)
        kv = kvstore.KVStore(ctx)
        try:
            for key in range(80):
                kv.declare(key, 64)
            print("NO_ERROR")
        except host.PSError as e:
            assert "channels" in str(e), str(e)
            print("RAN_OUT_AT", key)
        kvstore.finalize()
    """)
    assert r.returncode == 0 and "RAN_OUT_AT 63" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


def test_cpp_program_through_ps_start(cuda_device):
    """tests/cpp/device_plane.cc built for a real device: Start -> Push/Pull/PushPull on a
    registered tensor -> Wait -> Finalize, values staged from pageable host memory."""
    from ps_lite_b200 import _build
    _build.build_device()
    core = str(_build.build_core())
    libdir = os.path.dirname(core)
    out = os.path.join(ROOT, "build", "tests", "device_plane_gpu")
    os.makedirs(os.path.dirname(out), exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-DPLANE_DEVICE=0", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "device_plane.cc"), "-o", out, "-L", libdir,
           "-lpsb200_core", f"-Wl,-rpath,{libdir}", "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    env = dict(os.environ, DMLC_PS_VAN_TYPE="loop")
    env.pop("DMLC_ROLE", None)
    r = subprocess.run([out], capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0 and "DEVICE_PLANE_OK rank 0 of 1" in r.stderr, r.stderr[-3000:]


def test_keyed_store_through_kvworker(cuda_device):
    """Keyed tables from Python through KVWorker requests with device-resident keys: fixed
    width with the SGD handle, and per-key lengths with the sum handle (a pull returns the
    lengths that the owner holds)."""
    r = _run("""
        import torch
        from ps_lite_b200 import kvstore
        ctx = kvstore.init(heap_bytes=256 << 20)
        dev = ctx.device
        g = torch.Generator(device=dev); g.manual_seed(1)
        # fixed width 4, SGD lr 0.5 on values that start at 0
        ks = kvstore.KeyedStore(ctx, 7, 1 << 20, 5000, width=4, kind="sgd", lr=0.5)
        keys = torch.unique(torch.randint(0, 1 << 20, (4000,), device=dev, generator=g))
        vals = torch.randn(keys.numel() * 4, device=dev, generator=g)
        out = torch.empty_like(vals)
        ks.wait(ks.push_pull(keys, vals, out))
        torch.testing.assert_close(out, -0.5 * vals)
        ks.wait(ks.push(keys, vals))
        sub = keys[::3].contiguous()
        out2 = torch.empty(sub.numel() * 4, device=dev)
        ks.wait(ks.pull(sub, out2))
        torch.testing.assert_close(out2.view(-1, 4), (-1.0 * vals).view(-1, 4)[::3])
        # per-key lengths 1..3, sum handle
        kv = kvstore.KeyedStore(ctx, 8, 1 << 16, 3000, width=3, kind="sum", var_len=True)
        keys = torch.unique(torch.randint(0, 1 << 16, (2500,), device=dev, generator=g))
        lens = (keys % 3 + 1).int()
        total = int(lens.sum())
        vals = torch.randn(total, device=dev, generator=g)
        kv.wait(kv.push(keys, vals, lens))
        ask = torch.unique(torch.cat([keys[::2], torch.tensor([1, 5, 9], device=dev)]))
        out = torch.zeros(ask.numel() * 3, device=dev)
        lens_back = torch.full((ask.numel(),), -1, device=dev, dtype=torch.int32)
        kv.wait(kv.pull(ask, out, lens_back))
        known = torch.isin(ask, keys)
        want_lens = torch.where(known, (ask % 3 + 1).int(), torch.zeros_like(lens_back))
        assert torch.equal(lens_back, want_lens), (lens_back[:10], want_lens[:10])
        offs = torch.cumsum(lens.long(), 0) - lens.long()
        pos = torch.searchsorted(keys, ask[known])
        got_offs = (torch.cumsum(want_lens.long(), 0) - want_lens.long())[known]
        for j in range(3):
            m = lens[pos] > j
            torch.testing.assert_close(out[(got_offs + j)[m]], vals[(offs[pos] + j)[m]])
        kvstore.finalize()
        print("KEYED_OK")
    """)
    assert r.returncode == 0 and "KEYED_OK" in r.stdout, (r.stdout + r.stderr)[-4000:]
