"""Python binding of the host runtime, wire codec against google.protobuf, launchers."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _pb_classes():
    """PBMeta built from the field list of the wire contract (no protoc needed)."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory
    fd = descriptor_pb2.FileDescriptorProto(name="meta.proto", package="ps", syntax="proto2")
    T = descriptor_pb2.FieldDescriptorProto
    O, Q, R = T.LABEL_OPTIONAL, T.LABEL_REQUIRED, T.LABEL_REPEATED

    def msg(name, fields):
        m = fd.message_type.add(name=name)
        for n, num, typ, label, tn, packed in fields:
            f = m.field.add(name=n, number=num, type=typ, label=label)
            if tn:
                f.type_name = tn
            if packed:
                f.options.packed = True
    I, B, S, Y, U, M = T.TYPE_INT32, T.TYPE_BOOL, T.TYPE_STRING, T.TYPE_BYTES, T.TYPE_UINT64, T.TYPE_MESSAGE
    msg("PBNode", [("role", 1, I, Q, None, 0), ("id", 2, I, O, None, 0), ("hostname", 3, S, O, None, 0),
                   ("port", 4, I, O, None, 0), ("is_recovery", 5, B, O, None, 0),
                   ("customer_id", 10, I, O, None, 0)])
    msg("PBControl", [("cmd", 1, I, Q, None, 0), ("node", 2, M, R, ".ps.PBNode", 0),
                      ("barrier_group", 3, I, O, None, 0), ("msg_sig", 4, U, O, None, 0)])
    msg("PBMeta", [("head", 1, I, O, None, 0), ("body", 2, Y, O, None, 0),
                   ("control", 3, M, O, ".ps.PBControl", 0), ("request", 4, B, O, None, 0),
                   ("push", 5, B, O, None, 0), ("simple_app", 6, B, O, None, 0),
                   ("app_id", 7, I, O, None, 0), ("timestamp", 8, I, O, None, 0),
                   ("data_type", 9, I, R, None, 1), ("customer_id", 10, I, O, None, 0),
                   ("data_size", 11, I, O, None, 0), ("pull", 12, B, O, None, 0),
                   ("priority", 13, I, O, None, 0)])
    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    return message_factory.GetMessageClass(pool.FindMessageTypeByName("ps.PBMeta"))


def test_codec_bytes_equal_protobuf():
    from ps_lite_b200 import host
    PBMeta = _pb_classes()
    rng = np.random.default_rng(0)
    EMPTY = 2**31 - 1
    for trial in range(200):
        head = int(rng.integers(-5, 1000)) if trial % 3 else EMPTY
        app = int(rng.integers(0, 50)) if trial % 2 else EMPTY
        ts = int(rng.integers(0, 10**6)) if trial % 5 else EMPTY
        cust = int(rng.integers(0, 4))
        prio = int(rng.integers(-3, 100))
        flags = [bool(x) for x in rng.integers(0, 2, 4)]
        dts = [int(x) for x in rng.integers(0, 12, int(rng.integers(0, 4)))]
        body = bytes(rng.integers(0, 256, int(rng.integers(0, 30)), dtype=np.uint8))
        kind = trial % 4  # 0 data, 1 add_node, 2 barrier, 3 ack
        ref = PBMeta(head=head, request=flags[0], push=flags[1], simple_app=flags[3],
                     customer_id=cust, pull=flags[2], priority=prio)
        if app != EMPTY:
            ref.app_id = app
        if ts != EMPTY:
            ref.timestamp = ts
        if body:
            ref.body = body
        ref.data_type.extend(dts)
        kw = dict(head=head, app_id=app, timestamp=ts, customer_id=cust, priority=prio,
                  request=flags[0], push=flags[1], pull=flags[2], simple_app=flags[3],
                  data_types=dts, body=body)
        if kind == 1:
            nodes = [dict(role=int(rng.integers(0, 3)), id=int(rng.integers(8, 40)),
                          hostname=f"10.0.0.{i}", port=int(rng.integers(1000, 60000)),
                          is_recovery=bool(i % 2), customer_id=i) for i in range(int(rng.integers(1, 5)))]
            ref.control.cmd = 2
            for n in nodes:
                ref.control.node.add(role=n["role"], id=n["id"], hostname=n["hostname"],
                                     port=n["port"], is_recovery=n["is_recovery"],
                                     customer_id=n["customer_id"])
            kw.update(control_cmd=2, nodes=nodes)
        elif kind == 2:
            ref.control.cmd = 3
            ref.control.barrier_group = 7
            kw.update(control_cmd=3, barrier_group=7)
        elif kind == 3:
            sig = int(rng.integers(0, 2**63))
            ref.control.cmd = 4
            ref.control.msg_sig = sig
            kw.update(control_cmd=4, msg_sig=sig)
        mine = host.encode_meta(**kw)
        assert mine == ref.SerializeToString(), (trial, mine.hex(), ref.SerializeToString().hex())
        # and what protobuf writes is read back identically
        back = host.decode_meta(ref.SerializeToString())
        assert (back.head, back.customer_id, back.priority) == (head, cust, prio)
        assert back.app_id == app and back.timestamp == ts
        assert [back.data_types[i] for i in range(back.num_data_types)] == dts
        raw = bytes(memoryview(back).cast('B'))[host.MetaStruct.body.offset:][:back.body_len]
        assert raw == body


def test_decode_rejects_garbage():
    from ps_lite_b200 import host
    with pytest.raises(host.PSError):
        host.decode_meta(b"\x0a\xff\xff\xff")  # length runs past the end


WORKER_SCRIPT = r'''
import os, sys
import numpy as np
sys.path.insert(0, os.environ["PSB_ROOT"])
from ps_lite_b200 import host
host.start(0)
server = None
calls = []
if host.is_server():
    store = {}
    def handle(srv, req):
        # user-defined server-side update written in Python: w -= 0.5 * g
        out = []
        for i, k in enumerate(req["keys"]):
            if req["push"]:
                store[int(k)] = store.get(int(k), 0.0) - 0.5 * float(req["vals"][i])
            out.append(store.get(int(k), 0.0))
        if req["pull"]:
            srv.respond(req, req["keys"], np.array(out, np.float32))
        else:
            srv.respond(req)
    server = host.KVServer(0, handle if os.environ.get("PSB_PY_HANDLE") == "1" else None)
if host.is_worker():
    kv = host.KVWorker(0, 0)
    n = 1000
    keys = (np.arange(n, dtype=np.uint64) * np.uint64((2**64 - 1) // n)) + np.uint64(3)
    vals = np.arange(n, dtype=np.float32)
    for _ in range(4):
        kv.wait(kv.push(keys, vals))
    host.barrier(host.WORKER_GROUP)
    out = np.zeros(n, np.float32)
    kv.wait(kv.pull(keys, out))
    scale = 4 * host.num_workers() * (-0.5 if os.environ.get("PSB_PY_HANDLE") == "1" else 1.0)
    assert np.allclose(out, scale * vals), (out[:5], vals[:5])
    out2 = np.zeros(n, np.float32)
    kv.wait(kv.push_pull(keys, vals, out2))
    lo, hi = host.server_key_range(0)
    assert lo == 0 and hi > 0
    sent, recv = host.traffic()
    assert sent > n * 12 and recv > 0
    print("PY_WORKER_OK", host.my_rank(), flush=True)
    kv.close()
host.finalize(0)
if server: server.close()
'''


@pytest.mark.parametrize("py_handle", ["0", "1"], ids=["default-handle", "python-handle"])
@pytest.mark.parametrize("layout", [dict(num_workers=2, num_servers=2), dict(num_joint=2)],
                         ids=["separate", "joint"])
def test_python_binding_push_pull(tmp_path, py_handle, layout):
    from ps_lite_b200.launch.local import LocalJob
    script = tmp_path / "node.py"
    script.write_text(WORKER_SCRIPT)
    job = LocalJob([sys.executable, str(script)], env={"PSB_ROOT": ROOT, "PSB_PY_HANDLE": py_handle},
                   capture=True, **layout)
    job.start()
    rc = job.wait(120)
    out = job.output()
    assert rc == 0 and out.count("PY_WORKER_OK") == 2, out[-3000:]


def test_launcher_command_lines(tmp_path):
    from ps_lite_b200.launch import mpi, ssh, tracker
    hf = tmp_path / "hosts"
    hf.write_text("nodeA\nnodeB:2222\n")
    hosts = ssh.read_hosts(str(hf))
    assert hosts == [("nodeA", "22"), ("nodeB", "2222")]
    envs = {"DMLC_NUM_WORKER": "2", "DMLC_NUM_SERVER": "1", "DMLC_PS_ROOT_URI": "10.0.0.1",
            "DMLC_PS_ROOT_PORT": "9100"}
    cmds = ssh.build_commands(hosts, 2, 1, envs, ["./prog", "a b"], "/work")
    assert len(cmds) == 3 and "export DMLC_ROLE=server;" in cmds[0][-1]
    assert "export DMLC_ROLE=worker;" in cmds[2][-1] and cmds[1][3] == "nodeB"
    m = mpi.mpirun_commands(2, 1, envs, ["./prog"], flavor="mpich")
    assert m[0][:3] == ["mpirun", "-n", "1"] and "-env" in m[0]
    port = tracker.free_port()
    assert 1024 < port < 65536


def test_keepalive_restarts_on_exit_code_254(tmp_path):
    """A process that exits with 254 is started again with DMLC_NUM_ATTEMPT incremented."""
    from ps_lite_b200.launch.local import LocalJob
    marker = tmp_path / "attempts"
    script = tmp_path / "flaky.py"
    script.write_text(
        "import os, sys\n"
        f"open(r'{marker}', 'a').write(os.environ['DMLC_ROLE'] + os.environ['DMLC_NUM_ATTEMPT'] + '\\n')\n"
        "sys.exit(254 if os.environ['DMLC_ROLE'] == 'worker' and os.environ['DMLC_NUM_ATTEMPT'] == '0' else 0)\n")
    job = LocalJob([sys.executable, str(script)], num_workers=1, num_servers=1)
    job.start()
    assert job.wait(30) == 0
    lines = marker.read_text().split()
    assert "worker0" in lines and "worker1" in lines and "server1" not in lines


def test_repeat_stops_at_the_first_failure(tmp_path):
    """--repeat runs the job again and again (a race shaker) and stops when a run fails."""
    from ps_lite_b200.launch import local
    marker = tmp_path / "runs"
    script = tmp_path / "third_time_unlucky.py"
    script.write_text(
        "import os, sys\n"
        "if os.environ['DMLC_ROLE'] != 'worker':\n"
        "    sys.exit(0)\n"
        f"with open(r'{marker}', 'a') as f:\n"
        "    f.write('x')\n"
        f"sys.exit(3 if len(open(r'{marker}').read()) == 3 else 0)\n")
    rc = local.main(["--repeat", "10", "-n", "1", "-s", "1", sys.executable, str(script)])
    assert rc == 3 and marker.read_text() == "xxx"


def test_core_library_then_torch_in_one_process():
    """The host runtime library must not bring a second C++ runtime into the process: loading
    it first and importing torch afterwards used to crash where the compiler links libstdc++
    statically by default."""
    import subprocess
    code = ("from ps_lite_b200 import host\n"
            "host.lib(); host.shm_stats()\n"
            "import torch\n"
            "print('LOADED', torch.__version__)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300,
                       cwd=ROOT)
    assert r.returncode == 0 and "LOADED" in r.stdout, (r.stdout + r.stderr)[-2000:]


def test_p3_scheduler_order():
    from ps_lite_b200.parallel.optimizer import P3Scheduler
    s = P3Scheduler(slice_elems=16)
    assert s.add(0, 40, priority=1) == 3       # [0,16) [16,32) [32,40)
    assert s.add(100, 116, priority=5) == 1
    assert s.add(200, 232, priority=1) == 2
    got = []
    while len(s):
        got.append(s.pop())
    assert got == [(100, 116, 5), (0, 16, 1), (16, 32, 1), (32, 40, 1), (200, 216, 1),
                   (216, 232, 1)]


def test_lint_is_clean():
    """tests/lint.py (style and hygiene rules for C++/CUDA and Python sources) reports nothing."""
    r = __import__("subprocess").run([sys.executable, os.path.join(ROOT, "tests", "lint.py")],
                                     capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:]


PLANE_SCRIPT = r'''
import ctypes as C, os, sys
import numpy as np
sys.path.insert(0, os.environ["PSB_ROOT"])
from ps_lite_b200 import _lib, host
host.start(0)
if host.is_scheduler() and not host.is_worker():
    host.finalize(0)          # the scheduler takes part in start-up and shut-down only
    sys.exit(0)
L = host.lib()
# the device plane on its CPU stand-in (device = -1): arenas in shared memory, host loops
host._ck(L.psnvl_start(32 << 20, -1, b"auto", 0, b"", 1 << 18, 5_000_000_000))
R, W = L.psnvl_rank(), L.psnvl_world()
assert L.psnvl_backend().decode() == "sim" if hasattr(L, "psnvl_backend") else True
n = 100_003
n_pad = (n + 7) & ~7
blk = ((n_pad + W - 1) // W + 7) & ~7
local_len = ((n_pad + blk - 1) // blk + W - 1) // W * blk
master = np.zeros(local_len, np.float32)
t = _lib.Table()
t.grad_off = host._ck(L.psnvl_alloc(4 * n_pad, 256))
t.weight_off = host._ck(L.psnvl_alloc(4 * n_pad, 256))
t.n, t.blk = n_pad, blk
t.master = master.ctypes.data
t.grad_dtype = t.out_dtype = _lib.F32
o = _lib.Opt()
o.kind, o.scale, o.lr = _lib.OPT_SGD, 1.0, 0.5
ch = host._ck(L.psnvl_new_channel())
host._ck(L.psnvl_register_dense(0, 5, n, C.byref(t), C.byref(o), ch, 0, 0))
keys = np.zeros(W, np.uint64)
host._ck(L.psnvl_dense_keys(5, keys.ctypes.data_as(C.POINTER(C.c_uint64))))
assert np.all(np.diff(keys.astype(np.float64)) > 0)          # one key per shard, ascending
worker = L.ps_capi_bworker_new(0, 0)
assert worker
vals = np.full(n, float(R + 1), np.float32)
outs = np.zeros(n, np.float32)
kp = keys.ctypes.data_as(C.POINTER(C.c_uint64))
for step in range(1, 4):
    ts = L.ps_capi_bworker_request(worker, 1, 1, kp, W, vals.ctypes.data, 4 * n, outs.ctypes.data,
                                   4 * n, 0, 0)
    assert ts >= 0, L.ps_capi_last_error()
    host._ck(L.ps_capi_bworker_wait(worker, ts))
    want = -0.5 * step * W * (W + 1) / 2
    assert np.allclose(outs, want), (step, outs[:4], want)
# push only, then pull only
ts = L.ps_capi_bworker_request(worker, 1, 0, kp, W, vals.ctypes.data, 4 * n, None, 0, 0, 0)
host._ck(L.ps_capi_bworker_wait(worker, ts))
outs[:] = 0
ts = L.ps_capi_bworker_request(worker, 0, 1, kp, W, None, 0, outs.ctypes.data, 4 * n, 0, 0)
host._ck(L.ps_capi_bworker_wait(worker, ts))
assert np.allclose(outs, -0.5 * 4 * W * (W + 1) / 2)
# all-gather and barrier over the control plane
sizes = (C.c_size_t * W)()
buf = C.create_string_buffer(64 * W)
mine = ("rank%d" % R).encode()
total = L.psnvl_allgather(mine, len(mine), buf, len(buf), sizes)
assert total == sum(len("rank%d" % r) for r in range(W))
assert buf.raw[:total] == b"".join(("rank%d" % r).encode() for r in range(W))
host._ck(L.psnvl_barrier())
assert L.psnvl_launches() > 0
host._ck(L.psnvl_drain())
host._ck(L.ps_capi_bworker_delete(worker))
host._ck(L.psnvl_unregister_dense(0, 5))
host._ck(L.psnvl_stop())
print("PY_PLANE_OK", R, flush=True)
host.finalize(0)
'''


@pytest.mark.parametrize("nproc", [1, 3])
def test_device_plane_c_abi_on_the_cpu_stand_in(tmp_path, nproc):
    """The C ABI of the device plane (what the Python package calls) without a GPU: start,
    allocation, tensor registration, KVWorker requests on host arrays served by the plane's CPU
    stand-in, all-gather and barrier over the control plane, drain, stop."""
    from ps_lite_b200.launch.local import LocalJob
    script = tmp_path / "plane_node.py"
    script.write_text(PLANE_SCRIPT)
    if nproc == 1:
        env = dict(os.environ, PSB_ROOT=ROOT, DMLC_PS_VAN_TYPE="loop")
        env.pop("DMLC_ROLE", None)
        r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True,
                           timeout=120, env=env)
        assert r.returncode == 0 and "PY_PLANE_OK 0" in r.stdout, (r.stdout + r.stderr)[-3000:]
        return
    job = LocalJob([sys.executable, str(script)], env={"PSB_ROOT": ROOT, "DMLC_LOCAL": "1"},
                   capture=True, num_joint=nproc)
    job.start()
    rc = job.wait(120)
    out = job.output()
    assert rc == 0 and out.count("PY_PLANE_OK") == nproc, out[-3000:]


def test_exit_without_finalize_ends_with_the_programs_status():
    """A process that started the runtime and dies of an exception leaves with status 1 at once
    (it neither blocks in the destruction of the runtime nor aborts)."""
    code = ("import sys; sys.path.insert(0, %r)\n"
            "from ps_lite_b200 import host\n"
            "host.start(0)\n"
            "raise RuntimeError('user error after start')\n" % ROOT)
    env = dict(os.environ, DMLC_PS_VAN_TYPE="loop")
    env.pop("DMLC_ROLE", None)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60,
                       env=env)
    assert r.returncode == 1 and "user error after start" in r.stderr, r.stderr[-2000:]


def test_job_ends_when_a_node_dies_of_an_exception(tmp_path):
    """One node of a job raises after start-up: it leaves with status 1, and the launcher ends
    the others instead of letting them wait for it."""
    from ps_lite_b200.launch.local import LocalJob
    script = tmp_path / "failnode.py"
    script.write_text(
        "import os, sys\n"
        "sys.path.insert(0, os.environ['PSB_ROOT'])\n"
        "from ps_lite_b200 import host\n"
        "host.start(0)\n"
        "if host.is_worker() and host.my_rank() == 1:\n"
        "    raise RuntimeError('worker 1 fails after start')\n"
        "host.finalize(0)\n")
    job = LocalJob([sys.executable, str(script)], env={"PSB_ROOT": ROOT}, capture=True,
                   num_joint=2, fail_fast=True)
    job.start()
    rc = job.wait(60)
    assert rc == 1 and "worker 1 fails after start" in job.output(), job.output()[-2000:]


def test_job_ends_when_a_python_handle_raises(tmp_path):
    """A Python request handle that raises ends its server process with status 1 (the request
    would never be answered otherwise), and the launcher ends the job."""
    from ps_lite_b200.launch.local import LocalJob
    script = tmp_path / "badhandle.py"
    script.write_text(
        "import os, sys\n"
        "import numpy as np\n"
        "sys.path.insert(0, os.environ['PSB_ROOT'])\n"
        "from ps_lite_b200 import host\n"
        "host.start(0)\n"
        "server = None\n"
        "if host.is_server():\n"
        "    def handle(srv, req):\n"
        "        raise ValueError('handle is broken')\n"
        "    server = host.KVServer(0, handle)\n"
        "if host.is_worker():\n"
        "    kv = host.KVWorker(0, 0)\n"
        "    kv.wait(kv.push(np.array([1], np.uint64), np.ones(1, np.float32)))\n"
        "host.finalize(0)\n")
    job = LocalJob([sys.executable, str(script)], env={"PSB_ROOT": ROOT}, capture=True,
                   num_workers=1, num_servers=1, fail_fast=True)
    job.start()
    rc = job.wait(60)
    out = job.output()
    assert rc != 0 and "handle is broken" in out and "request handle raised" in out, out[-2000:]


def test_tracker_entry_points_of_the_reference(tmp_path):
    """Command lines written for the reference's tracker scripts work: same place, same flags."""
    hf = tmp_path / "hosts"
    hf.write_text("10.0.0.1\n10.0.0.2\n")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tracker", "dmlc_mpi.py"), "--nworker",
                        "2", "--server-nodes", "1", "-H", str(hf), "--log-level", "DEBUG",
                        "--dry-run", "./prog"], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "DMLC_ROLE=worker" in r.stdout and "DMLC_NUM_SERVER=1" in r.stdout
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tracker", "dmlc_ssh.py"), "-n", "2",
                        "-s", "1", "-H", str(hf), "--dry-run", "./prog"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "DMLC_ROLE=server" in r.stdout, r.stdout + r.stderr
    log = tmp_path / "launcher.log"
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tracker", "dmlc_local.py"), "-n", "1",
                        "-s", "1", "--log-file", str(log), sys.executable, "-c", "print('hi')"],
                       capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "job ended with exit code 0" in log.read_text()
