"""Host runtime (C++): unit tests and multi-process integration tests on CPU.

The integration programs are the same kind the reference ships (tests/test_*.cc run under
tests/local.sh: one process per role on one host); here they are built with g++ against
``include/`` and ``libpsb200_core.so`` and started by the package's local launcher.
"""
import os
import subprocess
import time

import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "build", "tests")
sys.path.insert(0, ROOT)
from baseline import reference_source  # noqa: E402

# the reference's own test programs: PS_REFERENCE_SRC, or the copy under baseline/_ref
REF_TESTS = os.path.join(reference_source() or os.path.join(ROOT, "missing"), "tests")


@pytest.fixture(scope="session")
def core_lib():
    from ps_lite_b200 import _build
    path = _build.build_core()
    assert path is not None
    return str(path)


def _compile(src, core_lib, out_name=None):
    os.makedirs(BIN, exist_ok=True)
    out = os.path.join(BIN, out_name or os.path.splitext(os.path.basename(src))[0])
    libdir = os.path.dirname(core_lib)
    deps = [src, core_lib]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return out
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-I", os.path.join(ROOT, "include"), src, "-o", out,
           "-L", libdir, "-lpsb200_core", f"-Wl,-rpath,{libdir}", "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-4000:]
    return out


def _prog(name, core_lib):
    return _compile(os.path.join(ROOT, "tests", "cpp", name + ".cc"), core_lib)


def _job(cmd, **kw):
    from ps_lite_b200.launch.local import LocalJob
    timeout = kw.pop("timeout", 90)
    job = LocalJob(cmd, capture=True, **kw)
    job.start()
    rc = job.wait(timeout)
    return rc, job.output()


def test_unit_core(core_lib):
    r = subprocess.run([_prog("unit_core", core_lib)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "UNIT_OK" in r.stdout, r.stderr[-3000:]


def test_loop_van_single_process(core_lib):
    r = subprocess.run([_prog("loop_kv", core_lib)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "LOOP_OK" in r.stderr, r.stderr[-3000:]


@pytest.mark.parametrize("env", [{}, {"DMLC_LOCAL": "1"}, {"DMLC_PS_VAN_TYPE": "p3"},
                                 {"DMLC_PS_VAN_TYPE": "zmq"}],
                         ids=["tcp", "ipc", "p3", "zmq-alias"])
def test_config1_separate_roles(core_lib, env):
    rc, out = _job([_prog("kv_config1", core_lib)], num_workers=2, num_servers=2, env=env)
    assert rc == 0 and out.count("CONFIG1_OK") == 2, out[-3000:]


@pytest.mark.parametrize("n", [1, 2, 4])
def test_config1_joint_processes(core_lib, n):
    """Every process is worker and server at once (the layout used with one process per GPU)."""
    rc, out = _job([_prog("kv_config1", core_lib)], num_joint=n)
    assert rc == 0 and out.count("CONFIG1_OK") == n, out[-3000:]


@pytest.mark.parametrize("layout", [dict(num_workers=3, num_servers=2), dict(num_joint=3)],
                         ids=["separate", "joint"])
def test_kv_features(core_lib, layout):
    rc, out = _job([_prog("kv_features", core_lib)], **layout)
    assert rc == 0 and out.count("FEATURES_OK") == 3, out[-3000:]


def test_two_customers_in_one_worker_process(core_lib):
    from ps_lite_b200.launch.local import LocalJob
    job = LocalJob([_prog("multi_customer", core_lib)], num_workers=2, num_servers=2, capture=True)
    job._spawn("scheduler", 0)
    job._spawn("server", 0)
    job._spawn("server", 1)
    job._spawn("worker", 0)  # one process, two customer threads
    rc = job.wait(90)
    out = job.output()
    assert rc == 0 and "CUSTOMER_OK 0" in out and "CUSTOMER_OK 1" in out, out[-3000:]


def test_device_plane_single_process_loop_van(core_lib):
    """Start -> Push/Pull/PushPull on a registered tensor -> Wait -> Finalize through KVWorker,
    served by the device plane (CPU stand-in) in one process under the loop van."""
    env = dict(os.environ, DMLC_PS_VAN_TYPE="loop")
    r = subprocess.run([_prog("device_plane", core_lib)], capture_output=True, text=True,
                       timeout=90, env=env)
    assert r.returncode == 0 and "DEVICE_PLANE_OK rank 0 of 1" in r.stderr, r.stderr[-3000:]


@pytest.mark.parametrize("layout", [dict(num_joint=2), dict(num_joint=4),
                                    dict(num_workers=3, num_servers=1),
                                    dict(num_joint=2, env={"DMLC_LOCAL": "1"})],
                         ids=["joint2", "joint4", "separate3", "joint2-ipc"])
def test_device_plane_multi_process(core_lib, layout):
    """The same program as several processes: arena handles travel over the control plane,
    barriers are Postoffice barriers, requests complete the Customer tracker, and a request
    that no peer matches fails with an error instead of hanging."""
    n = layout.get("num_joint") or layout["num_workers"]
    rc, out = _job([_prog("device_plane", core_lib)], **layout)
    assert rc == 0 and out.count("DEVICE_PLANE_OK") == n, out[-3000:]


def test_barrier_from_two_customers_of_two_processes(core_lib):
    """Explicit Barrier calls from both customer threads of two worker processes, one thread
    arriving late in one of them: every call passes exactly one round and nothing hangs."""
    from ps_lite_b200.launch.local import LocalJob
    job = LocalJob([_prog("multi_customer_barrier", core_lib)], num_workers=4, num_servers=1,
                   capture=True)
    job._spawn("scheduler", 0)
    job._spawn("server", 0)
    job._spawn("worker", 0)  # two processes, two customer threads each
    job._spawn("worker", 1)
    rc = job.wait(90)
    out = job.output()
    assert rc == 0 and out.count("BARRIER_ROUNDS_OK") == 2, out[-3000:]


@pytest.mark.parametrize("std", ["c++11", "c++14"])
def test_public_headers_compile_with_older_standards(std):
    """Programs written for the reference are built with -std=c++11 (its Makefile:21): the
    public headers must not need anything newer."""
    for prog in ("kv_config1", "kv_features", "checkpoint", "helper_headers"):
        r = subprocess.run(["g++", f"-std={std}", "-O0", "-pedantic-errors", "-fsyntax-only", "-I",
                            os.path.join(ROOT, "include"),
                            os.path.join(ROOT, "tests", "cpp", prog + ".cc")],
                           capture_output=True, text=True, timeout=300)
        assert r.returncode == 0, r.stderr[-3000:]


def test_key32_build(tmp_path):
    """USE_KEY32 (make/ps.mk:8-10 of the reference): keys are 32 bits wide; the runtime, the
    unit tests and the 2 x 2 correctness job are rebuilt with it."""
    import glob
    out = str(tmp_path)
    flags = ["-std=c++17", "-O1", "-fPIC", "-pthread", "-DUSE_KEY32=1", "-I",
             os.path.join(ROOT, "include"), "-I", os.path.join(ROOT, "src")]
    objs, procs = [], []
    for src in sorted(glob.glob(os.path.join(ROOT, "src", "core", "*.cc")) +
                      glob.glob(os.path.join(ROOT, "src", "van", "*.cc"))):
        objs.append(os.path.join(out, os.path.basename(src)[:-3] + ".o"))
        procs.append(subprocess.Popen(["g++", *flags, "-c", src, "-o", objs[-1]]))
    assert all(p.wait() == 0 for p in procs)
    lib = os.path.join(out, "libps_key32.a")
    if os.path.exists(lib):
        os.remove(lib)
    subprocess.check_call(["ar", "cr", lib, *objs])
    for prog in ("unit_core", "kv_config1"):
        subprocess.check_call(["g++", *flags, os.path.join(ROOT, "tests", "cpp", prog + ".cc"), lib,
                               "-o", os.path.join(out, prog)])
    r = subprocess.run([os.path.join(out, "unit_core")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "UNIT_OK" in r.stdout, r.stderr[-3000:]
    rc, text = _job([os.path.join(out, "kv_config1")], num_workers=2, num_servers=2)
    assert rc == 0 and text.count("CONFIG1_OK") == 2, text[-3000:]


@pytest.mark.parametrize("layout", [dict(num_workers=2, num_servers=2), dict(num_joint=2)],
                         ids=["separate", "joint"])
def test_checkpoint_commands(core_lib, tmp_path, layout):
    """Servers save and reload their shard on a group request (include/ps/kv_checkpoint.h)."""
    rc, out = _job([_prog("checkpoint", core_lib), str(tmp_path)], **layout)
    assert rc == 0 and out.count("CHECKPOINT_OK") == 2, out[-3000:]
    assert sorted(os.listdir(tmp_path)) == ["server-0.kv", "server-1.kv"]


def test_garbage_on_the_wire_does_not_hurt_a_node(core_lib):
    """Strangers talk to the scheduler's port while a job starts: random bytes, a frame header
    with an absurd meta length, a data frame of 2^62 bytes.  The connections are dropped, the
    node neither crashes nor allocates what it was told to, and the job completes."""
    import socket
    import struct
    import threading
    import time
    from ps_lite_b200.launch.local import LocalJob
    job = LocalJob([_prog("kv_config1", core_lib)], num_workers=2, num_servers=2, capture=True)
    job._spawn("scheduler", 0)
    magic = 0x32425350

    def stranger(payload):
        deadline = time.time() + 20
        while time.time() < deadline:
            try:
                with socket.create_connection(("127.0.0.1", job.port), timeout=2) as s:
                    s.sendall(payload)
                    time.sleep(0.2)
                return
            except OSError:
                time.sleep(0.05)

    payloads = [
        os.urandom(4096),
        struct.pack("<IiiII", magic, 9, 1, 0xFFFFFFF0, 0),                       # meta of 4 GB
        struct.pack("<IiiII", magic, 9, 1, 4, 1) + struct.pack("<Q", 1 << 62) + b"abcd",
        struct.pack("<IiiII", magic, 9, 1, 4, 65),                               # too many frames
    ]
    threads = [threading.Thread(target=stranger, args=(p,)) for p in payloads]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for i in range(2):
        job._spawn("server", i)
    for i in range(2):
        job._spawn("worker", i)
    rc = job.wait(90)
    out = job.output()
    assert rc == 0 and out.count("CONFIG1_OK") == 2, out[-3000:]


def test_shm_pool_unit(core_lib):
    """Shared-memory array pool: recycling, views that outlive their array, own segments echoed."""
    r = subprocess.run([_prog("shm_frames", core_lib)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "SHM_UNIT_OK" in r.stderr, r.stderr[-3000:]


@pytest.mark.parametrize("env", [{}, {"PS_RESEND": "1", "PS_RESEND_TIMEOUT": "200",
                                      "PS_DROP_MSG": "10"}], ids=["plain", "drop-resend"])
def test_shm_frames_between_processes(core_lib, env):
    """DMLC_LOCAL=1: large arrays are mapped by the receiver instead of being copied through the
    socket; a server that keeps received arrays must see them unchanged after the worker has
    freed and recycled its buffers."""
    env = dict(env, DMLC_LOCAL="1")
    rc, out = _job([_prog("shm_frames", core_lib), "job"], num_workers=2, num_servers=2, env=env)
    assert rc == 0 and out.count("SHM_JOB_OK") == 2, out[-3000:]


@pytest.mark.parametrize("repeat", range(3))
def test_message_loss_with_resend(core_lib, repeat):
    """10 % of received messages are dropped; ACK/resend/de-duplication must hide it."""
    env = {"PS_RESEND": "1", "PS_RESEND_TIMEOUT": "100", "PS_DROP_MSG": "10"}
    rc, out = _job([_prog("kv_config1", core_lib)], num_workers=2, num_servers=2, env=env)
    assert rc == 0 and out.count("CONFIG1_OK") == 2, out[-3000:]
    assert "drop message" in out


def test_dead_node_detection_and_recovery(core_lib):
    from ps_lite_b200.launch.local import LocalJob
    env = {"PS_HEARTBEAT_INTERVAL": "1", "PS_HEARTBEAT_TIMEOUT": "2"}
    job = LocalJob([_prog("recovery", core_lib)], num_workers=2, num_servers=1, env=env,
                   capture=True)
    job._spawn("scheduler", 0)
    job._spawn("server", 0)
    job._spawn("worker", 0)
    victim = job._spawn("worker", 1, extra_env={"PSB_TEST_DIE": "1"})
    victim["expected_dead"] = True
    sched = job.procs[0]["proc"]
    # wait until the scheduler reports the dead worker
    import selectors
    sel = selectors.DefaultSelector()
    sel.register(sched.stdout, selectors.EVENT_READ)
    dead_id, deadline, buf = None, time.time() + 40, ""
    os.set_blocking(sched.stdout.fileno(), False)
    while dead_id is None and time.time() < deadline:
        if sel.select(timeout=0.2):
            chunk = sched.stdout.read() or ""
            buf += chunk
            for line in buf.splitlines():
                if line.startswith("DEAD "):
                    dead_id = int(line.split()[1])
    job.procs[0]["output"] += buf
    assert dead_id is not None, "scheduler never reported a dead node\n" + buf[-2000:]
    os.set_blocking(sched.stdout.fileno(), True)
    job.spawn_replacement("worker", 1, extra_env={"PSB_TEST_REPLACEMENT": "1"})
    rc = job.wait(60)
    out = job.output()
    assert rc == 0, out[-4000:]
    assert f"RECOVERED {dead_id}" in out, out[-4000:]
    assert f"WORKER_DONE {dead_id}" in out


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="reference sources not mounted")
@pytest.mark.parametrize("name", ["test_connection", "test_simple_app", "test_kv_app"])
def test_reference_programs_build_and_pass_unchanged(core_lib, name):
    """The reference's own test programs compile against these headers without edits."""
    exe = _compile(os.path.join(REF_TESTS, name + ".cc"), core_lib, out_name="ref_" + name)
    rc, out = _job([exe], num_workers=2, num_servers=2)
    assert rc == 0, out[-3000:]


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="reference sources not mounted")
def test_reference_multi_worker_program(core_lib):
    from ps_lite_b200.launch.local import LocalJob
    exe = _compile(os.path.join(REF_TESTS, "test_kv_app_multi_workers.cc"), core_lib,
                   out_name="ref_multi_workers")
    job = LocalJob([exe], num_workers=2, num_servers=2, capture=True, role_as_arg=True)
    job._spawn("scheduler", 0)
    job._spawn("server", 0)
    job._spawn("server", 1)
    job._spawn("worker", 0)
    assert job.wait(90) == 0, job.output()[-3000:]


def test_program_that_returns_without_finalize_ends(core_lib, tmp_path):
    """A C++ program that starts the runtime and returns from main without Finalize ends with
    its own status: the van's threads still run, so the runtime is not torn down under them."""
    src = tmp_path / "nofin.cc"
    src.write_text('#include "ps/ps.h"\nint main() { ps::Start(0); return 3; }\n')
    exe = _compile(str(src), core_lib, out_name="nofin")
    env = dict(os.environ, DMLC_PS_VAN_TYPE="loop")
    env.pop("DMLC_ROLE", None)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=30, env=env)
    assert r.returncode == 3, r.stderr[-2000:]


def test_shell_entry_points_of_the_reference(core_lib):
    """tests/local.sh and tests/repeat.sh take the command lines of the reference's scripts of
    the same names."""
    exe = _prog("kv_config1", core_lib)
    r = subprocess.run(["bash", os.path.join(ROOT, "tests", "repeat.sh"), "2", "bash",
                        os.path.join(ROOT, "tests", "local.sh"), "2", "2", exe],
                       capture_output=True, text=True, timeout=180)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and out.count("CONFIG1_OK") == 4 and "run 2 of 2" in out, out[-2000:]
    r = subprocess.run(["bash", os.path.join(ROOT, "tests", "repeat.sh"), "3", "false"],
                       capture_output=True, text=True, timeout=30)
    assert r.returncode == 1 and "run 1 failed" in r.stdout and "run 2 of" not in r.stdout


@pytest.mark.skipif(not os.path.isdir(REF_TESTS), reason="reference sources not mounted")
def test_reference_multi_workers_through_its_shell_script(core_lib):
    """tests/local_multi_workers.sh: one worker process hosting both worker customers, role as
    last argument, on the reference's own test program."""
    exe = _compile(os.path.join(REF_TESTS, "test_kv_app_multi_workers.cc"), core_lib,
                   out_name="ref_multi_workers")
    r = subprocess.run(["bash", os.path.join(ROOT, "tests", "local_multi_workers.sh"), "2", "2",
                        exe], capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, (r.stdout + r.stderr)[-2000:]
