"""Race and memory-error detection for the host runtime: the C++ test programs rebuilt with
ThreadSanitizer, AddressSanitizer (+ leak check) and UndefinedBehaviorSanitizer and run in the
usual layouts.

Takes a few minutes of compile time, so it only runs when ``PS_RUN_SANITIZERS=1`` is set
(``PS_RUN_SANITIZERS=1 python -m pytest tests/test_sanitizers.py -q``).  The reference offers
the same through ``make ASAN=1`` (Makefile:29-31 there); ``make ASAN=1`` / ``make TSAN=1`` work
here too.
"""
import glob
import os
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.skipif(os.environ.get("PS_RUN_SANITIZERS") != "1",
                                reason="set PS_RUN_SANITIZERS=1 to run the sanitizer builds")
PROGRAMS = ["unit_core", "loop_kv", "shm_frames", "kv_config1", "kv_features", "multi_customer",
            "recovery", "checkpoint", "device_plane"]
MARKS = {"thread": "WARNING: ThreadSanitizer", "address": "ERROR: AddressSanitizer",
         "undefined": "runtime error:"}


@pytest.fixture(scope="module", params=["thread", "address", "undefined"])
def san(request):
    kind = request.param
    # outside the source tree: the instrumented objects are large
    out = os.path.join(tempfile.gettempdir(), f"psb200_san_{os.getuid()}", kind)
    os.makedirs(out, exist_ok=True)
    flags = ["-std=c++17", "-O1", "-g", "-fPIC", "-pthread", f"-fsanitize={kind}",
             "-fno-omit-frame-pointer", "-I", os.path.join(ROOT, "include"),
             "-I", os.path.join(ROOT, "src")]
    objs, procs = [], []
    for src in sorted(glob.glob(os.path.join(ROOT, "src", "core", "*.cc")) +
                      glob.glob(os.path.join(ROOT, "src", "van", "*.cc"))):
        obj = os.path.join(out, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        procs.append(subprocess.Popen(["g++", *flags, "-c", src, "-o", obj]))
    assert all(p.wait() == 0 for p in procs)
    lib = os.path.join(out, "libps_san.a")
    if os.path.exists(lib):
        os.remove(lib)
    subprocess.check_call(["ar", "cr", lib, *objs])
    procs = [subprocess.Popen(["g++", *flags, os.path.join(ROOT, "tests", "cpp", p + ".cc"), lib,
                               "-ldl", "-o", os.path.join(out, p)]) for p in PROGRAMS]
    assert all(p.wait() == 0 for p in procs)
    return kind, out


def _clean(kind, text):
    assert MARKS[kind] not in text, text[text.find(MARKS[kind]):][:4000]
    assert "LeakSanitizer" not in text, text[text.find("LeakSanitizer"):][:4000]


@pytest.mark.parametrize("prog,token", [("unit_core", "UNIT_OK"), ("loop_kv", "LOOP_OK"),
                                        ("shm_frames", "SHM_UNIT_OK")])
def test_single_process_programs(san, prog, token):
    kind, out = san
    r = subprocess.run([os.path.join(out, prog)], capture_output=True, text=True, timeout=600)
    _clean(kind, r.stdout + r.stderr)
    assert r.returncode == 0 and token in r.stdout + r.stderr


def test_device_plane_on_the_cpu_stand_in(san):
    """The device plane (arenas in shared memory, host loops for the kernels): handle exchange,
    KVWorker routing, staged requests, completion thread, timeout path, keyed tables."""
    kind, out = san
    env = dict(os.environ, DMLC_PS_VAN_TYPE="loop")
    r = subprocess.run([os.path.join(out, "device_plane")], capture_output=True, text=True,
                       timeout=600, env=env)
    _clean(kind, r.stdout + r.stderr)
    assert r.returncode == 0 and "DEVICE_PLANE_OK rank 0 of 1" in r.stderr, r.stderr[-3000:]


@pytest.mark.parametrize("prog,args,env,layout,token,count", [
    ("device_plane", [], {"DMLC_LOCAL": "1"}, dict(num_joint=2), "DEVICE_PLANE_OK", 2),
    ("kv_config1", [], {}, dict(num_workers=2, num_servers=2), "CONFIG1_OK", 2),
    ("kv_config1", [], {"DMLC_LOCAL": "1"}, dict(num_workers=2, num_servers=2), "CONFIG1_OK", 2),
    ("kv_config1", [], {"DMLC_PS_VAN_TYPE": "p3"}, dict(num_workers=2, num_servers=2),
     "CONFIG1_OK", 2),
    ("kv_config1", [], {}, dict(num_joint=2), "CONFIG1_OK", 2),
    ("kv_features", [], {}, dict(num_workers=3, num_servers=2), "FEATURES_OK", 3),
    ("kv_features", [], {}, dict(num_joint=3), "FEATURES_OK", 3),
    ("checkpoint", ["<tmp>"], {}, dict(num_workers=2, num_servers=2), "CHECKPOINT_OK", 2),
    ("shm_frames", ["job"], {"DMLC_LOCAL": "1"}, dict(num_workers=2, num_servers=2),
     "SHM_JOB_OK", 2),
    ("shm_frames", ["job"], {"DMLC_LOCAL": "1", "PS_RESEND": "1", "PS_RESEND_TIMEOUT": "300",
                             "PS_DROP_MSG": "10"}, dict(num_workers=2, num_servers=2),
     "SHM_JOB_OK", 2),
])
def test_multi_process_programs(san, prog, args, env, layout, token, count, tmp_path):
    from ps_lite_b200.launch.local import LocalJob
    kind, out = san
    args = [str(tmp_path) if a == "<tmp>" else a for a in args]
    job = LocalJob([os.path.join(out, prog), *args], capture=True, env=env, **layout)
    job.start()
    rc = job.wait(600)
    text = job.output()
    _clean(kind, text)
    assert rc == 0 and text.count(token) == count, text[-3000:]


@pytest.mark.parametrize("which", ["test_two_customers_in_one_worker_process",
                                   "test_dead_node_detection_and_recovery"])
def test_orchestrated_layouts(san, which, monkeypatch):
    """Two customer threads in one worker process; a worker that dies, is detected through
    heartbeats and replaced -- the orchestration of tests/test_host_runtime.py on the
    instrumented binaries."""
    import importlib.util
    from ps_lite_b200.launch import local
    kind, out = san
    spec = importlib.util.spec_from_file_location(
        "host_runtime_tests", os.path.join(ROOT, "tests", "test_host_runtime.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    monkeypatch.setattr(m, "_prog", lambda name, core_lib: os.path.join(out, name))
    texts = []
    original = local.LocalJob.output

    def recording(self):
        texts.append(original(self))
        return texts[-1]
    monkeypatch.setattr(local.LocalJob, "output", recording)
    getattr(m, which)("unused")
    assert texts
    for t in texts:
        _clean(kind, t)
