"""Launches the multi-process GPU checks when the box has at least two GPUs.

The checks are ordinary parameter-server jobs: one scheduler plus N joint processes (one per
GPU) started by this package's local launcher; arena handles, barriers and the ranks' results
travel over the control plane.  With ``PSB200_TEST_LOGS=<folder>`` the output of each job is kept
there."""
import os
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _job(script, nproc, timeout=240, extra_env=None, log=None):
    sys.path.insert(0, ROOT)
    from ps_lite_b200.launch.local import LocalJob
    job = LocalJob([sys.executable, os.path.join(HERE, script)], num_joint=nproc,
                   env=extra_env or {}, capture=True, fail_fast=True)
    job.start()
    rc = job.wait(timeout)
    out = job.output()
    keep = os.environ.get("PSB200_TEST_LOGS", "")
    if log and keep and os.path.isdir(keep):
        with open(os.path.join(keep, log), "w") as fh:
            fh.write(out)
    return rc, out


def _nproc():
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    return 8 if n >= 8 else (4 if n >= 4 else 2)


@pytest.mark.parametrize("heap,nvls", [("ipc", "0"), ("vmm", "0"), ("vmm", "1")],
                         ids=["ipc-peer-loads", "vmm-peer-loads", "vmm-nvswitch-multicast"])
def test_dense_push_pull_across_gpus(cuda_device, heap, nvls):
    """Dense push / pull / push-pull across GPUs on both arena backends: CUDA-IPC handles as
    byte strings over the control plane, and cuMem arenas whose descriptors travel over Unix
    sockets named over the control plane (with and without the NVSwitch multicast alias)."""
    nproc = _nproc()
    rc, out = _job("mp_dense_check.py", nproc, log=f"mp_dense_{heap}_nvls{nvls}_n{nproc}.log",
                   extra_env={"PSB200_NVLS": nvls, "PSB200_HEAP": heap,
                              "PSB200_MULTICAST": nvls})
    assert rc == 0 and "MP_DENSE_OK" in out, out[-4000:]
    assert f"heap={heap}" in out
    if nvls == "1" and "multicast=True" in out:
        assert "nvls_used=True" in out


def test_fused_pull_gemm_sparse_and_training_across_gpus(cuda_device):
    nproc = _nproc()
    rc, out = _job("mp_fused_check.py", nproc, log=f"mp_fused_n{nproc}.log")
    assert rc == 0 and "MP_FUSED_OK" in out, out[-4000:]


def test_cpp_program_through_ps_start_across_gpus(cuda_device):
    """tests/cpp/device_plane.cc on GPUs: a C++ program that only knows ps::Start, KVWorker and
    the plane's declaration call.  Includes a request that no peer matches: the kernel's wait
    runs out (a flag that nothing sets), Wait throws, the channel is cleared and used again.
    Runs with the multicast alias off, as every test of a failure path does."""
    import subprocess
    nproc = min(_nproc(), 4)
    sys.path.insert(0, ROOT)
    from ps_lite_b200 import _build
    from ps_lite_b200.launch.local import LocalJob
    _build.build_device()
    core = str(_build.build_core())
    libdir = os.path.dirname(core)
    exe = os.path.join(ROOT, "build", "tests", "device_plane_gpu")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-DPLANE_DEVICE=0", "-I", os.path.join(ROOT, "include"),
           os.path.join(ROOT, "tests", "cpp", "device_plane.cc"), "-o", exe, "-L", libdir,
           "-lpsb200_core", f"-Wl,-rpath,{libdir}", "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    job = LocalJob([exe], num_joint=nproc, capture=True, fail_fast=True,
                   env={"PSB200_NVLS": "0", "PSB200_MULTICAST": "0"})
    job.start()
    rc = job.wait(120)
    out = job.output()
    assert rc == 0 and out.count("DEVICE_PLANE_OK") == nproc, out[-4000:]


def test_bert_large_parity_with_single_process_adam(cuda_device):
    """Ten steps of BERT-large through the server-side Adam on N ranks against single-process
    torch Adam on the global batch, loss compared at every step."""
    nproc = min(_nproc(), 4)
    rc, out = _job("mp_bert_parity.py", nproc, timeout=400, log=f"mp_bert_parity_n{nproc}.log")
    assert rc == 0 and "MP_BERT_PARITY_OK" in out, out[-4000:]
