"""Launches the multi-process GPU checks when the box has at least two GPUs."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(script, nproc, timeout=600, extra_env=None):
    env = dict(os.environ)
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, script)]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("nvls", ["0", "1"], ids=["peer-loads", "nvswitch-multicast"])
def test_dense_push_pull_across_gpus(cuda_device, nvls):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 8 if n >= 8 else (4 if n >= 4 else 2)
    r = _torchrun("mp_dense_check.py", nproc, extra_env={"PSB200_NVLS": nvls})
    assert r.returncode == 0 and "MP_DENSE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
    if nvls == "1" and "multicast=True" in r.stdout:
        assert "nvls_used=True" in r.stdout


def test_fused_pull_gemm_sparse_and_training_across_gpus(cuda_device):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 8 if n >= 8 else (4 if n >= 4 else 2)
    r = _torchrun("mp_fused_check.py", nproc)
    assert r.returncode == 0 and "MP_FUSED_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(os.environ.get("PSB200_TEST_VMM_MULTI") != "1",
                    reason="set PSB200_TEST_VMM_MULTI=1: the import of cuMem arenas on a peer GPU "
                           "has not yet been run on a multi-GPU box")
def test_dense_push_pull_across_gpus_on_vmm_arenas(cuda_device):
    """Same check with the arenas of src/device/vmm_heap.cu: descriptors exchanged over Unix
    sockets, every rank maps every peer's physical allocation."""
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    nproc = 8 if n >= 8 else (4 if n >= 4 else 2)
    r = _torchrun("mp_dense_check.py", nproc,
                  extra_env={"PSB200_NVLS": "0", "PSB200_HEAP": "vmm"})
    assert r.returncode == 0 and "MP_DENSE_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
