"""Gives a Python process the environment of a parameter-server job, whoever launched it.

Three cases:

* The process was started by one of this package's launchers (``launch.local``, ``ssh``,
  ``mpi``) or by hand with the ``DMLC_*`` variables of the reference (docs/env.md): nothing
  to do.
* The process is one of N ranks started by ``python -m torch.distributed.run`` on one host
  (``RANK``, ``WORLD_SIZE``, ``LOCAL_RANK``, ``MASTER_ADDR``, ``MASTER_PORT``): the ranks
  become N joint nodes (worker and server at once, one per GPU).  Rank 0 picks a free port,
  starts the scheduler as a child process and publishes the port in a file under the
  temporary directory that the other ranks read; only the launcher's variables are read --
  ``torch.distributed`` itself is not used.
* Neither: a single process; the loop van makes it scheduler, server 0 and worker 0 at once.

The counterpart in the reference is ``tracker/dmlc_local.py`` (:59-97), which exports the same
variables before it starts the processes.
"""
from __future__ import annotations

import atexit
import os
import subprocess
import sys
import tempfile
import time
from typing import Optional

from .tracker import free_port

_state = {"scheduler": None, "file": None, "mode": None}


def _rendezvous_file() -> str:
    tag = "-".join([str(os.getppid()), os.environ.get("MASTER_PORT", "0"),
                    os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")])
    return os.path.join(tempfile.gettempdir(), f"psb200-rdzv-{tag}")


def _cleanup() -> None:
    f = _state.get("file")
    if f and os.path.exists(f):
        try:
            os.remove(f)
        except OSError:
            pass
    p = _state.get("scheduler")
    if p is not None and p.poll() is None:
        try:
            p.wait(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()


def abandon() -> None:
    """For a process that is about to leave without the orderly shutdown (``os._exit``): stops
    the scheduler it started, which would otherwise wait for nodes that will never report."""
    f = _state.get("file")
    if f and os.path.exists(f):
        try:
            os.remove(f)
        except OSError:
            pass
    p = _state.get("scheduler")
    if p is not None and p.poll() is None:
        p.kill()
        try:
            p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            pass


def ensure_env(timeout_s: float = 120.0) -> str:
    """Set the ``DMLC_*`` variables if the launcher did not; returns "dmlc", "torchrun" or
    "single"."""
    if _state["mode"]:
        return _state["mode"]
    env = os.environ
    if env.get("DMLC_ROLE") or env.get("DMLC_PS_VAN_TYPE") == "loop":
        _state["mode"] = "dmlc"
        return "dmlc"
    world = int(env.get("WORLD_SIZE", "1"))
    if world <= 1:
        env["DMLC_PS_VAN_TYPE"] = "loop"
        _state["mode"] = "single"
        return "single"
    rank = int(env.get("RANK", "0"))
    path = _rendezvous_file()
    t0 = time.time()
    env["DMLC_ROLE"] = "joint"
    env["DMLC_NUM_WORKER"] = env["DMLC_NUM_SERVER"] = str(world)
    env["DMLC_PS_ROOT_URI"] = "127.0.0.1"
    if rank == 0:
        port = free_port(20000, 45000)
        sched_env = dict(env)
        sched_env.update({"DMLC_ROLE": "scheduler", "DMLC_PS_ROOT_PORT": str(port)})
        for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
            sched_env.pop(k, None)
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        code = ("import sys; sys.path.insert(0, %r); from ps_lite_b200 import host; "
                "host.start(); host.finalize()" % root)
        _state["scheduler"] = subprocess.Popen([sys.executable, "-c", code], env=sched_env)
        tmp = path + ".tmp"
        with open(tmp, "w") as fh:
            fh.write(str(port))
        os.replace(tmp, path)
        _state["file"] = path
        atexit.register(_cleanup)
    else:
        port: Optional[int] = None
        while time.time() - t0 < timeout_s:
            try:
                # a file left behind by an earlier job of the same launcher is older than this
                # process by more than the launcher's start-up spread
                if os.path.getmtime(path) >= t0 - 300:
                    with open(path) as fh:
                        port = int(fh.read().strip())
                    break
            except (OSError, ValueError):
                pass
            time.sleep(0.05)
        if port is None:
            raise TimeoutError(f"rank 0 did not publish the scheduler port in {path}")
    env["DMLC_PS_ROOT_PORT"] = str(port)
    _state["mode"] = "torchrun"
    return "torchrun"


def launcher_rank() -> int:
    """Rank that the launcher gave this process (not the node rank the scheduler assigns):
    the one process that should print a job's report is launcher rank 0."""
    for k in ("RANK", "PSB200_LOCAL_INDEX"):
        if os.environ.get(k) is not None:
            return int(os.environ[k])
    return 0
