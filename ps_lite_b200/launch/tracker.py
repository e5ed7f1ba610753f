"""Job tracker: starts the scheduler and hands the DMLC_* environment to a launcher.

Role of the reference's ``tracker/tracker.py`` (``PSTracker`` :318-365 and ``submit``
:384-433): pick the scheduler address, export ``DMLC_NUM_WORKER``, ``DMLC_NUM_SERVER``,
``DMLC_PS_ROOT_URI`` and ``DMLC_PS_ROOT_PORT``, run the scheduler process, then call a
launcher callback that starts workers and servers with that environment.  The rabit
tree/ring bootstrap of the reference's tracker is not parameter-server functionality and
has no counterpart here.
"""
from __future__ import annotations

import os
import socket
import subprocess
import threading
from typing import Callable, Dict, Optional, Sequence


def free_port(lo: int = 9091, hi: int = 9999) -> int:
    """A TCP port in [lo, hi] that can be bound right now (falls back to any free port)."""
    for port in range(lo, hi + 1):
        with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
            try:
                s.bind(("", port))
                return port
            except OSError:
                continue
    with socket.socket() as s:
        s.bind(("", 0))
        return s.getsockname()[1]


def host_ip(prefer: Optional[str] = None) -> str:
    """Address other hosts can use to reach this one ("127.0.0.1" if none is found)."""
    if prefer and prefer not in ("auto", "ip", "dns"):
        return prefer
    try:
        with socket.socket(socket.AF_INET, socket.SOCK_DGRAM) as s:
            s.connect(("10.255.255.255", 1))
            return s.getsockname()[0]
    except OSError:
        return "127.0.0.1"


class PSTracker:
    """Runs the scheduler process of a job and knows the environment of its nodes."""

    def __init__(self, cmd: Optional[Sequence[str]], host: str = "127.0.0.1",
                 port: Optional[int] = None, envs: Optional[Dict[str, str]] = None):
        self.host = host
        self.port = port or free_port()
        self.cmd = list(cmd) if cmd else None
        self.proc: Optional[subprocess.Popen] = None
        self.envs = dict(envs or {})
        self.envs.update({"DMLC_PS_ROOT_URI": self.host, "DMLC_PS_ROOT_PORT": str(self.port)})

    def node_envs(self) -> Dict[str, str]:
        """Environment every worker and server of the job needs."""
        return dict(self.envs)

    def start(self) -> None:
        if self.cmd is None:
            return
        env = dict(os.environ)
        env.update(self.envs)
        env["DMLC_ROLE"] = "scheduler"
        self.proc = subprocess.Popen(self.cmd, env=env)

    def join(self, timeout: Optional[float] = None) -> int:
        if self.proc is None:
            return 0
        return self.proc.wait(timeout=timeout)

    def kill(self) -> None:
        if self.proc and self.proc.poll() is None:
            self.proc.kill()


def submit(nworker: int, nserver: int, fun_submit: Callable[[int, int, Dict[str, str]], None],
           pscmd: Optional[Sequence[str]], host: str = "127.0.0.1",
           envs: Optional[Dict[str, str]] = None, timeout: Optional[float] = None) -> int:
    """Start the scheduler, call ``fun_submit(nworker, nserver, envs)``, wait for the scheduler."""
    envs = dict(envs or {})
    envs.update({"DMLC_NUM_WORKER": str(nworker), "DMLC_NUM_SERVER": str(nserver)})
    tracker = PSTracker(pscmd, host=host, envs=envs)
    tracker.start()
    t = threading.Thread(target=fun_submit, args=(nworker, nserver, tracker.node_envs()),
                         daemon=True)
    t.start()
    rc = tracker.join(timeout)
    t.join(timeout)
    return rc
