"""Single-host launcher: scheduler + servers + workers (or joint nodes) as local processes.

Equivalent of the reference's ``tracker/dmlc_local.py`` (:59-97) and ``tests/local.sh``
(:8-37): every process gets ``DMLC_ROLE``, ``DMLC_NUM_WORKER``, ``DMLC_NUM_SERVER``,
``DMLC_PS_ROOT_URI`` and ``DMLC_PS_ROOT_PORT``; a process that exits with code 254 is
restarted with ``DMLC_NUM_ATTEMPT`` incremented (the reference's keep-alive loop,
dmlc_local.py:15-25).  ``--joint N`` starts N processes that are worker and server at once
(one per GPU) instead of separate workers and servers.

    python -m ps_lite_b200.launch.local -n 2 -s 2 ./my_program args...
    python -m ps_lite_b200.launch.local --joint 8 python train.py
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import threading
import time
from typing import Dict, List, Optional, Sequence

from .tracker import free_port


class LocalJob:
    """A set of local processes forming one parameter-server job."""

    def __init__(self, cmd: Sequence[str], num_workers: int = 0, num_servers: int = 0,
                 num_joint: int = 0, env: Optional[Dict[str, str]] = None,
                 port: Optional[int] = None, role_as_arg: bool = False,
                 capture: bool = False, per_role_env: Optional[Dict[str, Dict[str, str]]] = None,
                 fail_fast: bool = False, worker_processes: Optional[int] = None):
        self.cmd = list(cmd)
        # processes started with the worker role; fewer than num_workers when one process hosts
        # several worker customers (the reference's tests/local_multi_workers.sh starts one)
        self.worker_processes = worker_processes
        self.num_joint = num_joint
        self.num_workers = num_joint or num_workers
        self.num_servers = num_joint or num_servers
        self.port = port or free_port(20000, 45000)
        self.base_env = dict(os.environ)
        self.base_env.update(env or {})
        self.base_env.update({
            "DMLC_NUM_WORKER": str(self.num_workers), "DMLC_NUM_SERVER": str(self.num_servers),
            "DMLC_PS_ROOT_URI": "127.0.0.1", "DMLC_PS_ROOT_PORT": str(self.port)})
        self.role_as_arg = role_as_arg
        self.capture = capture
        self.per_role_env = per_role_env or {}
        # a process that fails ends the job: the others are stopped a few seconds later
        # instead of waiting at a barrier for a node that will never come
        self.fail_fast = fail_fast
        self.procs: List[dict] = []
        self._lock = threading.Lock()

    def _spawn(self, role: str, index: int, attempt: int = 0, extra_env=None) -> dict:
        env = dict(self.base_env)
        env["DMLC_ROLE"] = role
        env["DMLC_NUM_ATTEMPT"] = str(attempt)
        env["PSB200_LOCAL_INDEX"] = str(index)
        env.update(self.per_role_env.get(role, {}))
        env.update(extra_env or {})
        cmd = self.cmd + ([role] if self.role_as_arg else [])
        kw = dict(stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) if self.capture else {}
        p = subprocess.Popen(cmd, env=env, **kw)
        rec = {"role": role, "index": index, "proc": p, "attempt": attempt, "output": ""}
        with self._lock:
            self.procs.append(rec)
        return rec

    def start(self) -> None:
        self._spawn("scheduler", 0)
        if self.num_joint:
            for i in range(self.num_joint):
                self._spawn("joint", i, extra_env={"LOCAL_RANK": str(i)})
        else:
            for i in range(self.num_servers):
                self._spawn("server", i)
            for i in range(self.worker_processes or self.num_workers):
                self._spawn("worker", i)

    def spawn_replacement(self, role: str, index: int, extra_env=None) -> dict:
        """Start one more process of ``role`` (used to replace a node that died)."""
        return self._spawn(role, index, attempt=1, extra_env=extra_env)

    def wait(self, timeout: float = 120.0) -> int:
        """Wait for every process; returns 0 if all exited with 0, else the first bad code."""
        deadline = time.time() + timeout
        rc_final = 0
        pending = list(self.procs)
        while pending:
            for rec in list(pending):
                p = rec["proc"]
                rc = p.poll()
                if rc is None:
                    continue
                if self.capture and p.stdout:
                    rec["output"] += p.stdout.read() or ""
                pending.remove(rec)
                if rc == 254:  # keep-alive protocol: restart
                    new = self._spawn(rec["role"], rec["index"], rec["attempt"] + 1)
                    pending.append(new)
                elif rc != 0 and not rec.get("expected_dead") and rc_final == 0:
                    rc_final = rc
                    if self.fail_fast:
                        deadline = min(deadline, time.time() + 5.0)
            with self._lock:
                for rec in self.procs:
                    if rec not in pending and rec["proc"].poll() is None:
                        pending.append(rec)
            if time.time() > deadline:
                self.kill()
                return rc_final or 124
            time.sleep(0.02)
        return rc_final

    def kill(self) -> None:
        for rec in self.procs:
            if rec["proc"].poll() is None:
                rec["proc"].kill()
        for rec in self.procs:
            try:
                rec["proc"].wait(timeout=5)
            except subprocess.TimeoutExpired:
                pass
            if self.capture and rec["proc"].stdout:
                try:
                    rec["output"] += rec["proc"].stdout.read() or ""
                except ValueError:
                    pass

    def output(self) -> str:
        return "\n".join(f"--- {r['role']}[{r['index']}] ---\n{r['output']}" for r in self.procs)


def run(cmd: Sequence[str], num_workers: int = 0, num_servers: int = 0, num_joint: int = 0,
        env: Optional[Dict[str, str]] = None, timeout: float = 120.0, role_as_arg: bool = False,
        capture: bool = False, fail_fast: bool = False, worker_processes: Optional[int] = None):
    """Start a job, wait for it, return (exit code, LocalJob)."""
    job = LocalJob(cmd, num_workers, num_servers, num_joint, env, role_as_arg=role_as_arg,
                   capture=capture, fail_fast=fail_fast, worker_processes=worker_processes)
    job.start()
    rc = job.wait(timeout)
    return rc, job


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="launch a parameter-server job on this host")
    ap.add_argument("-n", "--num-workers", type=int, default=0)
    ap.add_argument("-s", "--num-servers", type=int, default=0)
    ap.add_argument("--joint", type=int, default=0,
                    help="number of processes that are worker and server at once")
    ap.add_argument("--env", action="append", default=[], help="KEY=VALUE for every process")
    ap.add_argument("--role-as-arg", action="store_true",
                    help="append the role name to the command line of each process")
    ap.add_argument("--worker-processes", type=int, default=None,
                    help="start this many worker processes instead of one per worker (a "
                         "process then hosts several worker customers)")
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("--keep-going", action="store_true",
                    help="do not stop the other processes when one exits with an error")
    ap.add_argument("--repeat", type=int, default=1,
                    help="run the job this many times, stop at the first failure (a race "
                         "shaker, like tests/repeat.sh of the reference)")
    # accepted for command lines written for the reference's tracker/dmlc_local.py
    ap.add_argument("--log-level", default="INFO", choices=["INFO", "DEBUG"],
                    help="logging level of the launcher itself")
    ap.add_argument("--log-file", default=None, help="file for the launcher's own log")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    import logging
    logging.basicConfig(level=getattr(logging, args.log_level), filename=args.log_file,
                        format="%(asctime)s %(levelname)s %(message)s")
    if not args.command:
        ap.error("no command given")
    if not args.joint and (args.num_workers <= 0 or args.num_servers <= 0):
        ap.error("give -n and -s, or --joint")
    env = dict(kv.split("=", 1) for kv in args.env)
    rc = 0
    for i in range(max(1, args.repeat)):
        logging.info("starting %s with %d workers, %d servers, %d joint nodes",
                     " ".join(args.command), args.num_workers, args.num_servers, args.joint)
        rc, _ = run(args.command, args.num_workers, args.num_servers, args.joint, env,
                    args.timeout, args.role_as_arg, fail_fast=not args.keep_going,
                    worker_processes=args.worker_processes)
        logging.info("job ended with exit code %d", rc)
        if rc != 0:
            if args.repeat > 1:
                print(f"run {i + 1} of {args.repeat} failed with exit code {rc}", file=sys.stderr)
            break
    return rc


if __name__ == "__main__":
    sys.exit(main())
