"""Multi-host launcher over ssh (role of the reference's ``tracker/dmlc_ssh.py`` :30-110).

Hosts are read from a hostfile (one ``host[:ssh_port]`` per line); servers then workers are
placed round-robin; the DMLC_* environment is forwarded as ``export K=V;`` prefixes; the
scheduler runs on this host.  ``--dry-run`` prints the commands instead of running them.
"""
from __future__ import annotations

import argparse
import os
import shlex
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

from . import tracker

_FORWARD = ("OMP_NUM_THREADS", "LD_LIBRARY_PATH", "PS_VERBOSE", "PS_RESEND", "PS_RESEND_TIMEOUT",
            "PS_HEARTBEAT_INTERVAL", "PS_HEARTBEAT_TIMEOUT", "DMLC_INTERFACE", "DMLC_PS_VAN_TYPE")


def read_hosts(path: str) -> List[Tuple[str, str]]:
    hosts = []
    with open(path) as fh:
        for line in fh:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            host, _, port = line.partition(":")
            hosts.append((host, port or "22"))
    if not hosts:
        raise ValueError(f"no hosts in {path}")
    return hosts


def build_commands(hosts: Sequence[Tuple[str, str]], nworker: int, nserver: int,
                   envs: Dict[str, str], command: Sequence[str], workdir: str) -> List[List[str]]:
    """ssh command lines for every server and worker of the job."""
    cmds = []
    for i in range(nserver + nworker):
        role = "server" if i < nserver else "worker"
        host, port = hosts[i % len(hosts)]
        exports = dict(envs)
        exports["DMLC_ROLE"] = role
        for k in _FORWARD:
            if k in os.environ and k not in exports:
                exports[k] = os.environ[k]
        prefix = " ".join(f"export {k}={shlex.quote(str(v))};" for k, v in sorted(exports.items()))
        remote = f"{prefix} cd {shlex.quote(workdir)}; {' '.join(shlex.quote(c) for c in command)}"
        cmds.append(["ssh", "-o", "StrictHostKeyChecking=no", host, "-p", port, remote])
    return cmds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="launch a parameter-server job over ssh")
    ap.add_argument("-n", "--num-workers", type=int, required=True)
    ap.add_argument("-s", "--num-servers", type=int, required=True)
    ap.add_argument("-H", "--hostfile", required=True)
    ap.add_argument("--host-ip", default="auto", help="address of this host for the scheduler")
    ap.add_argument("--sync-dir", default=None, help="rsync the working directory here first")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    hosts = read_hosts(args.hostfile)
    workdir = args.sync_dir or os.getcwd()
    procs = []

    def launch(nworker, nserver, envs):
        if args.sync_dir and not args.dry_run:
            for host, port in hosts:
                subprocess.check_call(["rsync", "-az", "--rsh", f"ssh -p {port}",
                                       os.getcwd() + "/", f"{host}:{args.sync_dir}"])
        for cmd in build_commands(hosts, nworker, nserver, envs, args.command, workdir):
            if args.dry_run:
                print(" ".join(shlex.quote(c) for c in cmd))
            else:
                procs.append(subprocess.Popen(cmd))
        for p in procs:
            p.wait()

    return tracker.submit(args.num_workers, args.num_servers, launch,
                          None if args.dry_run else args.command,
                          host=tracker.host_ip(args.host_ip))


if __name__ == "__main__":
    sys.exit(main())
