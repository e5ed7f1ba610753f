"""Launcher that places servers and workers with ``mpirun`` (role of the reference's
``tracker/dmlc_mpi.py`` :33-85).  MPI is only a process starter here, as in the reference;
the library makes no MPI call.  ``--dry-run`` prints the two mpirun command lines.
"""
from __future__ import annotations

import argparse
import shlex
import subprocess
import sys
from typing import Dict, List, Sequence

from . import tracker


def mpirun_commands(nworker: int, nserver: int, envs: Dict[str, str], command: Sequence[str],
                    hostfile: str | None = None, flavor: str = "openmpi") -> List[List[str]]:
    cmds = []
    for role, n in (("server", nserver), ("worker", nworker)):
        e = dict(envs)
        e["DMLC_ROLE"] = role
        cmd = ["mpirun", "-n", str(n)]
        if hostfile:
            cmd += ["--hostfile", hostfile]
        for k, v in sorted(e.items()):
            cmd += (["-x", f"{k}={v}"] if flavor == "openmpi" else ["-env", k, str(v)])
        cmds.append(cmd + list(command))
    return cmds


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="launch a parameter-server job with mpirun")
    # (--nworker / --server-nodes / --log-* / --host-ip: the spellings of the reference's
    # tracker/dmlc_mpi.py)
    ap.add_argument("-n", "--num-workers", "--nworker", type=int, required=True)
    ap.add_argument("-s", "--num-servers", "--server-nodes", type=int, default=0)
    ap.add_argument("-H", "--hostfile", default=None)
    ap.add_argument("--log-level", default="INFO", choices=["INFO", "DEBUG"])
    ap.add_argument("--log-file", default=None)
    ap.add_argument("--host-ip", default=None,
                    help="address of this host for the scheduler (DMLC_NODE_HOST)")
    ap.add_argument("--flavor", choices=["openmpi", "mpich"], default="openmpi")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("command", nargs=argparse.REMAINDER)
    args = ap.parse_args(argv)
    import logging
    logging.basicConfig(level=getattr(logging, args.log_level), filename=args.log_file,
                        format="%(asctime)s %(levelname)s %(message)s")
    if args.host_ip:
        import os
        os.environ["DMLC_NODE_HOST"] = args.host_ip

    def launch(nworker, nserver, envs):
        procs = []
        for cmd in mpirun_commands(nworker, nserver, envs, args.command, args.hostfile, args.flavor):
            if args.dry_run:
                print(" ".join(shlex.quote(c) for c in cmd))
            else:
                procs.append(subprocess.Popen(cmd))
        for p in procs:
            p.wait()

    return tracker.submit(args.num_workers, args.num_servers, launch,
                          None if args.dry_run else args.command)


if __name__ == "__main__":
    sys.exit(main())
