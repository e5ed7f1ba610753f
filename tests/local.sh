#!/bin/bash
# usage: local.sh num_servers num_workers program [args...]
# One scheduler, num_servers servers and num_workers workers of `program` on this host (the
# command line of the reference's script of the same name; the launcher is
# ps_lite_b200.launch.local).
if [ $# -lt 3 ]; then
    echo "usage: $0 num_servers num_workers program [args...]"
    exit 1
fi
servers=$1; workers=$2; shift 2
root=$(cd "$(dirname "$0")/.." && pwd)
PYTHONPATH="$root${PYTHONPATH:+:$PYTHONPATH}" exec python -m ps_lite_b200.launch.local \
    -s "$servers" -n "$workers" "$@"
