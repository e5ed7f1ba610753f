#!/bin/bash
# usage: local_multi_workers.sh num_servers num_workers program [args...]
# Like local.sh, but ONE worker process hosts all num_workers worker customers, and every
# process gets its role as last argument (what tests/test_kv_app_multi_workers.cc of the
# reference expects).
if [ $# -lt 3 ]; then
    echo "usage: $0 num_servers num_workers program [args...]"
    exit 1
fi
servers=$1; workers=$2; shift 2
root=$(cd "$(dirname "$0")/.." && pwd)
PYTHONPATH="$root${PYTHONPATH:+:$PYTHONPATH}" exec python -m ps_lite_b200.launch.local \
    -s "$servers" -n "$workers" --worker-processes 1 --role-as-arg "$@"
