#!/bin/bash
# usage: repeat.sh times command [args...]
# Runs the command up to `times` times and stops at the first failure (a race shaker).
if [ $# -lt 2 ]; then
    echo "usage: $0 times command [args...]"
    exit 1
fi
times=$1; shift
for ((run = 1; run <= times; ++run)); do
    echo "run $run of $times: $*"
    "$@" || { rc=$?; echo "run $run failed with exit code $rc"; exit $rc; }
done
