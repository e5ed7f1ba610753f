"""Builds the unmodified reference library into ``baseline/_ref`` for the reference arm.

The reference is a C++ library with no Python packaging, so ``pip install`` of it cannot work
(it reports that neither setup.py nor pyproject.toml exists).  Its own build fetches protobuf
and ZeroMQ with wget (make/deps.mk:9-48), which is impossible offline.  This script therefore
copies the sources verbatim, adds two dependency shims next to them -- ``zmq.h`` (declarations
for the libzmq shared library that ships inside pyzmq) and ``meta.pb.h`` (stand-in for the
protoc output of src/meta.proto) -- and compiles ``libps.a`` with the reference's own flags
(Makefile:21) plus the benchmark driver ``baseline/ref_bench.cc``.

    python baseline/build_ref.py [--reference <checkout of the reference>]
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
DST = os.path.join(HERE, "_ref")


def find_libzmq() -> str:
    import zmq  # noqa: F401  (only to locate site-packages)
    site = os.path.dirname(os.path.dirname(zmq.__file__))
    hits = sorted(glob.glob(os.path.join(site, "pyzmq.libs", "libzmq*.so*")))
    if not hits:
        raise RuntimeError("no libzmq shared library found next to pyzmq")
    return hits[0]


def build(reference: str) -> str:
    src_copy = os.path.join(DST, "ps-lite")
    if os.path.isdir(src_copy):
        shutil.rmtree(src_copy)
    os.makedirs(DST, exist_ok=True)
    shutil.copytree(reference, src_copy, ignore=shutil.ignore_patterns(".git"))
    for root, _, files in os.walk(src_copy):
        os.chmod(root, 0o755)
        for f in files:
            os.chmod(os.path.join(root, f), 0o644)
    deps_inc = os.path.join(DST, "deps", "include")
    os.makedirs(deps_inc, exist_ok=True)
    shutil.copy(os.path.join(HERE, "shims", "zmq.h"), deps_inc)
    shutil.copy(os.path.join(HERE, "shims", "meta.pb.h"), os.path.join(src_copy, "src"))
    libzmq = find_libzmq()
    cxx = os.environ.get("CXX", "g++")
    flags = ["-std=c++11", "-msse2", "-fPIC", "-O3", "-ggdb", "-Wall", "-finline-functions",
             "-I", os.path.join(src_copy, "src"), "-I", os.path.join(src_copy, "include"),
             "-I", deps_inc, "-Wno-unused-function", "-Wno-deprecated-declarations"]
    objs = []
    for name in ("customer", "postoffice", "van"):
        obj = os.path.join(DST, name + ".o")
        cmd = [cxx, *flags, "-c", os.path.join(src_copy, "src", name + ".cc"), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"reference build failed: {' '.join(cmd)}\n{r.stderr[-3000:]}")
        objs.append(obj)
    lib = os.path.join(DST, "libps.a")
    if os.path.exists(lib):
        os.remove(lib)
    subprocess.check_call(["ar", "crv", lib, *objs], stdout=subprocess.DEVNULL)
    exe = os.path.join(DST, "ref_bench")
    cmd = [cxx, *flags, os.path.join(HERE, "ref_bench.cc"), lib, libzmq,
           f"-Wl,-rpath,{os.path.dirname(libzmq)}", "-pthread", "-o", exe]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"ref_bench link failed: {' '.join(cmd)}\n{r.stderr[-3000:]}")
    # the reference's own correctness test, as a smoke check of the build
    t = os.path.join(DST, "test_kv_app")
    cmd = [cxx, *flags, os.path.join(src_copy, "tests", "test_kv_app.cc"), lib, libzmq,
           f"-Wl,-rpath,{os.path.dirname(libzmq)}", "-pthread", "-o", t]
    subprocess.run(cmd, capture_output=True, text=True)
    return exe


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PS_REFERENCE_SRC"), required=not
                    os.environ.get("PS_REFERENCE_SRC"),
                    help="directory of the unmodified reference sources (or PS_REFERENCE_SRC)")
    a = ap.parse_args()
    print(build(a.reference))
