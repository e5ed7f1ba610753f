"""In-tree build of the native libraries.

Two shared objects are produced under ``ps_lite_b200/lib``:

* ``libpsb200_device.so`` -- the sm_100a CUDA data plane (``src/kernels``, ``src/device``),
  exported through the C ABI of ``include/ps/device/psdev.h``.
* ``libpsb200_core.so`` -- the C++17 host runtime (``src/core``, ``src/van``, ``src/capi``):
  wire codec, vans, Postoffice, Customer, KV apps, exported through ``src/capi/ps_c_api.h``.

Both are plain ``nvcc`` / ``g++`` invocations (no JIT cache): the built files sit next to
the sources so that a snapshot of the tree is runnable as is.  The counterpart in the
reference is its ``Makefile``/``CMakeLists.txt`` producing ``libps.a`` (Makefile:47-49).
"""
from __future__ import annotations

import contextlib
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LIB_DIR = Path(__file__).resolve().parent / "lib"
OBJ_DIR = ROOT / "build" / "obj"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = os.environ.get("CXX") or shutil.which("g++") or "g++"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math" if os.environ.get("PSB200_FAST_MATH") else "-DPSB200_PRECISE",
    "-Xcompiler", "-fPIC", "-I", str(ROOT / "include"), "-I", str(ROOT / "src"),
]
CXX_FLAGS = ["-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-pthread",
             "-I", str(ROOT / "include"), "-I", str(ROOT / "src")]


def _sources(*dirs: str, exts=(".cu", ".cc")) -> list[Path]:
    out: list[Path] = []
    for d in dirs:
        p = ROOT / d
        if p.is_dir():
            out += sorted(f for f in p.iterdir() if f.suffix in exts)
    return out


def _headers_stamp(dirs=("include", "src")) -> str:
    """Hash of every header under `dirs`: part of each object's name, so that a changed header
    recompiles what may include it."""
    h = hashlib.sha1()
    for d in dirs:
        for f in sorted((ROOT / d).rglob("*")):
            if f.suffix in (".h", ".cuh", ".hpp", ".inl"):
                h.update(str(f.relative_to(ROOT)).encode())
                h.update(f.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, stamp: str, verbose: bool, extra: tuple = (),
                 obj_dir: Path = OBJ_DIR) -> Path:
    flags = [*(NVCC_FLAGS if src.suffix == ".cu" else CXX_FLAGS), *extra]
    flag_text = " ".join(flags).replace(str(ROOT), "")
    tag = hashlib.sha1(src.read_bytes() + stamp.encode() + flag_text.encode()).hexdigest()[:12]
    obj_dir.mkdir(parents=True, exist_ok=True)
    obj = obj_dir / f"{src.stem}.{tag}.o"
    if obj.exists():
        return obj
    for old in obj_dir.glob(f"{src.stem}.*.o"):
        old.unlink()
    if src.suffix == ".cu":
        cmd = [NVCC, *flags, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd[1:1] = ["-Xptxas", "-v"]
    else:
        cmd = [CXX, *flags, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and r.stderr:
        sys.stderr.write(r.stderr)
    return obj


def _link(objs: list[Path], out: Path, cuda: bool, extra: list[str]) -> None:
    manifest = out.with_suffix(".manifest")
    want = "\n".join(o.name for o in objs)
    if out.exists() and manifest.exists() and manifest.read_text() == want:
        return
    if cuda:
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(out), *map(str, objs), "-lcudart", *extra]
    else:
        # Always the shared libstdc++: some toolchains link the static one by default, and a
        # second copy of the C++ runtime inside this library clashes with the one that the
        # programs linking it, and torch in the same Python process, already use.
        cmd = [CXX, "-shared", "-pthread", "-nostdlib++", "-o", str(out), *map(str, objs),
               "-l:libstdc++.so.6", "-lm", *extra]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 and not cuda:
        # a compiler without -nostdlib++ or a system without that soname: default link
        cmd = [CXX, "-shared", "-pthread", "-o", str(out), *map(str, objs), *extra]
        r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    manifest.write_text(want)


@contextlib.contextmanager
def _build_lock():
    """Serialises concurrent builders (one process per GPU may import at the same time)."""
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    with open(LIB_DIR / ".build.lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            yield
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def build_device(verbose: bool = False, checks: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link libpsb200_device.so.

    ``checks=True`` builds the checks variant instead (``-DPSDEV_CHECKS``,
    libpsb200_device_checks.so): the dense kernel verifies every index against the table, the
    owner's state arrays and the arena before it touches memory, records
    ``PSDEV_ERR_BOUNDS`` in the channel status and skips the access instead of performing it.
    ``PSB200_DEVICE_CHECKS=1`` makes the package load that variant."""
    with _build_lock():
        return _build_device(verbose, checks)


def _build_device(verbose: bool, checks: bool = False) -> Path:
    srcs = _sources("src/kernels", "src/device", exts=(".cu",))
    # device sources include nothing outside these directories: a change to a host-only
    # header does not rebuild the kernels
    stamp = _headers_stamp(("include/ps/device", "src/kernels", "src/device"))
    extra = ("-DPSDEV_CHECKS=1",) if checks else ()
    obj_dir = ROOT / "build" / "obj_checks" if checks else OBJ_DIR
    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, stamp, verbose, extra, obj_dir), srcs))
    out = LIB_DIR / ("libpsb200_device_checks.so" if checks else "libpsb200_device.so")
    _link(objs, out, cuda=True, extra=[])
    return out


def build_core(verbose: bool = False) -> Path | None:
    """Compile the host runtime and link libpsb200_core.so (None if no sources yet)."""
    with _build_lock():
        return _build_core(verbose)


def _build_core(verbose: bool) -> Path | None:
    srcs = _sources("src/core", "src/van", "src/capi", exts=(".cc",))
    if not srcs:
        return None
    stamp = _headers_stamp()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, stamp, verbose), srcs))
    out = LIB_DIR / "libpsb200_core.so"
    _link(objs, out, cuda=False, extra=[])
    return out


def build_all(verbose: bool = False) -> dict[str, str]:
    res = {"device": str(build_device(verbose))}
    core = build_core(verbose)
    if core:
        res["core"] = str(core)
    return res


if __name__ == "__main__":
    print(build_all(verbose="-v" in sys.argv))
