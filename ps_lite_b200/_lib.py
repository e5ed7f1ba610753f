"""ctypes view of the native libraries (``include/ps/device/psdev.h``).

The libraries are built in-tree by :mod:`ps_lite_b200._build`; loading never falls back to
a Python implementation: if the shared object is missing or stale it is rebuilt, and a
failure to build or load raises.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

MAX_RANKS = 8
NUM_CHANNELS = 64
CTRL_BYTES = 65536
IPC_HANDLE_BYTES = 64

F32, BF16, I8 = 0, 1, 2
OPT_SUM, OPT_SGD, OPT_MOMENTUM, OPT_ADAM, OPT_ASSIGN = 0, 1, 2, 3, 4
OP_PUSH, OP_PULL, OP_PUSHPULL, OP_PUBLISH = 1, 2, 3, 4

ERR_NAMES = {
    0: "ok", -1: "bad argument", -2: "timeout waiting for peers to enter",
    -3: "timeout waiting for peers to leave", -4: "unsupported", -5: "out of heap memory",
    -6: "timeout inside a GEMM pipeline", -7: "output too wide for the static scratch",
    -8: "buffer or index outside the heap",
}


class World(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32),
                ("peer_base", C.c_void_p * MAX_RANKS), ("mc_base", C.c_void_p),
                ("heap_bytes", C.c_uint64)]


class Opt(C.Structure):
    _fields_ = [("kind", C.c_int32), ("scale", C.c_float), ("lr", C.c_float),
                ("momentum", C.c_float), ("weight_decay", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float),
                ("bias1", C.c_float), ("bias2", C.c_float), ("decoupled_wd", C.c_int32),
                ("user", C.c_float * 4)]


class Table(C.Structure):
    _fields_ = [("grad_off", C.c_uint64), ("weight_off", C.c_uint64),
                ("n", C.c_int64), ("blk", C.c_int64),
                ("master", C.c_void_p), ("state1", C.c_void_p), ("state2", C.c_void_p),
                ("grad_dtype", C.c_int32), ("out_dtype", C.c_int32), ("gscale_off", C.c_uint64),
                ("ll_off", C.c_uint64), ("ll_cap", C.c_int64)]


class Sparse(C.Structure):
    _fields_ = [("range", C.c_uint64), ("keys_off", C.c_uint64), ("grads_off", C.c_uint64),
                ("out_off", C.c_uint64), ("pos_off", C.c_uint64), ("acc_off", C.c_uint64),
                ("w", C.c_void_p), ("z", C.c_void_p), ("n", C.c_void_p),
                ("kind", C.c_int32), ("lr", C.c_float), ("alpha", C.c_float),
                ("beta", C.c_float), ("l1", C.c_float), ("l2", C.c_float),
                ("hkeys_off", C.c_uint64), ("capacity", C.c_uint64), ("overflow", C.c_void_p),
                ("width", C.c_int32), ("channel", C.c_int32), ("max_n", C.c_int64),
                ("max_vals", C.c_int64), ("slots", C.c_int64), ("lens_off", C.c_uint64),
                ("offs_off", C.c_uint64), ("klen", C.c_void_p), ("timeout_ns", C.c_uint64),
                ("state_stride", C.c_int32)]


class PsdevError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = code
        if code < 0:
            msg = ERR_NAMES.get(code, f"psdev error {code}")
        else:
            msg = f"CUDA error {code}"
        super().__init__(f"{what}: {msg}")


_lock = threading.Lock()
_device_lib = None


def _declare(lib: C.CDLL) -> None:
    vp, i32, i64, u64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_size_t
    sig = {
        "psdev_heap_create": (i32, [sz, C.POINTER(vp), C.c_char_p]),
        "psdev_heap_open": (i32, [C.c_char_p, C.POINTER(vp)]),
        "psdev_heap_close": (i32, [vp]),
        "psdev_heap_destroy": (i32, [vp]),
        "psdev_enable_peer": (i32, [i32]),
        "psdev_vmm_supported": (i32, []),
        "psdev_vmm_create": (i32, [sz, C.POINTER(vp), C.POINTER(C.c_int), C.POINTER(sz)]),
        "psdev_vmm_import": (i32, [i32, sz, C.POINTER(vp)]),
        "psdev_vmm_release": (i32, [vp]),
        "psdev_suballoc_new": (vp, [sz]),
        "psdev_suballoc_delete": (None, [vp]),
        "psdev_suballoc_alloc": (i64, [vp, sz, sz]),
        "psdev_suballoc_free": (i32, [vp, i64]),
        "psdev_suballoc_in_use": (sz, [vp]),
        "psdev_channel_status": (i32, [vp, i32, C.POINTER(C.c_int32), C.POINTER(u64)]),
        "psdev_channel_clear": (i32, [vp, i32]),
        "psdev_dense_op": (i32, [C.POINTER(World), C.POINTER(Table), i32, i64, i64,
                                 C.POINTER(Opt), i32, i32, u64, i32, vp]),
        "psdev_dense_op_multi": (i32, [C.POINTER(World), C.POINTER(Table), i32, vp, i32, vp,
                                       C.POINTER(Opt), i32, i32, u64, i32, vp]),
        "psdev_sched_bytes": (sz, [i32]),
        "psdev_launch_count": (u64, []),
        "psdev_ll_bytes": (sz, [i32, i64]),
        "psdev_handle_states": (i32, [i32]),
        "psdev_device_barrier": (i32, [C.POINTER(World), i32, u64, vp]),
        "psdev_multicast_pays": (i32, [i32, u64]),
        "psdev_link_copy": (i32, [vp, vp, sz, i32, vp]),
        "psdev_gemm_bf16": (i32, [vp, vp, vp, i64, i64, i64, i32, u64, vp]),
        "psdev_pull_gemm_bf16": (i32, [C.POINTER(World), C.POINTER(Table), i64, vp, vp, i64, i64,
                                       i64, i32, i32, u64, vp]),
        "psdev_gemm_config": (i32, [i32]),
        "psdev_pull_ring_config": (i32, [i32, i32]),
        "psdev_pull_plan_chunk": (i64, [i64, i64, i32, i32, i32, i64, C.POINTER(C.c_int),
                                        C.POINTER(i64), C.POINTER(i64)]),
        "psdev_gemm_status": (i32, [C.POINTER(C.c_int32)]),
        "psdev_filter_cast": (i32, [vp, vp, i64, C.c_float, i32, vp]),
        "psdev_filter_int8_pack": (i32, [vp, vp, vp, i64, vp]),
        "psdev_filter_int8_unpack": (i32, [vp, vp, vp, i64, i32, vp]),
        "psdev_sort_scratch_bytes": (sz, [i64, i32]),
        "psdev_sort_keys": (i32, [vp, vp, i64, i32, vp, sz, vp]),
        "psdev_sort_status": (i32, [vp, vp]),
        "psdev_ordered_match": (i32, [vp, vp, i64, vp, vp, i64, i32, i32, i32, vp, vp]),
        "psdev_key_shard_lookup": (i32, [vp, i64, u64, i32, vp, vp]),
        "psdev_sparse_scatter": (i32, [C.POINTER(World), C.POINTER(Sparse), i64, i32, vp]),
        "psdev_sparse_apply": (i32, [C.POINTER(World), C.POINTER(Sparse), i32, i32, vp]),
        "psdev_sparse_respond": (i32, [C.POINTER(World), C.POINTER(Sparse), i32, i32, vp]),
        "psdev_lens_to_offsets": (i32, [vp, i64, vp, vp]),
        "psdev_sparse_lens": (i32, [C.POINTER(World), C.POINTER(Sparse), i32, vp]),
    }
    for name, (res, args) in sig.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args


def device_lib() -> C.CDLL:
    """Load (building first if needed) the CUDA data-plane library."""
    global _device_lib
    with _lock:
        if _device_lib is None:
            from . import _build
            checks = os.environ.get("PSB200_DEVICE_CHECKS") == "1"
            path = _build.LIB_DIR / ("libpsb200_device_checks.so" if checks
                                     else "libpsb200_device.so")
            if os.environ.get("PSB200_NO_BUILD") != "1" or not path.exists():
                path = _build.build_device(checks=checks)
            lib = C.CDLL(str(path), mode=C.RTLD_GLOBAL)
            _declare(lib)
            _device_lib = lib
        return _device_lib


def check(code: int, what: str) -> None:
    if code != 0:
        raise PsdevError(int(code), what)
