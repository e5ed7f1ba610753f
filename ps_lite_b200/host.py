"""Python binding of the host runtime (``libpsb200_core.so`` through ``src/capi/ps_c_api.h``).

The functions and classes mirror the C++ API of ``include/ps/ps.h``: ``start``/``finalize``,
role queries, ``barrier``, :class:`KVWorker` (``push``/``pull``/``push_pull``/``wait``),
:class:`KVServer` with the built-in accumulate handle or a Python request handle, and
:class:`SimpleApp`.  Values are float32; keys are uint64 and must be sorted and unique.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
import threading
from typing import Callable, Optional

import numpy as np

_lock = threading.Lock()
_lib = None

SCHEDULER, SERVER_GROUP, WORKER_GROUP = 1, 2, 4
ALL = SCHEDULER + SERVER_GROUP + WORKER_GROUP


class Request(C.Structure):
    _fields_ = [("cmd", C.c_int), ("push", C.c_int), ("pull", C.c_int), ("sender", C.c_int),
                ("timestamp", C.c_int), ("customer_id", C.c_int),
                ("keys", C.POINTER(C.c_uint64)), ("nkeys", C.c_size_t),
                ("vals", C.POINTER(C.c_float)), ("nvals", C.c_size_t),
                ("lens", C.POINTER(C.c_int)), ("nlens", C.c_size_t)]


class _Node(C.Structure):
    _fields_ = [("role", C.c_int), ("id", C.c_int), ("port", C.c_int),
                ("is_recovery", C.c_int), ("customer_id", C.c_int), ("hostname", C.c_char * 64)]


class MetaStruct(C.Structure):
    _fields_ = [("head", C.c_int), ("app_id", C.c_int), ("customer_id", C.c_int),
                ("timestamp", C.c_int), ("request", C.c_int), ("push", C.c_int),
                ("pull", C.c_int), ("simple_app", C.c_int), ("priority", C.c_int),
                ("control_cmd", C.c_int), ("barrier_group", C.c_int), ("msg_sig", C.c_uint64),
                ("num_data_types", C.c_int), ("data_types", C.c_int * 8),
                ("num_nodes", C.c_int), ("nodes", _Node * 8),
                ("body", C.c_char * 256), ("body_len", C.c_int)]


HANDLE = C.CFUNCTYPE(None, C.c_void_p, C.POINTER(Request), C.c_void_p)
SIMPLE_HANDLE = C.CFUNCTYPE(None, C.c_int, C.POINTER(C.c_char), C.c_size_t, C.c_int, C.c_void_p)


def lib() -> C.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            from . import _build
            path = _build.build_core()
            L = C.CDLL(str(path))   # local scope: nothing else resolves against this library
            vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
            u64p, fp, ip = C.POINTER(C.c_uint64), C.POINTER(C.c_float), C.POINTER(C.c_int)
            L.ps_capi_last_error.restype = C.c_char_p
            L.ps_capi_setenv.argtypes = [C.c_char_p, C.c_char_p]
            L.ps_capi_dead_nodes.argtypes = [i, ip, i]
            L.ps_capi_server_key_range.argtypes = [i, u64p, u64p]
            L.ps_capi_traffic.argtypes = [u64p, u64p]
            L.ps_capi_shm_stats.argtypes = [C.POINTER(C.c_uint64 * 6)]
            L.ps_capi_worker_new.restype = vp
            L.ps_capi_worker_new.argtypes = [i, i]
            L.ps_capi_worker_delete.argtypes = [vp]
            L.ps_capi_worker_push.argtypes = [vp, u64p, sz, fp, sz, ip, sz, i, i]
            L.ps_capi_worker_pull.argtypes = [vp, u64p, sz, fp, sz, ip, sz, i, i]
            L.ps_capi_worker_push_pull.argtypes = [vp, u64p, sz, fp, sz, fp, ip, sz, i, i]
            L.ps_capi_worker_wait.argtypes = [vp, i]
            L.ps_capi_server_new.restype = vp
            L.ps_capi_server_new.argtypes = [i, vp, vp]
            L.ps_capi_server_delete.argtypes = [vp]
            L.ps_capi_server_respond.argtypes = [vp, C.POINTER(Request), u64p, sz, fp, sz, ip, sz]
            L.ps_capi_simple_new.restype = vp
            L.ps_capi_simple_new.argtypes = [i, i, vp, vp]
            L.ps_capi_simple_delete.argtypes = [vp]
            L.ps_capi_simple_request.argtypes = [vp, i, C.c_char_p, sz, i]
            L.ps_capi_simple_wait.argtypes = [vp, i]
            L.ps_capi_encode_meta.restype = C.c_long
            L.ps_capi_encode_meta.argtypes = [C.POINTER(MetaStruct), C.c_char_p, sz]
            L.ps_capi_decode_meta.argtypes = [C.c_char_p, sz, C.POINTER(MetaStruct)]
            # device plane (src/capi/ps_nvl_c_api.h)
            from ._lib import Opt, Table, World
            u64, i64 = C.c_uint64, C.c_int64
            L.psnvl_start.argtypes = [u64, i, C.c_char_p, i, C.c_char_p, u64, u64]
            L.psnvl_backend.restype = C.c_char_p
            L.psnvl_world_struct.argtypes = [C.POINTER(World)]
            L.psnvl_allgather.restype = C.c_long
            L.psnvl_allgather.argtypes = [C.c_char_p, sz, C.c_char_p, sz, C.POINTER(sz)]
            L.psnvl_alloc.restype = i64
            L.psnvl_alloc.argtypes = [u64, u64]
            L.psnvl_free.argtypes = [i64]
            L.psnvl_heap_in_use.restype = u64
            L.psnvl_register_dense.argtypes = [i, u64, i64, C.POINTER(Table), C.POINTER(Opt), i,
                                               i, i]
            L.psnvl_unregister_dense.argtypes = [i, u64]
            L.psnvl_set_optimizer.argtypes = [i, u64, C.POINTER(Opt)]
            L.psnvl_dense_keys.argtypes = [u64, u64p]
            L.psnvl_set_stream.argtypes = [vp]
            L.psnvl_set_slice_bytes.argtypes = [u64]
            L.psnvl_clear_status.argtypes = [i, u64]
            L.psnvl_launches.restype = u64
            L.ps_capi_bworker_new.restype = vp
            L.ps_capi_bworker_new.argtypes = [i, i]
            L.ps_capi_bworker_delete.argtypes = [vp]
            L.ps_capi_bworker_request.argtypes = [vp, i, i, u64p, sz, vp, sz, vp, sz, i, i]
            L.ps_capi_bworker_wait.argtypes = [vp, i]
            f32 = C.c_float
            L.psnvl_declare_sparse.argtypes = [i, u64, i64, i, i, f32, f32, f32, f32, f32, i]
            L.ps_capi_bworker_keyed_request.argtypes = [vp, i, i, vp, sz, vp, sz, vp, sz, vp, vp, i]
            _lib = L
        return _lib


class PSError(RuntimeError):
    pass


def _ck(rc: int) -> int:
    if rc < 0:
        raise PSError(lib().ps_capi_last_error().decode(errors="replace"))
    return rc


def setenv(key: str, value) -> None:
    _ck(lib().ps_capi_setenv(key.encode(), str(value).encode()))


_started = False


_exit_hook = False


def _leave_without_finalize() -> None:
    """Interpreter exit of a process that started the runtime and never finalized it (an uncaught
    exception, an early ``sys.exit``): stop this node's van without the closing barrier, so that
    the process ends with its own exit status instead of blocking in the destruction of a runtime
    whose threads still run.  The other nodes of the job are the launcher's business."""
    global _started
    if _started:
        _started = False
        try:
            lib().ps_capi_finalize(0, 0)
        except Exception:
            pass


def start(customer_id: int = 0, barrier: bool = True) -> None:
    global _started, _exit_hook
    _ck(lib().ps_capi_start(customer_id, int(barrier)))
    _started = True
    if not _exit_hook:
        import atexit
        atexit.register(_leave_without_finalize)
        _exit_hook = True


def finalize(customer_id: int = 0, barrier: bool = True) -> None:
    global _started
    _ck(lib().ps_capi_finalize(customer_id, int(barrier)))
    if customer_id == 0:
        _started = False


def started() -> bool:
    return _started


def barrier(group: int = ALL, customer_id: int = 0) -> None:
    _ck(lib().ps_capi_barrier(customer_id, group))


def num_workers() -> int: return lib().ps_capi_num_workers()
def num_servers() -> int: return lib().ps_capi_num_servers()
def my_rank() -> int: return _ck(lib().ps_capi_my_rank())
def is_worker() -> bool: return bool(lib().ps_capi_is_worker())
def is_server() -> bool: return bool(lib().ps_capi_is_server())
def is_scheduler() -> bool: return bool(lib().ps_capi_is_scheduler())
def is_recovery() -> bool: return bool(_ck(lib().ps_capi_is_recovery()))


def dead_nodes(timeout_s: int = 60) -> list[int]:
    buf = (C.c_int * 64)()
    n = _ck(lib().ps_capi_dead_nodes(timeout_s, buf, 64))
    return [buf[i] for i in range(min(n, 64))]


def server_key_range(rank: int) -> tuple[int, int]:
    b, e = C.c_uint64(), C.c_uint64()
    _ck(lib().ps_capi_server_key_range(rank, C.byref(b), C.byref(e)))
    return b.value, e.value


def traffic() -> tuple[int, int]:
    s, r = C.c_uint64(), C.c_uint64()
    _ck(lib().ps_capi_traffic(C.byref(s), C.byref(r)))
    return s.value, r.value


def shm_stats() -> dict:
    """Counters of the shared-memory array pool (large arrays between processes of one host)."""
    out = (C.c_uint64 * 6)()
    _ck(lib().ps_capi_shm_stats(C.byref(out)))
    names = ("segments_created", "segments_reused", "bytes_live", "bytes_pooled",
             "segments_received", "segments_received_already_mapped")
    return dict(zip(names, (int(v) for v in out)))


def _u64(a): return np.ascontiguousarray(a, dtype=np.uint64)
def _f32(a): return np.ascontiguousarray(a, dtype=np.float32)
def _i32(a): return np.ascontiguousarray(a, dtype=np.int32)
def _p(a, t): return a.ctypes.data_as(C.POINTER(t)) if a is not None and a.size else None


class KVWorker:
    """``KVWorker<float>`` (include/ps/kv_app.h)."""

    def __init__(self, app_id: int = 0, customer_id: int = 0):
        self._h = lib().ps_capi_worker_new(app_id, customer_id)
        if not self._h:
            raise PSError(lib().ps_capi_last_error().decode())
        self._alive = {}

    def push(self, keys, vals, lens=None, cmd: int = 0, priority: int = 0) -> int:
        k, v = _u64(keys), _f32(vals)
        l = _i32(lens) if lens is not None else None
        return _ck(lib().ps_capi_worker_push(self._h, _p(k, C.c_uint64), k.size,
                                             _p(v, C.c_float), v.size,
                                             _p(l, C.c_int), 0 if l is None else l.size,
                                             cmd, priority))

    def pull(self, keys, out: np.ndarray, lens_out: Optional[np.ndarray] = None, cmd: int = 0,
             priority: int = 0) -> int:
        k = _u64(keys)
        assert out.dtype == np.float32 and out.flags["C_CONTIGUOUS"]
        ts = _ck(lib().ps_capi_worker_pull(self._h, _p(k, C.c_uint64), k.size,
                                           _p(out, C.c_float), out.size,
                                           _p(lens_out, C.c_int),
                                           0 if lens_out is None else lens_out.size,
                                           cmd, priority))
        self._alive[ts] = (out, lens_out)
        return ts

    def push_pull(self, keys, vals, out: np.ndarray, lens=None, cmd: int = 0,
                  priority: int = 0) -> int:
        k, v = _u64(keys), _f32(vals)
        assert out.dtype == np.float32 and out.size == v.size
        l = _i32(lens) if lens is not None else None
        ts = _ck(lib().ps_capi_worker_push_pull(self._h, _p(k, C.c_uint64), k.size,
                                                _p(v, C.c_float), v.size, _p(out, C.c_float),
                                                _p(l, C.c_int), 0 if l is None else l.size,
                                                cmd, priority))
        self._alive[ts] = (out, l)
        return ts

    def wait(self, ts: int) -> None:
        _ck(lib().ps_capi_worker_wait(self._h, ts))
        self._alive.pop(ts, None)

    def close(self) -> None:
        if self._h:
            lib().ps_capi_worker_delete(self._h)
            self._h = None


def _handle_failed(what: str) -> None:
    """A Python handle raised on the runtime's receive thread.  The request it was serving will
    never be answered, so the requester would wait for ever: the process reports the error and
    ends with status 1, like a C++ handle that throws, and the launcher ends the job."""
    import traceback
    sys.stderr.write(f"ps_lite_b200: {what} raised; the process ends\n")
    traceback.print_exc()
    sys.stderr.flush()
    os._exit(1)


class KVServer:
    """``KVServer<float>``; ``handle(server, req)`` is a Python request handle, or None for the
    built-in accumulate handle.  A Python handle must call ``server.respond(req, ...)``."""

    def __init__(self, app_id: int = 0, handle: Optional[Callable] = None):
        self._py = handle
        self._cb = HANDLE(self._tramp) if handle else None
        self._h = lib().ps_capi_server_new(app_id, C.cast(self._cb, C.c_void_p) if handle else None,
                                           None)
        if not self._h:
            raise PSError(lib().ps_capi_last_error().decode())

    def _tramp(self, _server, reqp, _user):
        req = reqp.contents
        view = {
            "cmd": req.cmd, "push": bool(req.push), "pull": bool(req.pull),
            "sender": req.sender, "timestamp": req.timestamp, "customer_id": req.customer_id,
            "keys": np.ctypeslib.as_array(req.keys, (req.nkeys,)).copy() if req.nkeys else np.zeros(0, np.uint64),
            "vals": np.ctypeslib.as_array(req.vals, (req.nvals,)).copy() if req.nvals else np.zeros(0, np.float32),
            "lens": np.ctypeslib.as_array(req.lens, (req.nlens,)).copy() if req.nlens else np.zeros(0, np.int32),
            "_raw": Request.from_buffer_copy(req),
        }
        try:
            self._py(self, view)
        except BaseException:  # noqa: BLE001 - nothing above this frame can handle it
            _handle_failed("KVServer request handle")

    def respond(self, req: dict, keys=None, vals=None, lens=None) -> None:
        k = _u64(keys) if keys is not None else None
        v = _f32(vals) if vals is not None else None
        l = _i32(lens) if lens is not None else None
        _ck(lib().ps_capi_server_respond(self._h, C.byref(req["_raw"]),
                                         _p(k, C.c_uint64), 0 if k is None else k.size,
                                         _p(v, C.c_float), 0 if v is None else v.size,
                                         _p(l, C.c_int), 0 if l is None else l.size))

    def close(self) -> None:
        if self._h:
            lib().ps_capi_server_delete(self._h)
            self._h = None


class SimpleApp:
    def __init__(self, app_id: int = 0, customer_id: int = 0, on_request: Optional[Callable] = None):
        self._py = on_request
        self._cb = SIMPLE_HANDLE(self._tramp) if on_request else None
        self._h = lib().ps_capi_simple_new(app_id, customer_id,
                                           C.cast(self._cb, C.c_void_p) if on_request else None, None)
        if not self._h:
            raise PSError(lib().ps_capi_last_error().decode())

    def _tramp(self, head, body, n, sender, _user):
        try:
            self._py(head, C.string_at(body, n), sender)
        except BaseException:  # noqa: BLE001
            _handle_failed("SimpleApp request handle")

    def request(self, head: int, body: bytes, recver: int) -> int:
        return _ck(lib().ps_capi_simple_request(self._h, head, body, len(body), recver))

    def wait(self, ts: int) -> None:
        _ck(lib().ps_capi_simple_wait(self._h, ts))

    def close(self) -> None:
        if self._h:
            lib().ps_capi_simple_delete(self._h)
            self._h = None


def encode_meta(**fields) -> bytes:
    m = MetaStruct()
    EMPTY = 2**31 - 1
    m.head = m.app_id = m.customer_id = m.timestamp = EMPTY
    nodes = fields.pop("nodes", [])
    dts = fields.pop("data_types", [])
    body = fields.pop("body", b"")
    for k, v in fields.items():
        setattr(m, k, int(v))
    m.num_data_types = len(dts)
    for i, d in enumerate(dts):
        m.data_types[i] = d
    m.num_nodes = len(nodes)
    for i, n in enumerate(nodes):
        m.nodes[i].role, m.nodes[i].id, m.nodes[i].port = n["role"], n["id"], n["port"]
        m.nodes[i].is_recovery, m.nodes[i].customer_id = int(n.get("is_recovery", 0)), n.get("customer_id", 0)
        m.nodes[i].hostname = n["hostname"].encode()
    if len(body) > 255:
        raise ValueError("body longer than 255 bytes")
    C.memmove(C.addressof(m) + MetaStruct.body.offset, body, len(body))
    m.body_len = len(body)
    buf = C.create_string_buffer(4096)
    n = _ck(lib().ps_capi_encode_meta(C.byref(m), buf, 4096))
    return buf.raw[:n]


def decode_meta(data: bytes) -> MetaStruct:
    m = MetaStruct()
    _ck(lib().ps_capi_decode_meta(data, len(data), C.byref(m)))
    return m
