"""Thin PyTorch binding: push / pull of torch tensors through the parameter server.

``init`` is ``ps::Start`` for a GPU job: it starts the host runtime from the ``DMLC_*``
environment (set by this package's launchers, derived from a ``torch.distributed.run`` launch,
or a single process on the loop van), then starts the device plane (``Plane::Start``,
include/ps/device/plane.h): arena handles travel over the control plane, barriers are
``Postoffice::Barrier``; no collective library and no ``torch.distributed`` call is involved.

:class:`KVStore` mirrors ``KVWorker`` of the reference (include/ps/kv_app.h:54-372):
``push``, ``pull`` and ``push_pull`` return an integer timestamp at once, ``wait(ts)`` blocks
until that request has completed (``KVWorker::Wait``, :233), and the server-side update is
selected per key when the key is declared (the role of ``KVServer::set_request_handle``,
:414-420).  The calls ARE ``KVWorker`` calls: a declared tensor is registered with the device
plane under its key, and a request on it leaves ``KVWorker::ZPush/ZPull/ZPushPull`` as copies
and kernels on CUDA streams whose completion credits the worker's request tracker.

Tensors may live on the device or in (pinned) host memory.  Host tensors are streamed
through the device in slices: host-to-device copy, fused push/pull kernel and
device-to-host copy of consecutive slices overlap on three streams.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import numpy as np
import torch

from . import _lib, host
from .parallel.dense import DenseTable, ServerOptimizer
from .parallel.heap import SymmetricHeap

APP_ID = 0


class Context:
    """Per-process state: node rank, device, symmetric heap."""

    def __init__(self, heap_bytes: int = 1 << 30, device: Optional[torch.device] = None,
                 backend: str = "auto", multicast: int = -1, slice_bytes: int = 0,
                 timeout_s: Optional[float] = None):
        from .launch import bootstrap
        self.launch_mode = bootstrap.ensure_env()
        self._own_start = not host.started()
        if self._own_start:
            host.start()
        if host.is_scheduler() and not host.is_worker():
            # a program run by every role, like the reference's tests: the scheduler has
            # nothing to do on the device plane
            host.finalize()
            raise SystemExit(0)
        if device is None:
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK",
                                  os.environ.get("PSB200_LOCAL_INDEX", "0"))) %
                                  max(1, torch.cuda.device_count()))
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        # host staging buffers and copy threads next to the GPU (matters with several GPUs
        # per host: a pinned buffer on the far socket crosses the inter-socket link)
        from .utils.affinity import bind_to_gpu_cpus
        self.cpus = bind_to_gpu_cpus(self.device.index or 0)
        from . import _build
        dev_lib = _lib.device_lib()   # builds if needed; the plane binds the same file
        del dev_lib
        checks = os.environ.get("PSB200_DEVICE_CHECKS") == "1"
        path = _build.LIB_DIR / ("libpsb200_device_checks.so" if checks else "libpsb200_device.so")
        if timeout_s is None:
            from .parallel.dense import default_timeout_s
            timeout_s = default_timeout_s()
        L = host.lib()
        host._ck(L.psnvl_start(int(heap_bytes), int(self.device.index or 0), backend.encode(),
                               int(multicast), str(path).encode(), int(slice_bytes),
                               int(timeout_s * 1e9)))
        self.rank, self.world = int(L.psnvl_rank()), int(L.psnvl_world())
        self.heap = SymmetricHeap(heap_bytes, device=self.device, backend="plane")
        self.worker = L.ps_capi_bworker_new(APP_ID, 0)
        if not self.worker:
            raise host.PSError(L.ps_capi_last_error().decode())

    def new_channel(self) -> int:
        """A rendezvous channel for one more tensor; raises when all are taken."""
        return host._ck(host.lib().psnvl_new_channel())

    def host_barrier(self) -> None:
        """``Postoffice::Barrier`` over the workers."""
        host._ck(host.lib().psnvl_barrier())

    def allgather(self, payload: bytes) -> list:
        """Byte strings of all workers in rank order, over the control plane."""
        L = host.lib()
        sizes = (C.c_size_t * self.world)()
        cap = max(4096, (len(payload) + 64) * self.world * 2)
        for _ in range(2):
            buf = C.create_string_buffer(cap)
            total = L.psnvl_allgather(payload, len(payload), buf, cap, sizes)
            if total < 0:
                raise host.PSError(L.ps_capi_last_error().decode())
            if total <= cap:
                out, at = [], 0
                for r in range(self.world):
                    out.append(buf.raw[at:at + sizes[r]])
                    at += sizes[r]
                return out
            # cannot repeat a collective with a larger buffer: contributions are of one size
            raise ValueError("all-gather contributions differ too much in size")
        return []

    def max_over_ranks(self, value: float) -> float:
        import struct
        if self.world == 1:
            return float(value)
        return max(struct.unpack("<d", b)[0] for b in self.allgather(struct.pack("<d", value)))

    def close(self) -> None:
        L = host.lib()
        # requests that nobody waited for finish before their workers go away
        host._ck(L.psnvl_drain())
        for ks in getattr(self, "_keyed", []):
            ks.close()
        if self.worker:
            L.ps_capi_bworker_delete(self.worker)
            self.worker = None
        self.heap.close()
        torch.cuda.synchronize(self.device)
        host._ck(L.psnvl_stop())
        if self._own_start:
            host.finalize()


_ctx: Optional[Context] = None
_hook_installed = False


def _install_exit_hook() -> None:
    """An uncaught exception in a process that has joined a job ends the process at once, with
    status 1, after the traceback: the orderly exit would wait in ``Finalize`` for peers that
    may be waiting for this process, and the launcher is the one that cleans up a failed job
    (``launch.local`` stops the other nodes; the reference's launcher restarts on code 254)."""
    global _hook_installed
    if _hook_installed:
        return
    _hook_installed = True
    import sys
    import traceback
    prev = sys.excepthook

    def hook(tp, val, tb):
        try:
            traceback.print_exception(tp, val, tb)
            sys.stderr.flush()
            sys.stdout.flush()
        finally:
            if _ctx is not None and tp is not KeyboardInterrupt:
                from .launch import bootstrap
                bootstrap.abandon()
                os._exit(1)
            prev(tp, val, tb)

    sys.excepthook = hook


def init(heap_bytes: int = 1 << 30, device=None, **kw) -> Context:
    """Create the process-wide context (``ps::Start`` plus the device plane)."""
    global _ctx
    if _ctx is None:
        _ctx = Context(heap_bytes, device, **kw)
        _install_exit_hook()
    return _ctx


def context() -> Optional[Context]:
    return _ctx


def finalize() -> None:
    """Release the context (``ps::Finalize``)."""
    global _ctx
    if _ctx is not None:
        _ctx.close()
        _ctx = None


# Requests whose tensors are kept alive without the caller having waited for them; beyond this
# the oldest one is waited for on the caller's behalf.
MAX_UNWAITED = 4096


class KVStore:
    """Dense key-value store over the device data plane."""

    def __init__(self, ctx: Optional[Context] = None, slice_bytes: int = 0):
        self.ctx = ctx or init()
        self.tables: Dict[int, DenseTable] = {}
        self._keys: Dict[int, np.ndarray] = {}
        self._alive: Dict[int, tuple] = {}
        if slice_bytes:
            host._ck(host.lib().psnvl_set_slice_bytes(int(slice_bytes)))

    # -- declaration -----------------------------------------------------------------------
    def declare(self, key: int, numel: int, *, grad_dtype=torch.float32,
                out_dtype=torch.float32, optimizer: Optional[ServerOptimizer] = None,
                blk: Optional[int] = None, init: Optional[torch.Tensor] = None,
                num_ctas: int = 0) -> DenseTable:
        """Register tensor ``key`` of ``numel`` values; same call order on every rank.

        ``key`` is the tensor's id inside every device shard's key range: the tensor is
        addressed by the W keys ``range_j.begin + key`` (:meth:`keys_of`), key j naming the
        j-th of W contiguous pieces.  ``blk`` chooses which rank serves which values: the
        default gives rank j exactly piece j (the reference's contiguous server ranges,
        src/postoffice.cc:169-180); a smaller ``blk`` spreads blocks round-robin."""
        if key in self.tables:
            raise KeyError(f"key {key} already declared")
        t = DenseTable(self.ctx.heap, numel, grad_dtype, out_dtype, blk=blk,
                       optimizer=optimizer, channel=self.ctx.new_channel(), num_ctas=num_ctas)
        if init is not None:
            t.load_master(init)
        L = host.lib()
        o = t.optimizer.to_struct(1)
        host._ck(L.psnvl_register_dense(APP_ID, int(key), int(numel), C.byref(t._table),
                                        C.byref(o), t.channel, int(t.nvls), t.num_ctas))
        keys = np.zeros(self.ctx.world, dtype=np.uint64)
        host._ck(L.psnvl_dense_keys(int(key), keys.ctypes.data_as(C.POINTER(C.c_uint64))))
        self.tables[key] = t
        self._keys[key] = keys
        return t

    def keys_of(self, key: int) -> np.ndarray:
        """The uint64 keys of tensor ``key``, one per device shard."""
        return self._keys[key].copy()

    def set_optimizer(self, key: int, optimizer: ServerOptimizer) -> None:
        """Replace the hyper-parameters of the server handle of ``key`` (e.g. a new rate)."""
        t = self.tables[key]
        t.optimizer = optimizer
        o = optimizer.to_struct(1)
        host._ck(host.lib().psnvl_set_optimizer(APP_ID, int(key), C.byref(o)))

    # -- requests ----------------------------------------------------------------------------
    def _request(self, key: int, push: bool, pull: bool, value: Optional[torch.Tensor],
                 out: Optional[torch.Tensor], cmd: int = 0, priority: int = 0) -> int:
        t = self.tables[key]
        L = host.lib()
        keys = self._keys[key]
        cur = torch.cuda.current_stream(self.ctx.device)
        L.psnvl_set_stream(cur.cuda_stream)
        vptr = vbytes = optr = obytes = 0
        if push:
            if value is None:
                value = t.grad[: t.n_user]
            if not value.is_contiguous() or value.numel() != t.n_user or value.dtype != t.grad_dtype:
                raise ValueError("pushed values must be a contiguous tensor of the declared "
                                 "length and gradient dtype")
            vptr, vbytes = value.data_ptr(), value.numel() * value.element_size()
        if pull:
            if out is None:
                out = t.weight[: t.n_user]
            if not out.is_contiguous() or out.numel() != t.n_user or out.dtype != t.out_dtype:
                raise ValueError("the output must be a contiguous tensor of the declared "
                                 "length and weight dtype")
            optr, obytes = out.data_ptr(), out.numel() * out.element_size()
        ts = L.ps_capi_bworker_request(self.ctx.worker, int(push), int(pull),
                                       keys.ctypes.data_as(C.POINTER(C.c_uint64)), keys.size,
                                       vptr, vbytes, optr, obytes, int(cmd), int(priority))
        if ts < 0:
            raise host.PSError(L.ps_capi_last_error().decode())
        self._alive[ts] = (value, out, t)   # zero-copy: kept until the request completed
        if len(self._alive) > MAX_UNWAITED:
            self.wait(min(self._alive))   # a caller that never waits: retire the oldest
        return ts

    def push(self, key: int, value: Optional[torch.Tensor] = None, publish: bool = False) -> int:
        """``ZPush``: contribute ``value`` (this worker's gradient; default: the tensor's own
        gradient buffer) to ``key``.  ``publish``: owners also leave the new values in their
        own weight buffer, for a pull fused into a GEMM."""
        return self._request(key, True, False, value, None, cmd=0x5055424c if publish else 0)

    def pull(self, key: int, out: Optional[torch.Tensor] = None) -> int:
        """``ZPull``: fetch the current value of ``key`` into ``out`` (or ``table.weight``)."""
        return self._request(key, False, True, None, out)

    def push_pull(self, key: int, value: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> int:
        """``ZPushPull``: both, in one fused pass per slice."""
        return self._request(key, True, True, value, out)

    def wait(self, ts: int) -> None:
        """Block until request ``ts`` completed; raises if a device wait ran out."""
        L = host.lib()
        try:
            if L.ps_capi_bworker_wait(self.ctx.worker, int(ts)) < 0:
                raise host.PSError(L.ps_capi_last_error().decode())
        finally:
            self._alive.pop(ts, None)

    def wait_all(self) -> None:
        for ts in sorted(self._alive):
            self.wait(ts)

    def clear_error(self, key: int) -> None:
        """After a request on ``key`` failed because a peer did not arrive: make the tensor
        usable again.  Collective: every worker calls it."""
        host._ck(host.lib().psnvl_clear_status(APP_ID, int(key)))


class KeyedStore:
    """One keyed (sparse) table of the device plane, reached through a ``KVWorker``: sorted
    unique uint64 keys (int64 bit patterns) and fp32 values in DEVICE memory, ``width`` values
    per key or, with ``var_len``, ``lens[i] <= width`` values per key packed back to back (the
    reference's ``KVPairs`` with ``lens``, include/ps/kv_app.h:24-45).

    Every worker constructs its stores in the same order with the same arguments, and issues the
    same kind of request at the same position of its request sequence (each request carries a
    rendezvous of all workers).  ``kind``: ``"sum"``, ``"sgd"`` (``lr``) or ``"ftrl"``.
    """
    _KINDS = {"sum": 0, "sgd": 1, "ftrl": 2}
    _next_customer = 1

    def __init__(self, ctx: Context, app_id: int, key_space: int, max_keys: int, *,
                 width: int = 1, kind: str = "sum", lr: float = 0.01, alpha: float = 0.05,
                 beta: float = 1.0, l1: float = 0.0, l2: float = 0.0, var_len: bool = False):
        if app_id == APP_ID:
            raise ValueError(f"app {APP_ID} belongs to the dense store")
        self.ctx, self.app_id = ctx, int(app_id)
        self.width, self.var_len, self.max_keys = int(width), bool(var_len), int(max_keys)
        L = host.lib()
        host._ck(L.psnvl_declare_sparse(self.app_id, int(key_space), self.max_keys, self.width,
                                        self._KINDS[kind], lr, alpha, beta, l1, l2,
                                        int(self.var_len)))
        cid = KeyedStore._next_customer
        KeyedStore._next_customer += 1
        self.worker = L.ps_capi_bworker_new(self.app_id, cid)
        if not self.worker:
            raise host.PSError(L.ps_capi_last_error().decode())
        self._alive: Dict[int, tuple] = {}
        if not hasattr(ctx, "_keyed"):
            ctx._keyed = []
        ctx._keyed.append(self)   # closed with the context, before the plane stops

    def _check(self, t: Optional[torch.Tensor], dtype, what: str) -> None:
        if t is not None and not (t.is_cuda and t.is_contiguous() and t.dtype == dtype):
            raise ValueError(f"{what} must be a contiguous {dtype} tensor on the device")

    def request(self, keys: torch.Tensor, vals: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, lens: Optional[torch.Tensor] = None,
                lens_out: Optional[torch.Tensor] = None) -> int:
        """``vals`` given: push; ``out`` given: pull; both: ``ZPushPull``.  Returns a timestamp
        for :meth:`wait`.  The tensors must stay unchanged until then."""
        push, pull = vals is not None, out is not None
        if not (push or pull):
            raise ValueError("nothing to do: give vals, out or both")
        self._check(keys, torch.int64, "keys")
        self._check(vals, torch.float32, "vals")
        self._check(out, torch.float32, "out")
        self._check(lens, torch.int32, "lens")
        self._check(lens_out, torch.int32, "lens_out")
        n = keys.numel()
        if n > self.max_keys:
            raise ValueError("more keys than max_keys")
        if push and self.var_len and (lens is None or lens.numel() != n):
            raise ValueError("a push to a table with lengths names one length per key")
        if not self.var_len and (lens is not None or lens_out is not None):
            raise ValueError("this table holds fixed-width values")
        if lens_out is not None and lens_out.numel() != n:
            raise ValueError("lens_out needs one entry per key")
        L = host.lib()
        L.psnvl_set_stream(torch.cuda.current_stream(self.ctx.device).cuda_stream)
        ts = L.ps_capi_bworker_keyed_request(
            self.worker, int(push), int(pull), keys.data_ptr(), n,
            vals.data_ptr() if push else None, vals.numel() * 4 if push else 0,
            out.data_ptr() if pull else None, out.numel() * 4 if pull else 0,
            lens.data_ptr() if (push and lens is not None) else None,
            lens_out.data_ptr() if (pull and not push and lens_out is not None) else None, 0)
        if ts < 0:
            raise host.PSError(L.ps_capi_last_error().decode())
        self._alive[ts] = (keys, vals, out, lens, lens_out)
        if len(self._alive) > MAX_UNWAITED:
            self.wait(min(self._alive))
        return ts

    def push(self, keys, vals, lens=None) -> int:
        return self.request(keys, vals=vals, lens=lens)

    def pull(self, keys, out, lens_out=None) -> int:
        return self.request(keys, out=out, lens_out=lens_out)

    def push_pull(self, keys, vals, out, lens=None) -> int:
        return self.request(keys, vals=vals, out=out, lens=lens)

    def wait(self, ts: int) -> None:
        L = host.lib()
        try:
            if L.ps_capi_bworker_wait(self.worker, int(ts)) < 0:
                raise host.PSError(L.ps_capi_last_error().decode())
        finally:
            self._alive.pop(ts, None)

    def close(self) -> None:
        if self.worker:
            host._ck(host.lib().psnvl_drain())
            host.lib().ps_capi_bworker_delete(self.worker)
            self.worker = None
            self._alive.clear()
