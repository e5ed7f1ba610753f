"""Thin PyTorch binding: push / pull of torch tensors.

The calls mirror ``KVWorker`` of the reference (include/ps/kv_app.h:54-372): ``push``,
``pull`` and ``push_pull`` return an integer timestamp at once, ``wait(ts)`` blocks until
that request has completed (``KVWorker::Wait``, :233), and the server-side update is
selected per key when the key is declared (the role of ``KVServer::set_request_handle``,
:414-420).  Here a request is a kernel on a CUDA stream instead of messages to server
processes, and completion is a CUDA event plus a device status word.

Tensors may live on the device or in (pinned) host memory.  Host tensors are streamed
through the device in slices: host-to-device copy, fused push/pull kernel and
device-to-host copy of consecutive slices overlap on three streams.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from . import _lib
from .parallel.dense import DenseTable, ServerOptimizer
from .parallel.heap import SymmetricHeap


class Context:
    """Per-process state: rank, device, symmetric heap."""

    def __init__(self, heap_bytes: int = 1 << 30, device: Optional[torch.device] = None,
                 group=None):
        import torch.distributed as dist
        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        if device is None:
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        # host staging buffers and copy threads next to the GPU (matters with several GPUs
        # per host: a pinned buffer on the far socket crosses the inter-socket link)
        from .utils.affinity import bind_to_gpu_cpus
        self.cpus = bind_to_gpu_cpus(self.device.index or 0)
        self.heap = SymmetricHeap(heap_bytes, self.rank, self.world, group=group,
                                  device=self.device)
        self._next_channel = 0
        if self.world > 1:
            dist.barrier(group=group)

    def new_channel(self) -> int:
        c = self._next_channel
        self._next_channel = (c + 1) % (_lib.NUM_CHANNELS - 1)  # last channel: barriers
        return c

    def host_barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)

    def close(self) -> None:
        self.heap.close()


_ctx: Optional[Context] = None


def init(heap_bytes: int = 1 << 30, device=None, group=None) -> Context:
    """Create the process-wide context (``ps::Start`` for the device plane)."""
    global _ctx
    if _ctx is None:
        _ctx = Context(heap_bytes, device, group)
    return _ctx


def finalize() -> None:
    """Release the context (``ps::Finalize``)."""
    global _ctx
    if _ctx is not None:
        _ctx.host_barrier()
        _ctx.close()
        _ctx = None


class KVStore:
    """Dense key-value store over the device data plane."""

    def __init__(self, ctx: Optional[Context] = None, slice_bytes: int = 32 << 20):
        self.ctx = ctx or init()
        self.tables: Dict[int, DenseTable] = {}
        self._events: Dict[int, tuple] = {}
        self._ts = 0
        self.slice_bytes = int(slice_bytes)
        dev = self.ctx.device
        self._h2d = torch.cuda.Stream(dev)
        self._d2h = torch.cuda.Stream(dev)
        self._compute = torch.cuda.Stream(dev)

    # -- declaration -----------------------------------------------------------------------
    def declare(self, key: int, numel: int, *, grad_dtype=torch.float32,
                out_dtype=torch.float32, optimizer: Optional[ServerOptimizer] = None,
                blk: Optional[int] = None, init: Optional[torch.Tensor] = None,
                num_ctas: int = 0) -> DenseTable:
        """Register a dense key of ``numel`` values; same call order on every rank."""
        if key in self.tables:
            raise KeyError(f"key {key} already declared")
        t = DenseTable(self.ctx.heap, numel, grad_dtype, out_dtype, blk=blk,
                       optimizer=optimizer, channel=self.ctx.new_channel(), num_ctas=num_ctas)
        if init is not None:
            t.load_master(init)
        self.tables[key] = t
        return t

    # -- requests ----------------------------------------------------------------------------
    def _new_ts(self, event: torch.cuda.Event, table: DenseTable) -> int:
        self._ts += 1
        self._events[self._ts] = (event, table)
        return self._ts

    def _slices(self, t: DenseTable, itemsize: int):
        step = max(8, (self.slice_bytes // itemsize) & ~7)
        return [(b, min(b + step, t.n)) for b in range(0, t.n, step)]

    def _request(self, key: int, op: int, value: Optional[torch.Tensor],
                 out: Optional[torch.Tensor]) -> int:
        t = self.tables[key]
        cur = torch.cuda.current_stream(self.ctx.device)
        host_in = value is not None and not value.is_cuda
        host_out = out is not None and not out.is_cuda
        if not host_in and not host_out:
            # device path: one kernel on the caller's stream
            if value is not None and value.data_ptr() != t.grad.data_ptr():
                t.grad[: value.numel()].copy_(value.reshape(-1), non_blocking=True)
            t._run(op, 0, None, True, cur, None, True)
            if out is not None and out.data_ptr() != t.weight.data_ptr():
                out.reshape(-1).copy_(t.weight[: out.numel()], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(cur)
            return self._new_ts(ev, t)
        # host path: slice pipeline over three streams
        isz = t.grad.element_size() if op & _lib.OP_PUSH else t.weight.element_size()
        for s in (self._h2d, self._compute, self._d2h):
            s.wait_stream(cur)
        vflat = value.reshape(-1) if value is not None else None
        oflat = out.reshape(-1) if out is not None else None
        first = True
        for b, e in self._slices(t, isz):
            if vflat is not None:
                hi = min(e, vflat.numel())
                if host_in:
                    with torch.cuda.stream(self._h2d):
                        if hi > b:
                            t.grad[b:hi].copy_(vflat[b:hi], non_blocking=True)
                    self._compute.wait_stream(self._h2d)
                elif hi > b:
                    with torch.cuda.stream(self._compute):
                        t.grad[b:hi].copy_(vflat[b:hi], non_blocking=True)
            t._run(op, b, e, True, self._compute, None, first)
            first = False
            if oflat is not None:
                hi = min(e, oflat.numel())
                if hi > b:
                    if host_out:
                        self._d2h.wait_stream(self._compute)
                        with torch.cuda.stream(self._d2h):
                            oflat[b:hi].copy_(t.weight[b:hi], non_blocking=True)
                    else:
                        with torch.cuda.stream(self._compute):
                            oflat[b:hi].copy_(t.weight[b:hi], non_blocking=True)
        ev = torch.cuda.Event()
        self._compute.wait_stream(self._d2h)
        ev.record(self._compute)
        cur.wait_stream(self._compute)
        return self._new_ts(ev, t)

    def push(self, key: int, value: torch.Tensor) -> int:
        """``ZPush``: contribute ``value`` (this worker's gradient) to ``key``."""
        return self._request(key, _lib.OP_PUSH, value, None)

    def pull(self, key: int, out: Optional[torch.Tensor] = None) -> int:
        """``ZPull``: fetch the current value of ``key`` into ``out`` (or ``table.weight``)."""
        return self._request(key, _lib.OP_PULL, None, out)

    def push_pull(self, key: int, value: torch.Tensor, out: Optional[torch.Tensor] = None) -> int:
        """``ZPushPull``: both, in one fused pass per slice."""
        return self._request(key, _lib.OP_PUSHPULL, value, out)

    def wait(self, ts: int) -> None:
        """Block until request ``ts`` completed; raises if a device wait ran out."""
        ev, table = self._events.pop(ts)
        ev.synchronize()
        table.check()

    def wait_all(self) -> None:
        for ts in sorted(self._events):
            self.wait(ts)
