"""Data-parallel training through the parameter server: gradients are pushed as they are
produced, the server-side optimizer runs on the owners, weights are pulled before the next
forward pass.

The pattern is the one the reference documents for synchronous SGD (docs/overview.md:79-122)
and that its users build on ``KVWorker::Push/Pull`` with per-message priorities
(include/ps/kv_app.h:114-123; priority send queue, src/p3_van.h:12-57).  Here

* all parameters live in one :class:`DenseTable`; a parameter's storage *is* its slice of the
  pulled-weight buffer, so a pull updates the model in place;
* a gradient hook copies (and casts) each gradient into the table's gradient buffer and hands
  its slices to a priority scheduler; slices are at most ``slice_bytes`` long (4 MB by
  default) and their priority is the reverse of the layer order, so the weights the next
  forward pass needs first are exchanged first among the slices that are pending;
* slices are exchanged by fused push+pull kernels on a side stream, overlapping the rest of
  backward: as soon as ``batch_bytes`` (4 MiB by default, ``PSB200_BATCH_BYTES``) of gradients
  are pending, everything pending goes out in ONE launch whose CTAs take the slices in priority
  order, so small tensors share a rendezvous; with ``batch_bytes=0`` every hook launches up to
  ``slices_per_event`` single-slice kernels and the rest waits in the host queue.

Every rank makes the same scheduling decisions because they depend only on the order in which
gradient hooks fire, which is the same on every rank for the same model.
"""
from __future__ import annotations

import heapq
from typing import Iterable, List, Optional, Tuple

import torch

from .. import _lib
from .dense import DenseTable, ServerOptimizer
from .heap import SymmetricHeap


class P3Scheduler:
    """Priority queue of (begin, end) slices of one table; highest priority first, FIFO among
    equal priorities (same order as ``ThreadsafePQueue`` of the host runtime)."""

    def __init__(self, slice_elems: int):
        self.slice_elems = max(8, int(slice_elems) & ~7)
        self._heap: List[Tuple[int, int, int, int]] = []
        self._seq = 0
        self.pending_elems = 0

    def add(self, begin: int, end: int, priority: int) -> int:
        """Cut [begin, end) into slices and queue them; returns the number of slices."""
        n = 0
        b = begin
        while b < end:
            e = min(b + self.slice_elems, end)
            heapq.heappush(self._heap, (-priority, self._seq, b, e))
            self.pending_elems += e - b
            self._seq += 1
            n += 1
            b = e
        return n

    def pop(self) -> Optional[Tuple[int, int, int]]:
        if not self._heap:
            return None
        negp, _, b, e = heapq.heappop(self._heap)
        self.pending_elems -= e - b
        return b, e, -negp

    def __len__(self) -> int:
        return len(self._heap)


class DistributedOptimizer:
    """Server-side optimizer for the parameters of a model, one process per GPU."""

    def __init__(self, params: Iterable[torch.nn.Parameter], heap: SymmetricHeap,
                 optimizer: ServerOptimizer, grad_dtype=torch.bfloat16, blk: int = 4096,
                 slice_bytes: int = 4 << 20, slices_per_event: int = 2, channel: int = 0,
                 num_ctas: int = 32, overlap: bool = True, publish_first: int = 0,
                 nvls: Optional[bool] = None, publish_params=(),
                 batch_bytes: Optional[int] = None):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("no trainable parameters")
        wdt = self.params[0].dtype
        if any(p.dtype != wdt for p in self.params):
            raise ValueError("all parameters must share one dtype")
        self.heap = heap
        self.offsets, off = [], 0
        for p in self.params:
            self.offsets.append(off)
            off += (p.numel() + 7) & ~7
        self.total = off
        self.table = DenseTable(heap, self.total, grad_dtype, wdt, blk=blk, optimizer=optimizer,
                                channel=channel, num_ctas=num_ctas, nvls=nvls)
        gsz = torch.empty((), dtype=grad_dtype).element_size()
        self.sched = P3Scheduler(slice_bytes // gsz)
        self.slices_per_event = slices_per_event
        # gradients wait in the queue until `batch_bytes` are pending, then everything pending
        # goes out in one launch (small tensors share a rendezvous); 0 = launch from every hook
        if batch_bytes is None:
            import os
            batch_bytes = int(os.environ.get("PSB200_BATCH_BYTES", str(4 << 20)))
        self.batch_bytes = int(batch_bytes)
        self._gsz = gsz
        self.launches = 0
        self.overlap = overlap
        self.comm = torch.cuda.Stream(heap.device) if overlap else None
        # the first `publish_first` parameters are pushed with publish instead of push+pull:
        # their weights are pulled by a GEMM-fused pull in the next forward pass
        self.publish_first = publish_first
        pub = {id(p) for p in publish_params}
        self._publish = [i < publish_first or id(p) in pub for i, p in enumerate(self.params)]
        self.steps = 0
        self.launched_slices = 0
        # initial weights: rank 0's values, installed through an "assign" push
        full = torch.zeros(self.total, dtype=torch.float32, device=heap.device)
        for p, o in zip(self.params, self.offsets):
            full[o:o + p.numel()] = p.detach().reshape(-1).float()
        heap.broadcast(full, 0)
        self.table.load_master(full)
        self.table.pull()
        torch.cuda.synchronize(heap.device)
        # a parameter's storage is its slice of the pulled-weight buffer
        for p, o in zip(self.params, self.offsets):
            p.data = self.table.weight[o:o + p.numel()].view(p.shape)
        self._hooks = [p.register_post_accumulate_grad_hook(self._make_hook(i))
                       for i, p in enumerate(self.params)]
        self._pending_step = False

    def _make_hook(self, index: int):
        n_params = len(self.params)

        o = self.offsets[index]
        n = self.params[index].numel()
        # the parameter's slice of the gradient buffer, in the parameter's shape (made once: the
        # hook runs on the autograd thread, between the kernels of the backward pass)
        gview = self.table.grad[o:o + n].view(self.params[index].shape)

        def hook(p: torch.nn.Parameter):
            gview.copy_(p.grad, non_blocking=True)
            p.grad = None
            if not self._pending_step:
                self._pending_step = True
                self.table.step = self.steps + 1
            # reverse layer order: parameter 0 (needed first by the next forward) is most urgent
            pri = n_params - index
            if self._publish[index]:
                pri = -1 - index  # published slices carry no pull: least urgent
            self.sched.add(o, o + ((n + 7) & ~7), pri)
            if self.batch_bytes <= 0:
                self._launch(self.slices_per_event)
            elif self.sched.pending_elems * self._gsz >= self.batch_bytes:
                self._drain()
        return hook

    def _launch(self, count: int) -> None:
        if count <= 0 or not len(self.sched):
            return
        cur = torch.cuda.current_stream(self.heap.device)
        stream = self.comm or cur
        if self.comm is not None:
            self.comm.wait_stream(cur)
        for _ in range(count):
            item = self.sched.pop()
            if item is None:
                break
            b, e, pri = item
            if pri < 0:
                self.table.push(b, e, stream=stream, opt_step=False, publish=True)
            else:
                self.table.push_pull(b, e, stream=stream, opt_step=False)
            self.launched_slices += 1
            self.launches += 1

    def _drain(self) -> None:
        """Everything queued goes out in one launch per kind of operation; the kernel itself
        takes the slices in priority order (device-side schedule)."""
        if not len(self.sched):
            return
        cur = torch.cuda.current_stream(self.heap.device)
        stream = self.comm or cur
        if self.comm is not None:
            self.comm.wait_stream(cur)
        both, publish = [], []
        while True:
            item = self.sched.pop()
            if item is None:
                break
            (publish if item[2] < 0 else both).append(item)
        cap = self.table.MAX_SEGS
        if len(both) == 1:
            b, e, _ = both[0]
            self.table.push_pull(b, e, stream=stream, opt_step=False)
            self.launches += 1
        else:
            for i in range(0, len(both), cap):
                self.table.run_multi(_lib.OP_PUSHPULL, both[i:i + cap], stream=stream)
                self.launches += 1
        for i in range(0, len(publish), cap):
            self.table.run_multi(_lib.OP_PUSH | _lib.OP_PUBLISH, publish[i:i + cap], stream=stream)
            self.launches += 1
        self.launched_slices += len(both) + len(publish)

    def step(self) -> None:
        """Finish the exchange of this step's gradients; afterwards the parameters hold the
        weights for the next forward pass (except published ones, which their GEMM pulls)."""
        self._drain()
        if self.comm is not None:
            torch.cuda.current_stream(self.heap.device).wait_stream(self.comm)
        self.steps += 1
        self._pending_step = False

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None

    def check(self) -> None:
        self.table.check()

    def close(self) -> None:
        """Detach from the model and give the table's buffers back to the heap.  The
        parameters keep pointing at the pulled-weight buffer: drop the model too."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        torch.cuda.synchronize(self.heap.device)
        self.table.free()

    def offset_of(self, param: torch.nn.Parameter) -> int:
        for p, o in zip(self.params, self.offsets):
            if p is param:
                return o
        raise KeyError("parameter not managed by this optimizer")
