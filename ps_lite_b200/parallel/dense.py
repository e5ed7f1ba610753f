"""Dense key-value tables on the device data plane.

A :class:`DenseTable` is the device form of a set of ``(key -> fixed-length value)`` pairs
pushed and pulled by every worker (reference: ``KVWorker::ZPush/ZPull/ZPushPull``,
include/ps/kv_app.h:243-306, with the values of key block ``j`` owned by server
``j % num_servers``; the reference's uniform contiguous ranges, src/postoffice.cc:169-180,
are the special case ``blk = ceil(n / num_servers)``).

Worker side (in the symmetric heap, same offset on every rank): ``grad`` and ``weight``.
Server side (local memory): fp32 ``master`` and optimizer state for the owned blocks.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import math
from typing import Optional

import torch

from .. import _lib
from .heap import SymmetricHeap

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.int8: _lib.I8}


@dataclasses.dataclass
class ServerOptimizer:
    """Server-side request handle applied to pushed gradients (fused into the push kernel).

    ``kind``: ``"sum"`` (the reference's ``KVServerDefaultHandle``: ``store += val``,
    include/ps/kv_app.h:440-463), ``"assign"``, ``"sgd"``, ``"momentum"``, ``"adam"``,
    ``"adamw"``, or ``"user"`` with ``user_kind`` >= 100 for a handle that the application
    compiled and registered itself (include/ps/device/user_handle.cuh); ``user`` then carries
    up to four extra hyper-parameters of that handle.
    """
    kind: str = "sum"
    lr: float = 0.01
    momentum: float = 0.9
    weight_decay: float = 0.0
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    scale: float = 1.0  # multiplies the sum over workers (use 1/world to average)
    user_kind: int = 0
    user: tuple = ()

    _KINDS = {"sum": _lib.OPT_SUM, "assign": _lib.OPT_ASSIGN, "sgd": _lib.OPT_SGD,
              "momentum": _lib.OPT_MOMENTUM, "adam": _lib.OPT_ADAM, "adamw": _lib.OPT_ADAM}

    @property
    def num_states(self) -> int:
        if self.kind == "user":
            n = int(_lib.device_lib().psdev_handle_states(int(self.user_kind)))
            if n < 0:
                raise ValueError(f"no handle is registered as kind {self.user_kind}: load the "
                                 "shared object that defines it first")
            return n
        return {"momentum": 1, "adam": 2, "adamw": 2}.get(self.kind, 0)

    def to_struct(self, step: int = 1) -> _lib.Opt:
        o = _lib.Opt()
        o.kind = int(self.user_kind) if self.kind == "user" else self._KINDS[self.kind]
        for i, v in enumerate(self.user[:4]):
            o.user[i] = float(v)
        o.scale, o.lr, o.momentum, o.weight_decay = self.scale, self.lr, self.momentum, self.weight_decay
        o.beta1, o.beta2, o.eps = self.beta1, self.beta2, self.eps
        o.bias1 = 1.0 - self.beta1 ** step
        o.bias2 = math.sqrt(1.0 - self.beta2 ** step)
        o.decoupled_wd = 1 if self.kind == "adamw" else 0
        return o


def default_timeout_s() -> float:
    import os
    return float(os.environ.get("PSB200_DEVICE_TIMEOUT_S", "20"))


_NVTX = None
_OP_NAMES = {1: "ps.push", 2: "ps.pull", 3: "ps.push_pull", 5: "ps.push_publish"}


def _nvtx_enabled() -> bool:
    """NVTX ranges around every request when PSB200_NVTX=1 (for timeline tools)."""
    global _NVTX
    if _NVTX is None:
        import os
        _NVTX = os.environ.get("PSB200_NVTX") == "1"
    return _NVTX


class DenseTable:
    """``n`` values sharded block-cyclically over the ranks of ``heap``.

    Every rank must construct its tables in the same order with the same arguments.
    """

    def __init__(self, heap: SymmetricHeap, n: int, grad_dtype=torch.float32,
                 out_dtype=torch.float32, blk: Optional[int] = None,
                 optimizer: Optional[ServerOptimizer] = None, channel: int = 0,
                 num_ctas: int = 0, nvls: Optional[bool] = None, ll_cap: Optional[int] = None):
        self.heap = heap
        W = heap.world
        self.n_user = int(n)
        # int8 gradients carry one scale per 256 values: everything is aligned to 256 then
        align = 256 if grad_dtype == torch.int8 else 8
        self.n = (int(n) + align - 1) // align * align
        if blk is None:  # contiguous ranges, one per server
            blk = (self.n + W - 1) // W
        self.blk = max(align, (int(blk) + align - 1) // align * align)
        self.nblocks = (self.n + self.blk - 1) // self.blk
        self.local_blocks = (self.nblocks + W - 1) // W
        self.local_len = self.local_blocks * self.blk
        self.grad_dtype, self.out_dtype = grad_dtype, out_dtype
        self.optimizer = optimizer or ServerOptimizer("sum")
        self.channel, self.num_ctas = int(channel), int(num_ctas)
        self.step = 0
        self._opt_key, self._opt_cached = None, None
        self._default_timeout = default_timeout_s()
        # NVSwitch multicast path: on by default from four ranks up when the heap has a
        # multicast alias (with two ranks plain peer accesses move fewer bytes per link)
        if nvls is None:
            import os
            env = os.environ.get("PSB200_NVLS")
            nvls = (W >= 4) if env is None else (env == "1")
        self.nvls = bool(nvls and heap.mc_base and W > 1)
        # largest request that takes the multicast path; None = the library's measured rule
        # (psdev_multicast_pays: 4 MiB with up to 4 ranks, 512 MiB with more)
        self.nvls_max_bytes: Optional[int] = None
        gsz = torch.empty((), dtype=grad_dtype).element_size()
        osz = torch.empty((), dtype=out_dtype).element_size()
        self.grad_off = heap.alloc(self.n * gsz)
        self.weight_off = heap.alloc(self.n * osz)
        self.grad = heap.tensor(self.grad_off, self.n, grad_dtype)
        self.weight = heap.tensor(self.weight_off, self.n, out_dtype)
        self.gscale_off, self.gscale = 0, None
        if grad_dtype == torch.int8:
            self.gscale_off = heap.alloc(4 * (self.n // 256))
            self.gscale = heap.tensor(self.gscale_off, self.n // 256, torch.float32)
            self.gscale.fill_(1.0)
        dev = heap.device
        self.master = torch.zeros(self.local_len, dtype=torch.float32, device=dev)
        ns = self.optimizer.num_states
        self.state1 = torch.zeros(self.local_len, dtype=torch.float32, device=dev) if ns >= 1 else None
        self.state2 = torch.zeros(self.local_len, dtype=torch.float32, device=dev) if ns >= 2 else None
        self._world = heap.world_struct()
        self._table = _lib.Table()
        t = self._table
        t.grad_off, t.weight_off, t.n, t.blk = self.grad_off, self.weight_off, self.n, self.blk
        t.master = self.master.data_ptr()
        t.state1 = self.state1.data_ptr() if self.state1 is not None else None
        t.state2 = self.state2.data_ptr() if self.state2 is not None else None
        t.grad_dtype, t.out_dtype = _DT[grad_dtype], _DT[out_dtype]
        t.gscale_off = self.gscale_off
        self.grad.zero_()
        self.weight.zero_()
        # Low-latency region for small fused requests (include/ps/device/push_pull_ll.cuh):
        # up to `ll_cap` values per request travel next to a sequence number instead of between
        # two flag rendezvous.  Needs real ranks (kernels of all ranks run at the same time).
        if ll_cap is None:
            import os
            ll_cap = int(os.environ.get("PSB200_LL_CAP", str(128 << 10)))
        self.ll_cap = 0
        if W > 1 and ll_cap > 0 and grad_dtype != torch.int8 and not heap.emulated_ranks:
            self.ll_cap = min(int(ll_cap), self.n)
            nb = int(heap.lib.psdev_ll_bytes(W, self.ll_cap))
            self.ll_off = heap.alloc(nb)
            heap.tensor(self.ll_off, nb, torch.uint8).zero_()
            t.ll_off, t.ll_cap = self.ll_off, self.ll_cap
            # nobody writes into a peer's region before that peer has cleared it
            heap.barrier()

    def free(self) -> None:
        """Give the table's heap buffers back (every rank, in the same order as the other
        ranks' calls); the table must not be used afterwards."""
        for off in (self.grad_off, self.weight_off, self.gscale_off,
                    getattr(self, "ll_off", 0)):
            if off:
                self.heap.free(off)
        self.grad_off = self.weight_off = self.gscale_off = self.ll_off = 0

    def stage_int8(self, grad: torch.Tensor, begin: int = 0) -> None:
        """Compress an fp32 gradient into this table's int8 gradient buffer starting at element
        ``begin`` (a multiple of 256): values plus one scale per 256 (the block-scale filter)."""
        if self.gscale is None:
            raise TypeError("table was not created with grad_dtype=torch.int8")
        if begin % 256:
            raise ValueError("begin must be a multiple of 256")
        g = grad.reshape(-1).contiguous()
        s = torch.cuda.current_stream(self.heap.device)
        rc = self.heap.lib.psdev_filter_int8_pack(
            g.data_ptr(), self.grad[begin:].data_ptr(), self.gscale[begin // 256:].data_ptr(),
            g.numel(), s.cuda_stream)
        _lib.check(rc, "psdev_filter_int8_pack")

    # -- ownership helpers (host math mirrored by the kernels) ------------------------------
    def owner_of(self, i: int) -> int:
        return (i // self.blk) % self.heap.world

    def owned_index(self) -> torch.Tensor:
        """Global element indices of the values this rank owns, in state order."""
        W, R = self.heap.world, self.heap.rank
        if R >= self.nblocks:   # fewer blocks than ranks: this rank serves none
            return torch.empty(0, dtype=torch.int64, device=self.heap.device)
        blocks = torch.arange(R, self.nblocks, W, device=self.heap.device)
        idx = blocks[:, None] * self.blk + torch.arange(self.blk, device=self.heap.device)[None, :]
        return idx.reshape(-1)

    def load_master(self, full: torch.Tensor) -> None:
        """Initialise the owned part of the master weights from a full fp32 vector."""
        idx = self.owned_index()
        valid = idx < min(self.n_user, full.numel())
        flat = full.reshape(-1).to(self.heap.device, torch.float32)
        self.master.zero_()
        self.master[: idx.numel()][valid] = flat[idx[valid]]

    def gather_master(self, out: torch.Tensor) -> None:
        """Scatter the owned master values into a full-size fp32 vector (others untouched)."""
        idx = self.owned_index()
        valid = idx < min(self.n_user, out.numel())
        out.reshape(-1)[idx[valid]] = self.master[: idx.numel()][valid]

    # -- operations ---------------------------------------------------------------------------
    def _run(self, op: int, begin: int, end: Optional[int], sync: bool,
             stream: Optional[torch.cuda.Stream], timeout_s: Optional[float], opt_step: bool):
        end = self.n if end is None else end
        if op & _lib.OP_PUSH and opt_step:
            self.step += 1
        o = self._opt_struct()
        s = stream or torch.cuda.current_stream(self.heap.device)
        tmo = int((timeout_s if timeout_s is not None else self._default_timeout) * 1e9)
        if _nvtx_enabled():
            torch.cuda.nvtx.range_push(f"{_OP_NAMES.get(op, 'ps.op')}[{begin}:{end}]")
        nvls = self.nvls and self._multicast_pays((int(end) - int(begin)) * self.grad.element_size())
        rc = self.heap.lib.psdev_dense_op(C.byref(self._world), C.byref(self._table), op,
                                          int(begin), int(end), C.byref(o), self.channel,
                                          self.num_ctas, tmo,
                                          (1 if sync else 0) | (2 if nvls else 0),
                                          s.cuda_stream)
        if _nvtx_enabled():
            torch.cuda.nvtx.range_pop()
        _lib.check(rc, "psdev_dense_op")

    def _multicast_pays(self, nbytes: int) -> bool:
        if self.nvls_max_bytes is not None:
            return nbytes <= self.nvls_max_bytes
        return bool(self.heap.lib.psdev_multicast_pays(self.heap.world, int(nbytes)))

    def _opt_struct(self) -> _lib.Opt:
        """The handle's parameters for the current step (rebuilt only when something changed:
        small requests are launch-bound, and building the structure costs microseconds)."""
        p = self.optimizer
        key = (max(self.step, 1) if p.kind in ("adam", "adamw") else 0, p.kind, p.lr, p.momentum,
               p.weight_decay, p.beta1, p.beta2, p.eps, p.scale, p.user_kind, p.user)
        if key != self._opt_key:
            self._opt_key = key
            self._opt_cached = p.to_struct(max(self.step, 1))
        return self._opt_cached

    def push(self, begin: int = 0, end: Optional[int] = None, *, sync: bool = True, stream=None,
             timeout_s=None, opt_step: bool = True, publish: bool = False) -> None:
        """Reduce every worker's ``grad[begin:end]`` into the owners and apply the handle.

        ``publish``: owners also store the new values of their blocks into their own
        ``weight`` buffer, from where a pull fused with a GEMM fetches them.
        """
        op = _lib.OP_PUSH | (_lib.OP_PUBLISH if publish else 0)
        self._run(op, begin, end, sync, stream, timeout_s, opt_step)

    def pull(self, begin: int = 0, end: Optional[int] = None, *, sync: bool = True, stream=None,
             timeout_s=None) -> None:
        """Owners store ``master[begin:end]`` into every worker's ``weight`` buffer."""
        self._run(_lib.OP_PULL, begin, end, sync, stream, timeout_s, False)

    def push_pull(self, begin: int = 0, end: Optional[int] = None, *, sync: bool = True,
                  stream=None, timeout_s=None, opt_step: bool = True) -> None:
        """Push and pull in one kernel pass (``ZPushPull``, include/ps/kv_app.h:290-306)."""
        self._run(_lib.OP_PUSHPULL, begin, end, sync, stream, timeout_s, opt_step)

    # -- checkpoint of the server shard ----------------------------------------------------
    def save(self, path: str) -> None:
        """Write this rank's shard (master weights, optimizer state, step) to ``path``.

        The reference keeps server state inside the user's request handle and has no
        checkpoint facility (its users send a "save model" ``cmd``); here each server shard
        is one file whose header records the key layout it belongs to."""
        torch.cuda.synchronize(self.heap.device)
        torch.save({"n": self.n_user, "blk": self.blk, "world": self.heap.world,
                    "rank": self.heap.rank, "step": self.step, "kind": self.optimizer.kind,
                    "master": self.master.cpu(),
                    "state1": None if self.state1 is None else self.state1.cpu(),
                    "state2": None if self.state2 is None else self.state2.cpu()}, path)

    def load(self, path: str) -> None:
        """Restore a shard written by :meth:`save` for the same layout (a recovered node calls
        this, then every rank pulls)."""
        ck = torch.load(path, map_location="cpu")
        if (ck["n"], ck["blk"], ck["world"], ck["rank"]) != (self.n_user, self.blk,
                                                             self.heap.world, self.heap.rank):
            raise ValueError("checkpoint belongs to a different table layout or rank")
        self.master.copy_(ck["master"])
        if self.state1 is not None and ck["state1"] is not None:
            self.state1.copy_(ck["state1"])
        if self.state2 is not None and ck["state2"] is not None:
            self.state2.copy_(ck["state2"])
        self.step = int(ck["step"])

    MAX_SEGS = 1024
    SEG_SLOTS = 16

    def run_multi(self, op: int, segments, *, sync: bool = True, stream=None, timeout_s=None) -> None:
        """Run ``op`` on several slices ``(begin, end, priority)`` in one launch and one
        rendezvous; the kernel's CTAs take the slices in priority order (device-side P3
        schedule).  At most ``MAX_SEGS`` slices per call."""
        if not segments:
            return
        if len(segments) > self.MAX_SEGS:
            raise ValueError("too many slices for one launch")
        s = stream or torch.cuda.current_stream(self.heap.device)
        if not hasattr(self, "_seg_ring"):
            # a ring of staging slots (pinned host list, device copy, device schedule): the host
            # waits only when it comes back to a slot whose copy has not run yet
            nb = self.heap.lib.psdev_sched_bytes(self.MAX_SEGS)
            dev = self.heap.device
            self._seg_ring = [
                (torch.empty(self.MAX_SEGS * 3, dtype=torch.int64).pin_memory(),
                 torch.empty(self.MAX_SEGS * 3, dtype=torch.int64, device=dev),
                 torch.empty(nb, dtype=torch.uint8, device=dev), torch.cuda.Event())
                for _ in range(self.SEG_SLOTS)]
            self._seg_next = 0
            self._seg_used = [False] * self.SEG_SLOTS
        slot = self._seg_next
        self._seg_next = (slot + 1) % self.SEG_SLOTS
        seg_host, seg_dev, sched_dev, seg_free = self._seg_ring[slot]
        if self._seg_used[slot]:
            seg_free.synchronize()   # that slot's previous launch has read the staging buffer
        self._seg_used[slot] = True
        flat = [int(v) for seg in segments for v in seg]
        seg_host[: len(flat)] = torch.tensor(flat, dtype=torch.int64)
        with torch.cuda.stream(s):
            seg_dev[: len(flat)].copy_(seg_host[: len(flat)], non_blocking=True)
        seg_free.record(s)
        o = self._opt_struct()
        gsz = self.grad.element_size()
        nvls = self.nvls and self._multicast_pays(sum(int(e) - int(b) for b, e, _ in segments) * gsz)
        tmo = int((timeout_s if timeout_s is not None else self._default_timeout) * 1e9)
        rc = self.heap.lib.psdev_dense_op_multi(
            C.byref(self._world), C.byref(self._table), op, seg_dev.data_ptr(),
            len(segments), sched_dev.data_ptr(), C.byref(o), self.channel, self.num_ctas,
            tmo, (1 if sync else 0) | (2 if nvls else 0), s.cuda_stream)
        _lib.check(rc, "psdev_dense_op_multi")

    def check(self) -> None:
        """Raise if a device wait on this table's channel ran out."""
        self.heap.check_channel(self.channel)
