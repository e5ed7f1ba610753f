"""Sparse key-value table on the device data plane (direct-index store, range-sharded keys).

Per step every worker pushes sorted unique uint64 keys with their fp32 values and pulls the
updated values of the same keys (``KVWorker::ZPush`` + ``ZPull`` of the reference,
include/ps/kv_app.h:243-280).  A value has ``width`` elements, or, with ``var_len=True``, a
per-key number of elements up to ``width`` given by ``lens`` (the reference's dynamic-length
values, kv_app.h:24-31): the values of a request are then packed back to back and the kernels
find value ``i`` at the prefix sum of the lengths, as ``DefaultSlicer`` does (kv_app.h:547-567).
Server ``s`` owns keys ``[s*range, (s+1)*range)`` (src/postoffice.cc:169-180) and applies
``sum``, ``sgd`` or FTRL-proximal element-wise to the keys that were pushed.  See
``src/kernels/sparse.cu`` for the kernels.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from .heap import SymmetricHeap

_KINDS = {"sum": 0, "sgd": 1, "ftrl": 2}


class SparseTable:
    """Every rank must create its tables in the same order with the same arguments."""

    def __init__(self, heap: SymmetricHeap, key_space: int, max_keys: int, kind: str = "ftrl",
                 lr: float = 0.01, alpha: float = 0.1, beta: float = 1.0, l1: float = 1.0,
                 l2: float = 1.0, barrier_channel: int = _lib.NUM_CHANNELS - 2,
                 hash_capacity: int = 0, width: int = 1, var_len: bool = False):
        self.heap = heap
        W = heap.world
        self.key_space, self.max_keys, self.kind = int(key_space), int(max_keys), kind
        self.range = (self.key_space + W - 1) // W
        # store: direct index (one slot per key of the range) or, with hash_capacity > 0, an
        # open-addressing table of that many slots per server for huge or unbounded key spaces
        self.capacity = 0
        if hash_capacity:
            self.capacity = 1 << (int(hash_capacity) - 1).bit_length()
        slots = self.capacity or self.range
        self.slots, self.width, self.var_len = slots, int(width), bool(var_len)
        if self.width < 1:
            raise ValueError("width must be at least 1")
        max_vals = max_keys * self.width
        self.max_vals = max_vals
        self.keys_off = heap.alloc(8 * max_keys)
        self.grads_off = heap.alloc(4 * max_vals)
        self.out_off = heap.alloc(4 * max_vals)
        self.pos_off = heap.alloc(8 * (W + 2))
        self.acc_off = heap.alloc(4 * slots * self.width)
        self.hkeys_off = heap.alloc(8 * self.capacity) if self.capacity else 0
        self.lens_off = heap.alloc(4 * max_keys) if var_len else 0
        self.offs_off = heap.alloc(8 * (max_keys + 1)) if var_len else 0
        self.keys = heap.tensor(self.keys_off, max_keys, torch.int64)  # bit pattern of uint64
        self.grads = heap.tensor(self.grads_off, max_vals, torch.float32)
        self.out = heap.tensor(self.out_off, max_vals, torch.float32)
        self.pos = heap.tensor(self.pos_off, W + 2, torch.int64)
        self.acc = heap.tensor(self.acc_off, slots * self.width, torch.float32)
        self.lens = heap.tensor(self.lens_off, max_keys, torch.int32) if var_len else None
        self.offs = heap.tensor(self.offs_off, max_keys + 1, torch.int64) if var_len else None
        self.hkeys = (heap.tensor(self.hkeys_off, self.capacity, torch.int64)
                      if self.capacity else None)
        if self.hkeys is not None:
            self.hkeys.fill_(-1)   # all ones = empty slot
        self.acc.zero_()
        self.pos.zero_()
        dev = heap.device
        ne = slots * self.width
        if kind == "ftrl":
            # three numbers per value, side by side ({w, z, n, -}): an update touches one
            # 16-byte group instead of three sectors of three arrays; w, z, n are strided views
            self.state = torch.zeros(ne * 4, dtype=torch.float32, device=dev)
            sv = self.state.view(ne, 4)
            self.w, self.z, self.n = sv[:, 0], sv[:, 1], sv[:, 2]
            self.state_stride = 4
        else:
            self.w = torch.zeros(ne, dtype=torch.float32, device=dev)
            self.z = self.n = None
            self.state_stride = 1
        self.klen = torch.zeros(slots, dtype=torch.int32, device=dev) if var_len else None
        self.overflow = torch.zeros(1, dtype=torch.int32, device=dev)
        self._world = heap.world_struct()
        t = _lib.Sparse()
        t.range = self.range
        t.keys_off, t.grads_off, t.out_off = self.keys_off, self.grads_off, self.out_off
        t.pos_off, t.acc_off = self.pos_off, self.acc_off
        t.w = self.w.data_ptr()
        t.z = self.z.data_ptr() if self.z is not None else None
        t.n = self.n.data_ptr() if self.n is not None else None
        t.kind = _KINDS[kind]
        t.lr, t.alpha, t.beta, t.l1, t.l2 = lr, alpha, beta, l1, l2
        t.hkeys_off, t.capacity = self.hkeys_off, self.capacity
        t.overflow = self.overflow.data_ptr()
        t.width, t.channel = self.width, int(barrier_channel)
        t.max_n, t.max_vals, t.slots = int(max_keys), int(max_vals), int(slots)
        t.lens_off, t.offs_off = self.lens_off, self.offs_off
        t.state_stride = self.state_stride
        t.klen = self.klen.data_ptr() if self.klen is not None else None
        from .dense import default_timeout_s
        t.timeout_ns = int(default_timeout_s() * 1e9)
        self._t = t
        self.barrier_channel = barrier_channel
        self.count = 0

    # -- the three phases; `sync=False` lets a test run all ranks' phases on one GPU ----------
    def stage(self, keys: torch.Tensor, grads: torch.Tensor,
              lens: "torch.Tensor | None" = None) -> None:
        """Copy a request into the heap buffers: sorted unique keys and their values (``width``
        per key, or ``lens[i]`` per key back to back for a ``var_len`` table)."""
        n = keys.numel()
        if n > self.max_keys:
            raise ValueError("more keys than max_keys")
        nv = grads.numel()
        if self.var_len:
            if lens is None or lens.numel() != n:
                raise ValueError("a var_len table needs one length per key")
            if nv > self.max_vals:
                raise ValueError("more values than the table was sized for")
            self.lens[:n].copy_(lens.to(torch.int32), non_blocking=True)
        elif nv != n * self.width:
            raise ValueError(f"expected {self.width} values per key")
        self.keys[:n].copy_(keys.view(torch.int64), non_blocking=True)
        self.grads[:nv].copy_(grads.reshape(-1), non_blocking=True)
        self.count, self.count_vals = n, nv

    def scatter(self, stream=None) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_scatter(C.byref(self._world), C.byref(self._t),
                                                      self.count, 0, s.cuda_stream), "sparse_scatter")

    def apply(self, stream=None, sync: bool = False) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_apply(C.byref(self._world), C.byref(self._t), 0,
                                                    int(sync), s.cuda_stream), "sparse_apply")

    def respond(self, stream=None, sync: bool = False) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_respond(C.byref(self._world), C.byref(self._t), 0,
                                                      int(sync), s.cuda_stream), "sparse_respond")

    def push_pull(self, keys: torch.Tensor, grads: torch.Tensor,
                  lens: "torch.Tensor | None" = None) -> torch.Tensor:
        """One step: push (keys, values), apply the handle on the owners, pull the new values.

        Three launches: scatter; apply, which first waits for every rank's scatter; respond,
        which ends when every rank's answers have landed.  Returns a view of the heap output
        buffer (valid until the next call), laid out like the pushed values."""
        self.stage(keys, grads, lens)
        self.scatter()
        multi = self.heap.world > 1
        self.apply(sync=multi)
        self.respond(sync=multi)
        return self.out[: self.count_vals]

    def pull(self, keys: torch.Tensor, sync: "bool | None" = None):
        """Pull without push.  Fixed width: the values of ``keys`` (``width`` per key).  With
        ``var_len``: the owners first store the lengths they hold into this rank's array of
        lengths (between two device barriers), then answer; returns ``(values, lens)`` with the
        values packed back to back.  Collective on several ranks, like ``push_pull``."""
        n = keys.numel()
        if n > self.max_keys:
            raise ValueError("more keys than max_keys")
        multi = self.heap.world > 1 if sync is None else sync
        lib, s = self.heap.lib, torch.cuda.current_stream(self.heap.device)
        self.keys[:n].copy_(keys.view(torch.int64), non_blocking=True)
        self.count = n
        if not self.var_len:
            self.count_vals = n * self.width
            self.grads[: self.count_vals].zero_()
            self.scatter()
            self.apply(sync=multi)
            self.respond(sync=multi)
            return self.out[: self.count_vals]
        self.lens[:n].zero_()
        _lib.check(lib.psdev_key_shard_lookup(self.keys.data_ptr(), n, self.range,
                                              self.heap.world, self.pos.data_ptr(),
                                              s.cuda_stream), "key_shard_lookup")
        if multi:
            self.heap.barrier(self.barrier_channel)
        _lib.check(lib.psdev_sparse_lens(C.byref(self._world), C.byref(self._t), 0,
                                         s.cuda_stream), "sparse_lens")
        if multi:
            self.heap.barrier(self.barrier_channel)
        _lib.check(lib.psdev_lens_to_offsets(self.lens.data_ptr(), n, self.offs.data_ptr(),
                                             s.cuda_stream), "lens_to_offsets")
        self.apply(sync=multi)
        self.respond(sync=multi)
        self.count_vals = int(self.offs[n].item())
        return self.out[: self.count_vals], self.lens[:n]

    def check(self) -> None:
        self.heap.check_channel(self.barrier_channel)
        if self.capacity and int(self.overflow.item()):
            raise RuntimeError("sparse hash store is full: raise hash_capacity")

    def save(self, path: str) -> None:
        """Write this rank's key range (values and FTRL state) to ``path``."""
        torch.cuda.synchronize(self.heap.device)
        torch.save({"key_space": self.key_space, "world": self.heap.world, "rank": self.heap.rank,
                    "kind": self.kind, "width": self.width, "w": self.w.cpu(),
                    "klen": None if self.klen is None else self.klen.cpu(),
                    "z": None if self.z is None else self.z.cpu(),
                    "n": None if self.n is None else self.n.cpu()}, path)

    def load(self, path: str) -> None:
        ck = torch.load(path, map_location="cpu")
        if (ck["key_space"], ck["world"], ck["rank"]) != (self.key_space, self.heap.world,
                                                          self.heap.rank):
            raise ValueError("checkpoint belongs to a different key layout or rank")
        if ck.get("width", 1) != self.width:
            raise ValueError("checkpoint has another value width")
        self.w.copy_(ck["w"])
        if self.klen is not None and ck.get("klen") is not None:
            self.klen.copy_(ck["klen"])
        if self.z is not None and ck["z"] is not None:
            self.z.copy_(ck["z"])
            self.n.copy_(ck["n"])
