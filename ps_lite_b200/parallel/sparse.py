"""Sparse key-value table on the device data plane (direct-index store, range-sharded keys).

Per step every worker pushes sorted unique uint64 keys with one fp32 gradient each and pulls
the updated values of the same keys (``KVWorker::ZPush`` + ``ZPull`` of the reference,
include/ps/kv_app.h:243-280).  Server ``s`` owns keys ``[s*range, (s+1)*range)``
(src/postoffice.cc:169-180) and applies ``sum``, ``sgd`` or FTRL-proximal to the keys that were
pushed.  See ``src/kernels/sparse.cu`` for the kernels.
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
                 hash_capacity: int = 0):
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
        self.keys_off = heap.alloc(8 * max_keys)
        self.grads_off = heap.alloc(4 * max_keys)
        self.out_off = heap.alloc(4 * max_keys)
        self.pos_off = heap.alloc(8 * (W + 2))
        self.acc_off = heap.alloc(4 * slots)
        self.hkeys_off = heap.alloc(8 * self.capacity) if self.capacity else 0
        self.keys = heap.tensor(self.keys_off, max_keys, torch.int64)  # bit pattern of uint64
        self.grads = heap.tensor(self.grads_off, max_keys, torch.float32)
        self.out = heap.tensor(self.out_off, max_keys, torch.float32)
        self.pos = heap.tensor(self.pos_off, W + 2, torch.int64)
        self.acc = heap.tensor(self.acc_off, slots, torch.float32)
        self.hkeys = (heap.tensor(self.hkeys_off, self.capacity, torch.int64)
                      if self.capacity else None)
        if self.hkeys is not None:
            self.hkeys.fill_(-1)   # all ones = empty slot
        self.acc.zero_()
        self.pos.zero_()
        dev = heap.device
        self.w = torch.zeros(slots, dtype=torch.float32, device=dev)
        self.z = torch.zeros(slots, dtype=torch.float32, device=dev) if kind == "ftrl" else None
        self.n = torch.zeros(slots, dtype=torch.float32, device=dev) if kind == "ftrl" else None
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
        self._t = t
        self.barrier_channel = barrier_channel
        self.count = 0

    # -- the three phases; `sync=False` lets a test run all ranks' phases on one GPU ----------
    def stage(self, keys: torch.Tensor, grads: torch.Tensor) -> None:
        """Copy a request (sorted unique keys, one gradient each) into the heap buffers."""
        n = keys.numel()
        if n > self.max_keys:
            raise ValueError("more keys than max_keys")
        self.keys[:n].copy_(keys.view(torch.int64), non_blocking=True)
        self.grads[:n].copy_(grads, non_blocking=True)
        self.count = n

    def scatter(self, stream=None) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_scatter(C.byref(self._world), C.byref(self._t),
                                                      self.count, 0, s.cuda_stream), "sparse_scatter")

    def apply(self, stream=None) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_apply(C.byref(self._world), C.byref(self._t), 0,
                                                    s.cuda_stream), "sparse_apply")

    def respond(self, stream=None) -> None:
        s = stream or torch.cuda.current_stream(self.heap.device)
        _lib.check(self.heap.lib.psdev_sparse_respond(C.byref(self._world), C.byref(self._t), 0,
                                                      s.cuda_stream), "sparse_respond")

    def push_pull(self, keys: torch.Tensor, grads: torch.Tensor) -> torch.Tensor:
        """One step: push (keys, grads), apply the handle on the owners, pull the new values.

        Returns a view of the heap output buffer (valid until the next call)."""
        self.stage(keys, grads)
        self.scatter()
        self.heap.barrier(self.barrier_channel)   # every worker's gradients are accumulated
        self.apply()
        self.respond()
        self.heap.barrier(self.barrier_channel)   # every server's answers have landed
        return self.out[: self.count]

    def check(self) -> None:
        self.heap.check_channel(self.barrier_channel)
        if self.capacity and int(self.overflow.item()):
            raise RuntimeError("sparse hash store is full: raise hash_capacity")

    def save(self, path: str) -> None:
        """Write this rank's key range (values and FTRL state) to ``path``."""
        torch.cuda.synchronize(self.heap.device)
        torch.save({"key_space": self.key_space, "world": self.heap.world, "rank": self.heap.rank,
                    "kind": self.kind, "w": self.w.cpu(),
                    "z": None if self.z is None else self.z.cpu(),
                    "n": None if self.n is None else self.n.cpu()}, path)

    def load(self, path: str) -> None:
        ck = torch.load(path, map_location="cpu")
        if (ck["key_space"], ck["world"], ck["rank"]) != (self.key_space, self.heap.world,
                                                          self.heap.rank):
            raise ValueError("checkpoint belongs to a different key layout or rank")
        self.w.copy_(ck["w"])
        if self.z is not None and ck["z"] is not None:
            self.z.copy_(ck["z"])
            self.n.copy_(ck["n"])
