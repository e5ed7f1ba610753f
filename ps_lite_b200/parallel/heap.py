"""Symmetric device heap shared by the ranks of one box.

Each rank allocates an arena of the same size, exports it, and maps every peer's arena.
Buffers are carved out with a deterministic first-fit allocator, so the same sequence of
``alloc`` calls yields the same offsets on every rank and a kernel can address a peer's
copy of a tensor as ``peer_base[p] + offset``.

This is the device counterpart of the reference's registered memory pool and address
exchange for RDMA (src/ibverbs_van.h:86-214 ``SimpleMempool``; :632-724 rendezvous).
A job's heap normally comes from the device plane of the host runtime (backend ``"plane"``,
src/van/nvl_van.cc): the arenas were created, exchanged over the control plane and mapped by
``Plane::Start``, and this object is a view of them.  The other backends build a heap
without a job: one rank (tests, single-GPU use), ranks emulated on one GPU, or ranks of a
``torch.distributed`` group whose handles travel through that group or through a
caller-supplied ``exchange`` callable.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Sequence

import torch

from .. import _lib


class _RawCuda:
    """Adapter exposing a raw device range through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, keepalive=None):
        self.__cuda_array_interface__ = {
            "shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2,
        }
        self._keepalive = keepalive


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device, keepalive=None) -> torch.Tensor:
    """A uint8 tensor aliasing ``nbytes`` of device memory at ``ptr`` (no copy)."""
    return torch.as_tensor(_RawCuda(ptr, nbytes, keepalive), device=device)


class SymmetricHeap:
    """One rank's view of the job-wide symmetric heap."""

    def __init__(self, nbytes: int, rank: int = 0, world: int = 1, group=None,
                 device: Optional[torch.device] = None,
                 exchange: Optional[Callable[[bytes], Sequence[bytes]]] = None,
                 backend: str = "auto",
                 _bases: Optional[Sequence[int]] = None, _owner: bool = True):
        if world < 1 or world > _lib.MAX_RANKS:
            raise ValueError(f"world must be in [1, {_lib.MAX_RANKS}]")
        self.lib = _lib.device_lib()
        self.rank, self.world = int(rank), int(world)
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        self.nbytes = int(nbytes) & ~255
        self._owner = _owner
        self._opened: list[int] = []
        self._sub = self.lib.psdev_suballoc_new(self.nbytes)
        self._siblings: list["SymmetricHeap"] = []
        self.mc_base = 0        # NVSwitch multicast alias of the arena (0: none)
        self._symm = None       # torch symmetric-memory tensor and handle, when used
        self.backend = "ipc"
        self._plane = False
        self.emulated_ranks = _bases is not None  # ranks of one process on one GPU
        if backend == "plane":
            self._init_plane()
            return
        if _bases is not None:  # view created by `emulated`
            self.bases = list(_bases)
            self._base = self.bases[self.rank]
            return
        if backend == "auto":
            import os
            backend = os.environ.get("PSB200_HEAP", "symm" if world > 1 and exchange is None
                                     else "ipc")
        if backend == "symm" and world > 1:
            try:
                self._init_symm(group)
                return
            except Exception as exc:  # fall back to CUDA IPC (no multicast alias then)
                import warnings
                warnings.warn(f"symmetric-memory heap unavailable ({exc}); using CUDA IPC")
        if backend == "vmm":
            self._init_vmm(group, exchange)
            return
        with torch.cuda.device(self.device):
            base = C.c_void_p()
            handle = C.create_string_buffer(_lib.IPC_HANDLE_BYTES)
            _lib.check(self.lib.psdev_heap_create(self.nbytes, C.byref(base), handle),
                       "psdev_heap_create")
            self._base = base.value
            self.bases = [0] * world
            self.bases[rank] = self._base
            if world > 1:
                mine = bytes(handle.raw)
                if exchange is not None:
                    handles = list(exchange(mine))
                else:
                    import torch.distributed as dist
                    handles = [None] * world
                    dist.all_gather_object(handles, mine, group=group)
                for p, h in enumerate(handles):
                    if p == rank:
                        continue
                    ptr = C.c_void_p()
                    _lib.check(self.lib.psdev_heap_open(h, C.byref(ptr)), f"psdev_heap_open({p})")
                    self.bases[p] = ptr.value
                    self._opened.append(ptr.value)

    def _init_plane(self) -> None:
        """View of the arenas that the host runtime's device plane has set up."""
        from .. import host
        L = host.lib()
        if not L.psnvl_started():
            raise RuntimeError("the device plane is not started (kvstore.init does that)")
        ws = _lib.World()
        L.psnvl_world_struct(C.byref(ws))
        self.lib.psdev_suballoc_delete(self._sub)
        self._sub = None
        self._plane, self._owner = True, False
        self.rank, self.world = int(ws.rank), int(ws.world)
        self.bases = [int(ws.peer_base[p] or 0) for p in range(self.world)]
        self._base = self.bases[self.rank]
        self.mc_base = int(ws.mc_base or 0)
        self.nbytes = int(ws.heap_bytes)
        self.backend = L.psnvl_backend().decode()

    def _init_vmm(self, group, exchange) -> None:
        """Arena from the virtual-memory-management API (src/device/vmm_heap.cu): the physical
        allocation is exported as a file descriptor, the descriptors go round over Unix sockets
        (``fd_exchange.py``) and every rank maps every arena.  No multicast alias."""
        import os
        from .fd_exchange import exchange_fds
        with torch.cuda.device(self.device):
            if not self.lib.psdev_vmm_supported():
                raise RuntimeError("this device cannot export allocations as file descriptors")
            base, fd, mapped = C.c_void_p(), C.c_int(-1), C.c_size_t(0)
            _lib.check(self.lib.psdev_vmm_create(self.nbytes, C.byref(base), C.byref(fd),
                                                 C.byref(mapped)), "psdev_vmm_create")
            self._base = base.value
            self._vmm_bytes = int(mapped.value)
            self.bases = [0] * self.world
            self.bases[self.rank] = self._base
            self.backend = "vmm"
            try:
                if self.world > 1:
                    if exchange is not None:
                        gather = exchange
                    else:
                        import torch.distributed as dist

                        def gather(payload: bytes):
                            got = [None] * self.world
                            dist.all_gather_object(got, payload, group=group)
                            return got
                    sizes = [int(x) for x in gather(str(self._vmm_bytes).encode())]
                    fds = exchange_fds(self.rank, self.world, fd.value, gather)
                    try:
                        for p in range(self.world):
                            if p == self.rank:
                                continue
                            ptr = C.c_void_p()
                            _lib.check(self.lib.psdev_vmm_import(fds[p], sizes[p], C.byref(ptr)),
                                       f"psdev_vmm_import({p})")
                            self.bases[p] = ptr.value
                            self._opened.append(ptr.value)
                    finally:
                        for f in fds:
                            os.close(f)
            finally:
                os.close(fd.value)

    def _init_symm(self, group) -> None:
        """Arena from torch's symmetric memory: cuMem allocations exchanged among the ranks
        and, where the fabric supports it, bound to an NVSwitch multicast object."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        grp = group if group is not None else dist.group.WORLD
        with torch.cuda.device(self.device):
            t = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(t, group=grp)
            t[: _lib.CTRL_BYTES].zero_()
            torch.cuda.synchronize()
        self._symm = (t, hdl)
        self.bases = [int(p) for p in hdl.buffer_ptrs]
        self._base = self.bases[self.rank]
        if self._base != t.data_ptr():
            raise RuntimeError("symmetric memory handle does not describe the arena")
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
        self.mc_base = mc
        self.backend = "symm"
        self._owner = False  # torch owns the allocation
        dist.barrier(group=grp)

    # -- single-GPU emulation of a multi-rank job --------------------------------------
    @classmethod
    def emulated(cls, nbytes: int, world: int, device=None,
                 backend: str = "ipc") -> list["SymmetricHeap"]:
        """``world`` heaps on one GPU in one process; element r is rank r's view.

        Kernels that rendezvous must not be launched on these views (all "ranks" share a
        GPU); they are for running every rank's role back to back with ``sync=False``.
        """
        dev = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device())
        owners = [cls(nbytes, 0, 1, device=dev, backend=backend) for _ in range(world)]
        bases = [h._base for h in owners]
        views = [cls(nbytes, r, world, device=dev, _bases=bases, _owner=False)
                 for r in range(world)]
        for v in views:
            v._siblings = owners  # keep the allocations alive
        return views

    # -- allocation ------------------------------------------------------------------------
    def alloc(self, nbytes: int, align: int = 256) -> int:
        if self._plane:
            from .. import host
            off = host.lib().psnvl_alloc(int(nbytes), int(align))
            if off < 0:
                raise _lib.PsdevError(-5, f"symmetric heap alloc of {nbytes} bytes")
            return int(off)
        off = self.lib.psdev_suballoc_alloc(self._sub, int(nbytes), int(align))
        if off < 0:
            raise _lib.PsdevError(int(off), f"symmetric heap alloc of {nbytes} bytes")
        return int(off)

    def free(self, offset: int) -> None:
        if self._plane:
            from .. import host
            host._ck(host.lib().psnvl_free(int(offset)))
            return
        _lib.check(self.lib.psdev_suballoc_free(self._sub, int(offset)), "suballoc_free")

    @property
    def in_use(self) -> int:
        if self._plane:
            from .. import host
            return int(host.lib().psnvl_heap_in_use())
        return int(self.lib.psdev_suballoc_in_use(self._sub))

    def tensor(self, offset: int, numel: int, dtype: torch.dtype, rank: Optional[int] = None
               ) -> torch.Tensor:
        """Typed view of ``numel`` elements at ``offset`` in rank ``rank``'s arena."""
        r = self.rank if rank is None else rank
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if offset < 0 or offset + nbytes > self.nbytes:
            raise ValueError("view outside the heap")
        raw = tensor_from_ptr(self.bases[r] + offset, nbytes, self.device, keepalive=self)
        return raw.view(dtype)

    def world_struct(self) -> _lib.World:
        w = _lib.World()
        w.rank, w.world = self.rank, self.world
        for p in range(self.world):
            w.peer_base[p] = self.bases[p]
        w.mc_base = self.mc_base or None
        w.heap_bytes = self.nbytes
        return w

    # -- channel state -----------------------------------------------------------------------
    def channel_status(self, channel: int) -> tuple[int, int]:
        """(status, epoch) of a channel; synchronises the device."""
        st, ep = C.c_int32(), C.c_uint64()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.psdev_channel_status(self._base, channel, C.byref(st),
                                                     C.byref(ep)), "channel_status")
        return st.value, ep.value

    def check_channel(self, channel: int) -> None:
        st, _ = self.channel_status(channel)
        if st != 0:
            raise _lib.PsdevError(st, f"device channel {channel} on rank {self.rank}")

    def clear_channel(self, channel: int) -> None:
        with torch.cuda.device(self.device):
            _lib.check(self.lib.psdev_channel_clear(self._base, channel), "channel_clear")

    def barrier(self, channel: int = _lib.NUM_CHANNELS - 1, timeout_s: float = 20.0,
                stream: Optional[torch.cuda.Stream] = None) -> None:
        """Device-side barrier of all ranks (flag exchange in peer memory)."""
        s = stream or torch.cuda.current_stream(self.device)
        w = self.world_struct()
        _lib.check(self.lib.psdev_device_barrier(C.byref(w), channel, int(timeout_s * 1e9),
                                                 s.cuda_stream), "device_barrier")

    def broadcast(self, t: torch.Tensor, src: int = 0, chunk_bytes: int = 64 << 20) -> None:
        """Overwrite ``t`` (contiguous, on this heap's device) on every rank with rank
        ``src``'s values, moved through a scratch buffer of the heap: ``src`` copies a chunk
        into its arena, a device barrier, the others read it from the peer arena with the
        library's 16-byte copy kernel, another barrier.  Collective."""
        if self.world == 1:
            return
        flat = t.reshape(-1).view(torch.uint8)
        chunk = min((flat.numel() + 255) & ~255, int(chunk_bytes))
        off = self.alloc(chunk)
        mine = self.tensor(off, chunk, torch.uint8)
        s = torch.cuda.current_stream(self.device)
        try:
            for b in range(0, flat.numel(), chunk):
                e = min(b + chunk, flat.numel())
                if self.rank == src:
                    mine[: e - b].copy_(flat[b:e])
                self.barrier()
                if self.rank != src:
                    n16 = (e - b + 15) & ~15
                    tmp = torch.empty(n16, dtype=torch.uint8, device=self.device)
                    _lib.check(self.lib.psdev_link_copy(tmp.data_ptr(), self.bases[src] + off,
                                                        n16, 0, s.cuda_stream), "link_copy")
                    flat[b:e].copy_(tmp[: e - b])
                self.barrier()
            torch.cuda.synchronize(self.device)
        finally:
            self.free(off)

    def close(self) -> None:
        if self._sub:
            self.lib.psdev_suballoc_delete(self._sub)
            self._sub = None
        if not self._owner:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            vmm = self.backend == "vmm"
            for p in self._opened:
                (self.lib.psdev_vmm_release if vmm else self.lib.psdev_heap_close)(p)
            self._opened = []
            if self._base:
                (self.lib.psdev_vmm_release if vmm else self.lib.psdev_heap_destroy)(self._base)
                self._base = 0
