"""Counters of the data and control planes in one place.

The reference accumulates ``send_bytes_``/``recv_bytes_`` in its van but never reports them
(include/ps/internal/van.h:145-146, src/van.cc:391,417).  Here they are readable, together with
the number of kernels the device plane has launched and the heap usage."""
from __future__ import annotations



def snapshot(heap=None, host: bool = False) -> dict:
    """Current counters: device launches, heap bytes in use, and (if the host runtime is
    started) bytes sent/received by the van."""
    from .. import _lib
    out = {"device_kernel_launches": int(_lib.device_lib().psdev_launch_count())}
    if heap is not None:
        out["heap_bytes_in_use"] = heap.in_use
        out["heap_bytes_total"] = heap.nbytes
        out["heap_backend"] = heap.backend
        out["nvswitch_multicast"] = bool(heap.mc_base)
    if host:
        from .. import host as h
        sent, recv = h.traffic()
        out["van_bytes_sent"], out["van_bytes_received"] = sent, recv
        out["shared_memory_arrays"] = h.shm_stats()
    return out
