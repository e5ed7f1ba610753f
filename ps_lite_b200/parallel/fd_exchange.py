"""All-to-all exchange of file descriptors between the ranks of one host.

A descriptor is only meaningful inside its process, so it cannot travel through
``torch.distributed`` or the host runtime's messages as a number; the kernel has to install a
copy in the receiving process.  Every rank binds a Unix datagram socket in the abstract
namespace (no file system entry), the socket names are exchanged through any all-gather the
caller provides, and each rank then sends its descriptor to every peer as ``SCM_RIGHTS``
ancillary data.  Used for the arenas of the virtual-memory-management heap backend
(``heap.py``); the host runtime's shared-memory frames pass descriptors the same way inside
the socket van (src/van/tcp_van.cc).
"""
from __future__ import annotations

import array
import os
import socket
import struct
import uuid
from typing import Callable, List, Sequence


def exchange_fds(rank: int, world: int, fd: int,
                 all_gather: Callable[[bytes], Sequence[bytes]],
                 timeout_s: float = 60.0) -> List[int]:
    """Give ``fd`` to every peer and collect theirs.

    ``all_gather(payload)`` must return the payloads of all ranks in rank order (for example a
    wrapper around ``torch.distributed.all_gather_object``).  Returns a list of ``world``
    descriptors owned by the caller; element ``rank`` is a duplicate of ``fd``.
    """
    if world == 1:
        return [os.dup(fd)]
    name = b"\0psb200-fd-" + uuid.uuid4().hex.encode() + b"-%d" % rank
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
    try:
        srv.bind(name)
        srv.settimeout(timeout_s)
        names = [bytes(n) for n in all_gather(name)]   # everyone is bound once this returns
        if len(names) != world or names[rank] != name:
            raise RuntimeError("all_gather did not return one socket name per rank in rank order")
        out = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        try:
            for p in range(world):
                if p != rank:
                    # (socket.send_fds drops its address argument: use sendmsg itself)
                    out.sendmsg([struct.pack("<i", rank)],
                                [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))],
                                0, names[p])
        finally:
            out.close()
        got: List[int] = [-1] * world
        got[rank] = os.dup(fd)
        try:
            for _ in range(world - 1):
                msg, fds, _flags, _addr = socket.recv_fds(srv, 16, 4)
                if len(msg) != 4 or len(fds) != 1:
                    for f in fds:
                        os.close(f)
                    raise RuntimeError("malformed descriptor message")
                src = struct.unpack("<i", msg)[0]
                if not 0 <= src < world or src == rank or got[src] >= 0:
                    os.close(fds[0])
                    raise RuntimeError(f"unexpected descriptor from rank {src}")
                got[src] = fds[0]
        except BaseException:
            for f in got:
                if f >= 0:
                    os.close(f)
            raise
        return got
    finally:
        srv.close()
