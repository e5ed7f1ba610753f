"""Key-list utilities on the device: radix sort, unique, ordered match (merge-join).

Device counterparts of the reference's ``ParallelSort`` and ``ParallelOrderedMatch`` helpers
(include/ps/internal/parallel_sort.h:23-55, parallel_kv_match.h:29-120) and its ``AssignOp``
operators (assign_op.h:12-21)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib

ASSIGN, PLUS, MINUS, TIMES, DIVIDE, AND, OR, XOR = range(8)


def sort_keys(keys: torch.Tensor, key_bits: int = 64, return_perm: bool = False,
              check: bool = False) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Sort uint64 keys (stored as int64 bit patterns) ascending, in place; keys must be below
    ``2**key_bits``.  With ``return_perm`` also returns the stable permutation (int32 indices
    into the input).  ``check`` waits for the sort and raises if one of its bounded waits (a
    tile looking back at the tiles before it) ran out."""
    assert keys.is_cuda and keys.dtype == torch.int64 and keys.is_contiguous()
    lib = _lib.device_lib()
    n = keys.numel()
    perm = torch.empty(n, dtype=torch.int32, device=keys.device) if return_perm else None
    nbytes = lib.psdev_sort_scratch_bytes(n, 1 if return_perm else 0)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=keys.device)
    rc = lib.psdev_sort_keys(keys.data_ptr(), perm.data_ptr() if perm is not None else None, n,
                             key_bits, scratch.data_ptr(), nbytes,
                             torch.cuda.current_stream(keys.device).cuda_stream)
    _lib.check(rc, "psdev_sort_keys")
    if check:
        _lib.check(lib.psdev_sort_status(scratch.data_ptr(),
                                         torch.cuda.current_stream(keys.device).cuda_stream),
                   "psdev_sort_status")
    return keys, perm


def sort_unique_sum(keys: torch.Tensor, vals: torch.Tensor, key_bits: int = 64
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Turn arbitrary (key, value) pairs into the sorted unique keys a push needs, summing the
    values of repeated keys."""
    k = keys.clone()
    k, perm = sort_keys(k, key_bits, return_perm=True)
    v = vals[perm.long()]
    uk, inv = torch.unique_consecutive(k, return_inverse=True)
    out = torch.zeros(uk.numel(), dtype=vals.dtype, device=vals.device)
    out.index_add_(0, inv, v)
    return uk, out


def ordered_match(src_keys: torch.Tensor, src_vals: torch.Tensor, dst_keys: torch.Tensor,
                  dst_vals: torch.Tensor, op: int = ASSIGN, k: int = 1) -> int:
    """``dst_vals[j] op= src_vals[i]`` for every key in both sorted unique lists (``k`` values
    per key); returns how many keys matched."""
    assert src_vals.dtype == dst_vals.dtype and src_vals.dtype in (torch.float32, torch.int32)
    matched = torch.zeros(1, dtype=torch.int64, device=dst_vals.device)
    rc = _lib.device_lib().psdev_ordered_match(
        src_keys.data_ptr(), src_vals.data_ptr(), src_keys.numel(), dst_keys.data_ptr(),
        dst_vals.data_ptr(), dst_keys.numel(), k, op,
        0 if src_vals.dtype == torch.float32 else 1, matched.data_ptr(),
        torch.cuda.current_stream(dst_vals.device).cuda_stream)
    _lib.check(rc, "psdev_ordered_match")
    return int(matched.item())
