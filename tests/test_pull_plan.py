"""The pull plan of the GEMM-fused pull (ring mode), checked on the host against a plain
enumeration: every element of W that another rank owns is covered exactly once, nothing of
this rank's own blocks or outside W is touched, chunks never cross a block, are at most 8 KB,
16-byte aligned, and come in address order."""
import ctypes as C

import pytest

from ps_lite_b200 import _lib


def _plan(off, nk, blk, world, rank):
    lib = _lib.device_lib()
    owner, b, e = C.c_int(0), C.c_int64(0), C.c_int64(0)
    n = lib.psdev_pull_plan_chunk(off, nk, blk, world, rank, -1, None, None, None)
    out = []
    for i in range(n):
        lib.psdev_pull_plan_chunk(off, nk, blk, world, rank, i, C.byref(owner), C.byref(b),
                                  C.byref(e))
        if b.value < e.value:
            out.append((owner.value, b.value, e.value))
    return out


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("blk", [8, 1024, 4096, 4104, 12288])
@pytest.mark.parametrize("off,nk", [(0, 256 * 1024), (1024, 768 * 256), (8, 8), (40960, 99992),
                                     (4096 * 7 + 16, 3 * 12288 + 24)])
def test_plan_covers_remote_blocks_once(world, blk, off, nk):
    for rank in range(world):
        chunks = _plan(off, nk, blk, world, rank)
        covered = 0
        last_end = -1
        for owner, b, e in chunks:
            assert owner != rank and 0 <= owner < world
            assert off <= b < e <= off + nk
            assert b % 8 == 0 and e % 8 == 0          # 16-byte aligned bf16 ranges
            assert e - b <= 4096                       # at most 8 KB
            assert b // blk == (e - 1) // blk          # inside one block ...
            assert (b // blk) % world == owner         # ... that `owner` owns
            assert b >= last_end                       # address order, no overlap
            last_end = e
            covered += e - b
        want = sum(min((j + 1) * blk, off + nk) - max(j * blk, off)
                   for j in range(off // blk, (off + nk - 1) // blk + 1) if j % world != rank)
        assert covered == want
