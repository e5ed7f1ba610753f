"""Host-side extent validation of the dense launcher (no GPU needed: a request whose buffers do
not fit into the arena is refused before anything is launched)."""
import ctypes as C

from ps_lite_b200 import _lib


def _world(heap_bytes):
    w = _lib.World()
    w.rank, w.world = 0, 2
    for p in range(2):
        w.peer_base[p] = 0x10000000 * (p + 1)   # never dereferenced: the call is refused first
    w.heap_bytes = heap_bytes
    return w


def _table(grad_off, weight_off, n):
    t = _lib.Table()
    t.grad_off, t.weight_off, t.n, t.blk = grad_off, weight_off, n, 1024
    t.master = 0x20000000                        # never dereferenced either
    t.grad_dtype, t.out_dtype = 0, 0
    return t


def test_buffers_outside_the_arena_are_refused():
    lib = _lib.device_lib()
    opt = _lib.Opt()
    n = 1 << 20
    heap = 65536 + 2 * 4 * n                      # control region + gradient + weight, exactly
    cases = {
        "weight buffer ends past the arena": (_world(heap - 8), _table(65536, 65536 + 4 * n, n)),
        "gradient buffer inside the control region": (_world(heap), _table(4096, 65536 + 4 * n, n)),
        "offset beyond the arena": (_world(heap), _table(heap + 64, 65536, n)),
    }
    for why, (w, t) in cases.items():
        rc = lib.psdev_dense_op(C.byref(w), C.byref(t), _lib.OP_PUSHPULL, 0, n, C.byref(opt), 0, 0,
                                10**9, 0, None)
        assert rc == -8, why
