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


def test_sparse_descriptor_is_checked_against_the_arena():
    """A layout made the way SparseTable makes it passes the extent check (the call then fails
    later for want of a GPU, or succeeds on a GPU box: anything but -8); one that leaves the
    arena is refused."""
    lib = _lib.device_lib()
    world, max_keys, slots = 2, 1 << 16, 1 << 18
    heap = 1 << 26
    sub = lib.psdev_suballoc_new(heap)
    offs = [lib.psdev_suballoc_alloc(sub, nbytes, 256) for nbytes in
            (8 * max_keys, 4 * max_keys, 4 * max_keys, 8 * (world + 2), 4 * slots)]
    lib.psdev_suballoc_delete(sub)
    assert all(o >= 65536 for o in offs)

    def table(keys_off):
        t = _lib.Sparse()
        t.range = 1 << 20
        t.keys_off, t.grads_off, t.out_off, t.pos_off, t.acc_off = keys_off, *offs[1:]
        t.w = 0x20000000                         # never dereferenced on this path
        t.kind = 0
        t.width, t.channel, t.max_n, t.max_vals, t.slots = 1, 3, max_keys, max_keys, slots
        return t
    w = _world(heap)
    good, bad = table(offs[0]), table(heap - 64)
    rc_bad = lib.psdev_sparse_scatter(C.byref(w), C.byref(bad), max_keys, 1, None)
    assert rc_bad == -8
    import torch
    if not torch.cuda.is_available():            # with a GPU the good call would really launch
        rc_good = lib.psdev_sparse_scatter(C.byref(w), C.byref(good), max_keys, 1, None)
        assert rc_good != -8 and rc_good != -1


def test_multicast_size_rule():
    """Which path a dense launch takes, by ranks and bytes (the measured cross-overs)."""
    lib = _lib.device_lib()
    mib = 1 << 20
    assert lib.psdev_multicast_pays(1, mib) == 0                # nobody to reach
    assert lib.psdev_multicast_pays(4, 1 * mib) == 1
    assert lib.psdev_multicast_pays(4, 4 * mib) == 1
    assert lib.psdev_multicast_pays(4, 16 * mib) == 0           # peer path from 16 MiB on 4 ranks
    assert lib.psdev_multicast_pays(2, 64 * mib) == 0
    assert lib.psdev_multicast_pays(8, 256 * mib) == 1
    assert lib.psdev_multicast_pays(8, 512 * mib) == 1
    assert lib.psdev_multicast_pays(8, 1024 * mib) == 0         # very large: peer path again
