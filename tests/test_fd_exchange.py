"""Descriptor exchange between processes (CPU): every rank owns a memfd with its own
contents, hands it to all peers and must be able to read everybody's bytes afterwards."""
import multiprocessing as mp
import os
import time


def _file_all_gather(directory, rank, world):
    """An all-gather over a directory of files (stands in for torch.distributed here)."""
    calls = {"n": 0}

    def gather(payload: bytes):
        n = calls["n"]
        calls["n"] += 1
        tmp = os.path.join(directory, f".tmp-{n}-{rank}")
        with open(tmp, "wb") as f:
            f.write(payload)
        os.rename(tmp, os.path.join(directory, f"{n}-{rank}"))
        out = []
        deadline = time.time() + 30
        for p in range(world):
            path = os.path.join(directory, f"{n}-{p}")
            while not os.path.exists(path):
                assert time.time() < deadline, "peer did not show up"
                time.sleep(0.01)
            with open(path, "rb") as f:
                out.append(f.read())
        return out
    return gather


def _rank_main(directory, rank, world, result):
    from ps_lite_b200.parallel.fd_exchange import exchange_fds
    fd = os.memfd_create(f"rank{rank}")
    os.write(fd, bytes([65 + rank]) * (1000 + rank))
    fds = exchange_fds(rank, world, fd, _file_all_gather(directory, rank, world), timeout_s=30)
    ok = len(fds) == world
    for p, f in enumerate(fds):
        data = os.pread(f, 4096, 0)
        ok = ok and data == bytes([65 + p]) * (1000 + p)
        os.close(f)
    os.close(fd)
    result.put((rank, ok))


def test_every_rank_reads_every_peers_descriptor(tmp_path):
    world = 3
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(str(tmp_path), r, world, result))
             for r in range(world)]
    for p in procs:
        p.start()
    got = dict(result.get(timeout=90) for _ in range(world))
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert got == {0: True, 1: True, 2: True}


def test_single_rank_gets_a_duplicate():
    from ps_lite_b200.parallel.fd_exchange import exchange_fds
    fd = os.memfd_create("solo")
    os.write(fd, b"x")
    fds = exchange_fds(0, 1, fd, lambda b: [b])
    assert len(fds) == 1 and fds[0] != fd and os.pread(fds[0], 1, 0) == b"x"
    os.close(fds[0])
    os.close(fd)
