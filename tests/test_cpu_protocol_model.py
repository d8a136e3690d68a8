"""Signal-pad barrier protocol on the host: CPU processes sharing an mmap'd region run the same
semaphore protocol the kernels run over NVLink, including injected failures (no GPU involved)."""
import ctypes
import mmap
import multiprocessing as mp
import os
import tempfile

import pytest

from kraken_b200.ops import lib as klib

PAD_WORDS = 256


def _map(path, ws):
    fd = os.open(path, os.O_RDWR)
    mm = mmap.mmap(fd, ws * PAD_WORDS * 4)
    os.close(fd)
    base = ctypes.addressof(ctypes.c_char.from_buffer(mm))
    return mm, base


def _rank(path, rank, ws, rounds, fault, q):
    L = klib.lib()
    mm, base = _map(path, ws)
    status = []
    # processes start seconds apart (imports): meet once with a generous deadline first
    assert L.kr_host_barrier(base, PAD_WORDS, 7, rank, ws, 60000.0, 0, 0) == 0
    for i in range(rounds):
        skip = 1 if (fault == "lost_signal" and rank == 1 and i == 2) else 0
        extra = 1 if (fault == "double_send" and rank == 1 and i == 2) else 0
        if fault == "absent" and rank == 1 and i >= 2:
            break                                        # this rank never arrives again
        st = L.kr_host_barrier(base, PAD_WORDS, i % 4, rank, ws, 1500.0 if fault != "none" else 20000.0, skip, extra)
        status.append(int(st))
        if st:
            break
    q.put((rank, status, int(L.kr_host_pad_nonzero(base, PAD_WORDS, rank))))


def _run(ws, rounds, fault):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    with tempfile.NamedTemporaryFile(dir="/dev/shm" if os.path.isdir("/dev/shm") else None) as f:
        f.truncate(ws * PAD_WORDS * 4)
        procs = [ctx.Process(target=_rank, args=(f.name, r, ws, rounds, fault, q)) for r in range(ws)]
        for p in procs:
            p.start()
        res = dict()
        for _ in procs:
            r, st, nz = q.get(timeout=60)
            res[r] = (st, nz)
        for p in procs:
            p.join(timeout=30)
    return res


@pytest.mark.parametrize("ws", [2, 4])
def test_barriers_complete_and_pads_return_to_zero(ws):
    res = _run(ws, 200, "none")
    for r in range(ws):
        st, nz = res[r]
        assert len(st) == 200 and not any(st)
        assert nz == 0


def test_absent_rank_is_reported_with_its_rank_number():
    res = _run(3, 6, "absent")
    for r in (0, 2):
        st, _ = res[r]
        assert st[:2] == [0, 0] and st[-1] != 0
        assert klib.decode_status(st[-1]).startswith("cross-device signal wait")
        assert (st[-1] >> 16) & 0xFF == 1            # the peer that never arrived


def test_lost_signal_times_out_only_the_waiters():
    res = _run(2, 6, "lost_signal")
    st0, _ = res[0]
    assert st0[:2] == [0, 0] and st0[2] != 0 and (st0[2] >> 16) & 0xFF == 1


def test_double_send_leaves_a_token_behind():
    # a duplicated signal does not break the barrier that follows, but the pad no longer returns to
    # zero: the invariant the GPU tests check after every op catches exactly this
    res = _run(2, 6, "double_send")
    st0, nz0 = res[0]
    assert not any(st0)
    assert nz0 == 1
