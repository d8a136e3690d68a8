"""The allocation-free all-gather entry point, called through its exported C symbol.

Some users of this library may not allocate device memory themselves mid-run: servers that give
every component a fixed arena up front, or hosts that cannot tolerate the implicit device
synchronisation of an allocation inside their serving loop. For them the library exports
``kr_all_gather_sm_noalloc``, whose arrival counters live in a fixed array inside the library.
This test checks that it produces exactly what the regular entry point produces, on two calls in
a row (the second call sees the scratch the first one left behind), and that oversized requests
are refused; that the built-in status word (used when the caller passes none) reports a wait that
gave up and does not poison the calls after it. It runs last so that a failure here cannot hide
results of the other tests.
"""
import ctypes

import pytest
import torch

from kraken_b200.ops import lib as klib

pytestmark = pytest.mark.gpu


def _symbol():
    klib.lib()                                       # builds the library first when it is missing or stale
    handle = ctypes.CDLL(klib.lib_path())
    fn = handle.kr_all_gather_sm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p,
                   ctypes.c_void_p]
    err = handle.kr_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def _status_symbols():
    klib.lib()
    handle = ctypes.CDLL(klib.lib_path())
    rd = handle.kr_noalloc_read_status
    rd.restype = ctypes.c_int
    rd.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32), ctypes.c_int]
    st = handle.kr_noalloc_set_timeout_ms
    st.restype = ctypes.c_int
    st.argtypes = [ctypes.c_double]
    return rd, st


def test_no_alloc_all_gather_matches_regular_entry_point():
    fn, err = _symbol()
    L = klib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    rows, cols, splits = 512, 1024, 4
    stream = torch.cuda.current_stream().cuda_stream
    pad = torch.zeros(2304, dtype=torch.int32, device=dev)                 # caller-owned signal pad
    pads = torch.tensor([pad.data_ptr()], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for call in range(2):
        shard = torch.randn(rows, cols, generator=torch.Generator().manual_seed(100 + call)).to(torch.bfloat16).to(dev)
        bufs = torch.tensor([shard.data_ptr()], dtype=torch.int64, device=dev)
        out_new = torch.full((rows, cols), float("nan"), dtype=torch.bfloat16, device=dev)
        out_old = torch.full((rows, cols), float("nan"), dtype=torch.bfloat16, device=dev)
        prog_new = torch.zeros(splits, dtype=torch.int32, device=dev)
        prog_old = torch.zeros(splits, dtype=torch.int32, device=dev)
        counters = torch.zeros(splits, dtype=torch.int32, device=dev)
        rc = fn(bufs.data_ptr(), 0, pads.data_ptr(), 0, 1, out_new.data_ptr(), prog_new.data_ptr(), splits,
                shard.numel(), 0, 0, status.data_ptr(), stream)
        assert rc == 0, err().decode()
        klib.check(L.kr_all_gather_sm(bufs.data_ptr(), 0, pads.data_ptr(), 0, 1, out_old.data_ptr(),
                                      prog_old.data_ptr(), counters.data_ptr(), splits, shard.numel(), 0, 0, stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(out_new, out_old)          # a copy: the tolerance is exact equality
        assert torch.equal(out_new, shard)
        assert torch.equal(prog_new, prog_old) and bool((prog_new == 1).all())
        assert int(pad.abs().sum()) == 0              # barrier slots are back to zero


def test_no_alloc_rejects_requests_beyond_its_scratch():
    fn, err = _symbol()
    dev = torch.device("cuda", torch.cuda.current_device())
    x = torch.zeros(8 * 2048, dtype=torch.bfloat16, device=dev)
    bufs = torch.tensor([x.data_ptr()], dtype=torch.int64, device=dev)
    pad = torch.zeros(2304, dtype=torch.int32, device=dev)
    pads = torch.tensor([pad.data_ptr()], dtype=torch.int64, device=dev)
    out = torch.empty_like(x)
    prog = torch.zeros(2048, dtype=torch.int32, device=dev)
    rc = fn(bufs.data_ptr(), 0, pads.data_ptr(), 0, 1, out.data_ptr(), prog.data_ptr(), 2048, x.numel(), 0, 0, None,
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
    assert "exceeds the built-in scratch" in err().decode()


def test_no_alloc_built_in_status_word_success_path():
    # status = NULL: the library's own word is used, cleared at the start of the call, and reads 0
    fn, err = _symbol()
    rd, _ = _status_symbols()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    shard = torch.randn(256, 512, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(dev)
    bufs = torch.tensor([shard.data_ptr()], dtype=torch.int64, device=dev)
    pad = torch.zeros(2304, dtype=torch.int32, device=dev)
    pads = torch.tensor([pad.data_ptr()], dtype=torch.int64, device=dev)
    for _ in range(2):
        out = torch.full_like(shard, float("nan"))
        prog = torch.zeros(2, dtype=torch.int32, device=dev)
        rc = fn(bufs.data_ptr(), 0, pads.data_ptr(), 0, 1, out.data_ptr(), prog.data_ptr(), 2, shard.numel(), 0, 0, None,
                stream)
        assert rc == 0, err().decode()
        word = ctypes.c_uint32(123)
        assert rd(stream, ctypes.byref(word), 0) == 0
        assert word.value == 0
        assert torch.equal(out, shard) and bool((prog == 1).all())


@pytest.mark.expects_timeout
def test_no_alloc_timeout_is_reported_and_does_not_stick():
    # A host-made failure: the call claims a world of two ranks, but the "peer" is a zeroed pad that
    # nothing ever signals from, so the entry barrier's wait runs out after a few milliseconds. The
    # kernel returns, the built-in status word says so, and the next call works.
    fn, err = _symbol()
    rd, set_timeout = _status_symbols()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream().cuda_stream
    shard = torch.ones(64, 64, dtype=torch.bfloat16, device=dev)
    peer = torch.zeros(64, 64, dtype=torch.bfloat16, device=dev)
    pad_own = torch.zeros(2304, dtype=torch.int32, device=dev)
    pad_peer = torch.zeros(2304, dtype=torch.int32, device=dev)
    bufs2 = torch.tensor([shard.data_ptr(), peer.data_ptr()], dtype=torch.int64, device=dev)
    pads2 = torch.tensor([pad_own.data_ptr(), pad_peer.data_ptr()], dtype=torch.int64, device=dev)
    out2 = torch.zeros(128, 64, dtype=torch.bfloat16, device=dev)
    prog2 = torch.zeros(2, dtype=torch.int32, device=dev)
    assert set_timeout(5.0) == 0
    try:
        rc = fn(bufs2.data_ptr(), 0, pads2.data_ptr(), 0, 2, out2.data_ptr(), prog2.data_ptr(), 1, shard.numel(), 1, 0,
                None, stream)
        assert rc == 0, err().decode()
        word = ctypes.c_uint32(0)
        assert rd(stream, ctypes.byref(word), 0) == 0
        assert word.value != 0 and (word.value & 0xFF) == 1          # cross-device signal wait ran out
        assert int(prog2.abs().sum()) == 0                              # nothing was reported as landed
    finally:
        assert set_timeout(0.0) == 0
    assert float(torch.ones(4, device=dev).sum()) == 4.0                # the context is alive
    # next call with the built-in word: cleared on entry, succeeds
    bufs1 = torch.tensor([shard.data_ptr()], dtype=torch.int64, device=dev)
    pad = torch.zeros(2304, dtype=torch.int32, device=dev)
    pads1 = torch.tensor([pad.data_ptr()], dtype=torch.int64, device=dev)
    out1 = torch.zeros(64, 64, dtype=torch.bfloat16, device=dev)
    prog1 = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = fn(bufs1.data_ptr(), 0, pads1.data_ptr(), 0, 1, out1.data_ptr(), prog1.data_ptr(), 1, shard.numel(), 0, 0, None,
            stream)
    assert rc == 0, err().decode()
    assert rd(stream, ctypes.byref(word), 1) == 0
    assert word.value == 0
    assert torch.equal(out1, shard) and int(prog1.item()) == 1
