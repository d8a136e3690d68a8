"""The allocation-free all-gather entry point, called through its exported C symbol.

Some users of this library may not allocate device memory themselves mid-run: servers that give
every component a fixed arena up front, or hosts that cannot tolerate the implicit device
synchronisation of an allocation inside their serving loop. For them the library exports
``kr_all_gather_sm_noalloc``, whose arrival counters live in a fixed array inside the library.
This test checks that it produces exactly what the regular entry point produces, on two calls in
a row (the second call sees the scratch the first one left behind), and that oversized requests
are refused. It runs last so that a failure here cannot hide results of the other tests.
"""
import ctypes

import pytest
import torch

from kraken_b200.ops import lib as klib

pytestmark = pytest.mark.gpu


def _symbol():
    handle = ctypes.CDLL(klib.lib_path())
    fn = handle.kr_all_gather_sm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_ulonglong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_ulonglong, ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p,
                   ctypes.c_void_p]
    err = handle.kr_last_error
    err.restype = ctypes.c_char_p
    return fn, err


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
