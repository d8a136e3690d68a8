"""Single-GPU tests of the synchronisation primitives (the reference's test/test_ptx_utils.py
checks the same two invariants on 4 GPUs: signal pads return to zero after barriers, and the
gmem arrive/wait pair orders a producer's write before its consumers' reads)."""
import pytest
import torch

import kraken_b200
from kraken_b200 import _ptx_utils as ptx
from kraken_b200.ops import lib as klib
from kraken_b200.parallel import EmuWorld, symm_mem

pytestmark = pytest.mark.gpu


def test_native_library_is_loaded_on_gpu():
    L = klib.lib()
    assert L.kr_num_sms() > 0
    with open("/proc/self/maps") as f:
        assert "libkraken_b200.so" in f.read()


def test_symm_alloc_single_rank_roundtrip():
    t = symm_mem.empty(1024, dtype=torch.float32, device="cuda")
    t.fill_(3.0)
    hdl = symm_mem.rendezvous(t)
    assert hdl.rank == 0 and hdl.world_size == 1
    v = hdl.get_buffer(0, (1024,), torch.float32)
    assert float(v.sum()) == 3.0 * 1024
    pad = hdl.get_signal_pad(0)
    assert int(pad.to(torch.int64).abs().sum()) == 0
    assert symm_mem.rendezvous(t) is hdl      # cached
    hdl.barrier()
    torch.cuda.synchronize()
    assert int(hdl.get_signal_pad(0).to(torch.int64).abs().sum()) == 0


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_symm_mem_barrier_pads_return_to_zero(ws):
    world = EmuWorld(ws)
    ts = world.symmetric((4096,), torch.float32)
    nblocks = 148 // ws if ws > 1 else 32
    outs = world.run(lambda r: ptx.symm_mem_sync(symm_mem.rendezvous(ts[r]), None, r, ws, num_blocks=min(32, nblocks)))
    torch.cuda.synchronize()
    for r in range(ws):
        assert bool((outs[r] == 1).all()), f"rank {r}: a barrier wait failed"
    for r in range(ws):
        with world.rank(r):
            hdl = symm_mem.rendezvous(ts[r])
        assert int(hdl.get_signal_pad(r).to(torch.int64).abs().sum()) == 0


def test_gmem_barrier_arrive_wait():
    flags, seen = ptx.gmem_barrier_test(num_producers=8, num_blocks=40)
    torch.cuda.synchronize()
    assert bool((flags == 1).all())
    assert bool((seen == 7).all())


@pytest.mark.expects_timeout
def test_bounded_wait_reports_timeout_and_context_survives():
    L = klib.lib()
    old = L.kr_get_timeout_ms()
    klib.check(L.kr_set_timeout_ms(5.0))
    try:
        out = ptx.wait_timeout_test(num_blocks=4)
        with pytest.raises(kraken_b200.KrakenSyncTimeout):
            kraken_b200.check_status()
        assert bool((out == 2).all())
        # the context is still usable and the status is clear again
        x = torch.ones(16, device="cuda")
        assert float(x.sum()) == 16.0
        kraken_b200.check_status()
    finally:
        klib.check(L.kr_set_timeout_ms(old))


@pytest.mark.parametrize("ws", [2, 4])
@pytest.mark.parametrize("prev,subseq", [(False, False), (False, True), (True, False), (True, True)])
def test_symm_mem_sync_single_pattern(ws, prev, subseq):
    # the reference's signature: one barrier of the pattern named by the two flags
    world = EmuWorld(ws)
    ts = world.symmetric((64,), torch.float32)
    outs = world.run(lambda r: ptx.symm_mem_sync(symm_mem.rendezvous(ts[r]), None, r, ws, prev, subseq, num_blocks=3))
    torch.cuda.synchronize()
    for r in range(ws):
        assert outs[r].tolist() == [1, 1, 1]
        with world.rank(r):
            hdl = symm_mem.rendezvous(ts[r])
        assert int(hdl.get_signal_pad(r).to(torch.int64).abs().sum()) == 0      # every token consumed
