"""Ops are plain stream-ordered kernel launches with self-resetting flags, so they can be captured
in a CUDA graph and replayed (the reference's harness offers graph replay for its kernels:
kraken/_logging/benchmarking.py:99-108). Single GPU, world size 1."""
import pytest
import torch

from kraken_b200 import comm, fused
from kraken_b200.parallel import symm_mem

pytestmark = pytest.mark.gpu


def test_ops_replay_under_cuda_graph():
    dev = torch.device("cuda", torch.cuda.current_device())
    x = symm_mem.empty(256, 1024, dtype=torch.bfloat16, device=dev)
    symm_mem.rendezvous(x)
    w = (1 + 0.1 * torch.randn(1024, device=dev)).to(torch.bfloat16)
    bt = (0.05 * torch.randn(512, 1024, device=dev)).to(torch.bfloat16)
    x.copy_(torch.randn(256, 1024, device=dev).to(torch.bfloat16))

    def chain():
        y = comm.one_shot_all_reduce(x)           # world size 1: a copy through the kernel
        z = fused.rms_norm(y, w, 1e-5)
        return fused.matmul(z, bt.t())

    ref = chain()                                  # warm-up outside capture (first-use set-up happens here)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = chain()
    for _ in range(3):
        x.copy_(torch.randn(256, 1024, device=dev).to(torch.bfloat16))
        g.replay()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), chain().float(), atol=2e-2, rtol=2e-2)
    assert ref.shape == out.shape


def test_benchmark_harness_times_outside_the_profiler_and_traces_on_request(tmp_path, monkeypatch):
    # profile_ranks asks for a trace: it is recorded in extra calls after the timed loop
    from kraken_b200._logging.benchmarking import benchmark_with_event

    monkeypatch.setenv("KRAKEN_TRACE_DIR", str(tmp_path))
    monkeypatch.delenv("NO_TRACE", raising=False)
    x = torch.randn(1 << 20, device="cuda")
    calls = []

    def fn():
        calls.append(1)
        x.mul_(1.0)

    us = benchmark_with_event(fn, warmup_iters=3, benchmark_iters=5, profile_ranks=[0], flush_l2=True, max_over_ranks=False)
    assert us > 0 and len(calls) == 3 + 5 + 3
    traces = list(tmp_path.glob("kraken_b200_trace_rank0_*.json"))
    assert len(traces) == 1 and traces[0].stat().st_size > 0
    calls.clear()
    us_g = benchmark_with_event(fn, warmup_iters=2, benchmark_iters=5, cuda_graph=True, max_over_ranks=False)
    assert us_g > 0 and len(calls) == 2           # captured once after one eager call; replays do not re-enter Python


def test_capability_queries_are_safe_inside_stream_capture():
    # ops ask whether multicast is supported on every call; under capture the answer must come from
    # a cache (anything that touches the context, like cudaFree, invalidates a capture)
    from kraken_b200.ops import lib as klib

    L = klib.lib()
    before = L.kr_symm_multicast_supported()
    x = torch.randn(1024, device="cuda")
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        assert L.kr_symm_multicast_supported() == before
        y = x * 2
    g.replay()
    torch.cuda.synchronize()
    torch.testing.assert_close(y, x * 2)
