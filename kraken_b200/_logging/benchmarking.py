"""Timing harness (reference: kraken/_logging/benchmarking.py:10-163).

``benchmark_with_event`` times each call with CUDA events on the launching stream after warm-up,
optionally flushing L2 (a 256 MB write) before each timed call outside the event pair, optionally
replaying a CUDA graph, and returns the median in microseconds. Unlike the reference (which reports
rank 0's number) ``max_over_ranks=True`` (the default) returns the maximum of the per-rank medians,
because a collective is only done when its slowest rank is. ``benchmark_with_profiler`` returns the
median device time of the kernels whose name matches a regex, from ``torch.profiler``.
"""
from __future__ import annotations

import os
import re
from contextlib import nullcontext
from typing import Callable

import torch
import torch.distributed as dist

L2_FLUSH_BYTES = 256 * 1000 * 1000


def _max_over_ranks(value: float) -> float:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device="cuda" if dist.get_backend() == "nccl" else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _align_ranks() -> None:
    if dist.is_available() and dist.is_initialized():
        if dist.get_backend() == "nccl":
            dist.barrier(device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier()
    torch.cuda.synchronize()


def benchmark_with_event(target_fn: Callable[[], None], warmup_iters: int = 200, benchmark_iters: int = 25,
                         profile_ranks: list[int] | None = None, flush_l2: bool = False, cuda_graph: bool = False,
                         max_over_ranks: bool = True, return_all: bool = False):
    """Median device time of `target_fn` in microseconds (max over ranks by default). With
    ``profile_ranks`` given, those ranks also record a short profiler trace after the timed loop."""
    if cuda_graph:
        target_fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            target_fn()
        inner = g.replay
    else:
        inner = target_fn
    if "BENCHMARK_ITERS" in os.environ:
        benchmark_iters = int(os.environ["BENCHMARK_ITERS"])
    cache = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda") if flush_l2 else None
    for _ in range(warmup_iters):
        inner()
    _align_ranks()
    begin = [torch.cuda.Event(enable_timing=True) for _ in range(benchmark_iters)]
    end = [torch.cuda.Event(enable_timing=True) for _ in range(benchmark_iters)]
    # Queue the launches behind a short device-side spin so host launch overhead is hidden.
    torch.cuda._sleep(int(2e7))
    for i in range(benchmark_iters):
        if cache is not None:
            cache.zero_()
        begin[i].record()
        inner()
        end[i].record()
    torch.cuda.synchronize()
    lat = sorted(b.elapsed_time(e) * 1000.0 for b, e in zip(begin, end))
    med = lat[len(lat) // 2] if len(lat) % 2 else 0.5 * (lat[len(lat) // 2 - 1] + lat[len(lat) // 2])
    if max_over_ranks:
        med = _max_over_ranks(med)
    if profile_ranks is not None:
        _trace_pass(inner, profile_ranks)
    if return_all:
        return med, lat
    return med


def _trace_pass(fn: Callable[[], None], profile_ranks: list[int], iters: int = 3) -> str | None:
    """A few extra calls under ``torch.profiler`` on the ranks named, AFTER the timed loop, so that
    no reported time is taken under a profiler (the reference wraps its timed loop in the profiler:
    kraken/_logging/benchmarking.py:131-152). The trace goes to a user-supplied
    ``trace_handler.trace_handler`` when that module is importable, else as a Chrome trace into
    ``$KRAKEN_TRACE_DIR`` (default: the temp directory). ``NO_TRACE`` in the environment skips it.
    Returns the path written, if any."""
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    if rank not in profile_ranks or "NO_TRACE" in os.environ:
        return None
    try:
        from trace_handler import trace_handler  # user-supplied module, optional
    except ImportError:
        trace_handler = None
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
                                on_trace_ready=trace_handler) as prof:
        for _ in range(iters):
            fn()
        torch.cuda.synchronize()
    if trace_handler is not None:
        return None
    import tempfile

    out_dir = os.environ.get("KRAKEN_TRACE_DIR", tempfile.gettempdir())
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"kraken_b200_trace_rank{rank}_{os.getpid()}.json")
    prof.export_chrome_trace(path)
    return path


def benchmark_with_profiler(target_fn: Callable[[], None], event_key_regex: str, warmup_iters: int = 200,
                            benchmark_iters: int = 25, profile_ranks: list[int] | None = None,
                            flush_l2: bool = False, max_over_ranks: bool = True) -> float:
    """Median device time (microseconds) of profiler events whose name matches `event_key_regex`."""
    if "BENCHMARK_ITERS" in os.environ:
        benchmark_iters = int(os.environ["BENCHMARK_ITERS"])
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    profile_ranks = profile_ranks or [0]
    cache = torch.empty(L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda") if flush_l2 else None
    for _ in range(warmup_iters):
        target_fn()
    _align_ranks()
    trace_handler = None
    if "NO_TRACE" not in os.environ:
        try:
            from trace_handler import trace_handler  # user-supplied module, optional
        except ImportError:
            trace_handler = None
    prof = (torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA],
                                   on_trace_ready=trace_handler)
            if rank in profile_ranks else nullcontext())
    with prof:
        torch.cuda._sleep(int(2e7))
        for _ in range(benchmark_iters):
            if cache is not None:
                cache.zero_()
            target_fn()
        torch.cuda.synchronize()
    med = 0.0
    if rank in profile_ranks:
        pat = re.compile(event_key_regex)
        times = sorted(ev.device_time for ev in prof.events() if pat.search(ev.key) and ev.device_time > 0)
        if times:
            med = float(times[len(times) // 2])
    return _max_over_ranks(med) if max_over_ranks else med


def bus_bandwidth_gbs(op: str, nbytes: int, world_size: int, micros: float) -> float:
    """Bus bandwidth in GB/s: 2(n-1)/n * S / t for all-reduce, (n-1)/n * S / t for all-gather and
    reduce-scatter (S = full tensor bytes)."""
    if micros <= 0 or world_size <= 1:
        return 0.0
    n = world_size
    factor = 2.0 * (n - 1) / n if op == "all_reduce" else (n - 1) / n
    return factor * nbytes / (micros * 1e-6) / 1e9
