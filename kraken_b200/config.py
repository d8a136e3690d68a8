"""Environment-backed settings of the library (the reference has only kwargs and three env vars:
``BENCHMARK_ITERS``, ``NO_TRACE``, ``SYMM_DUMP_KERNEL`` — kraken/_logging/benchmarking.py:34,49,
kraken/comm/two_shot_all_reduce.py:153).

=========================  ==========================================================================
``KRAKEN_SYNC_TIMEOUT_MS``  deadline of every device-side wait (default 4000)
``KRAKEN_NVLS``             ``0`` disables NVLS multicast binding and the multimem kernels (default 1)
``KRAKEN_SIGNAL_PAD_BYTES`` signal-pad size of blocks from the native allocator (default 1 MiB)
``KRAKEN_FORCE_ALGO``       ``one_shot`` / ``two_shot`` / ``multimem``: overrides all-reduce selection
``KRAKEN_NUM_COMM_SMS``     comm CTAs of the in-kernel all-gather engine (default: from the problem shape)
``KRAKEN_GEMM_PAIR``        ``0`` forces the single-CTA GEMM kernel (default: CTA pairs when eligible)
``KRAKEN_GEMM_GROUP``       row tiles per column sweep of the GEMM tile order (default 16)
``KRAKEN_TMA_STORE``        ``0`` makes the GEMM epilogue use vector stores instead of TMA stores
``KRAKEN_AG_MODE``          engine of the fused all-gather GEMM: ``auto`` (default: ``push``; ``ce`` above 2 ranks when
                            the workspace has no multicast mapping),
                            ``push`` (comm CTAs write the own shard into the peers' gathered buffers), ``ce`` (copy
                            engines + stream flags) or ``sm`` (comm CTAs pull the peers' shards)
``KRAKEN_AG_MC``            ``0`` / ``1``: whether the push engine writes once through the NVSwitch (multimem.st); default:
                            above 2 ranks when a multicast mapping exists
``KRAKEN_RS_ALGO``          ``scatter`` (default: tiles are stored into the owner's staging, reducer warps sum local
                            memory), ``pull`` (reducer warps sum the ranks' staged tiles with peer loads) or
                            ``push`` (tiles are stored into the owner's staging and summed in its epilogue)
``KRAKEN_ONE_SHOT``         ``push`` (default: small one-shot all-reduces write into the peers' workspace and meet in
                            one barrier) or ``pull`` (copy-in, barrier, remote loads, exit barrier)
``KRAKEN_RS_NVLS``          ``1``: the pull reduce-scatter sums with ``multimem.ld_reduce`` (default 0: peer loads)
``KRAKEN_DEBUG``            ``1`` loads the debug build of the native library (device-side bounds checks that record
                            an error code and skip the access; built on first use)
``KRAKEN_NVTX``             ``1`` wraps every public op in an NVTX range named after it (for timeline tools)
``KRAKEN_DUMP_KERNEL``      ``1`` prints the kernel variant / tiling each op picks (rank 0)
``KRAKEN_SYMM_BACKEND``     ``native`` (default) or ``torch`` (torch.distributed._symmetric_memory)
``BENCHMARK_ITERS``         overrides the iteration count of the timing harness
=========================  ==========================================================================
"""
from __future__ import annotations

import os


def _env_int(name: str, default: int) -> int:
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def sync_timeout_ms() -> float:
    try:
        return float(os.environ.get("KRAKEN_SYNC_TIMEOUT_MS", 4000))
    except ValueError:
        return 4000.0


def nvls_enabled() -> bool:
    return os.environ.get("KRAKEN_NVLS", "1") != "0"


def signal_pad_bytes() -> int:
    v = _env_int("KRAKEN_SIGNAL_PAD_BYTES", 1 << 20)
    return max(16384, (v + 15) // 16 * 16)


def force_algo() -> str | None:
    v = os.environ.get("KRAKEN_FORCE_ALGO", "").strip().lower()
    return v or None


def num_comm_sms() -> int:
    return max(1, _env_int("KRAKEN_NUM_COMM_SMS", 8))


def ag_mode() -> str:
    v = os.environ.get("KRAKEN_AG_MODE", "auto").strip().lower()
    return v if v in ("auto", "push", "sm", "ce") else "auto"


def ag_multicast(world_size: int) -> bool:
    """Whether the push engine of the all-gather GEMM writes through the NVSwitch (multimem.st) when
    the gathered buffer has a multicast mapping. Default: above 2 ranks. A comm CTA forwards about
    10 GB/s with multimem.st and about 20 GB/s with bulk stores to one peer, but the multicast form
    sends one copy instead of ws - 1: measured fastest engine at 8 GPUs (359 us against 371 us for
    the copy engines at M = 8192), slower than peer-by-peer stores at 2. KRAKEN_AG_MC=0/1 forces."""
    v = os.environ.get("KRAKEN_AG_MC", "")
    if v in ("0", "1"):
        return v == "1"
    return world_size > 2


def rs_algo() -> str:
    v = os.environ.get("KRAKEN_RS_ALGO", "scatter").strip().lower()
    return v if v in ("pull", "push", "scatter") else "scatter"


def one_shot_mode() -> str:
    v = os.environ.get("KRAKEN_ONE_SHOT", "push").strip().lower()
    return v if v in ("push", "pull") else "push"


def rs_nvls() -> bool:
    """Whether the pull reduce-scatter sums in the NVSwitch (multimem.ld_reduce) instead of with
    peer loads. Off by default: measured at 2 GPUs, 16-byte multimem.ld_reduce requests delivered
    about 90 GB/s per GPU next to a running GEMM, far below what peer loads reach."""
    return os.environ.get("KRAKEN_RS_NVLS", "0") == "1"


def _env_float(name: str, default: float) -> float:
    try:
        return float(os.environ.get(name, default))
    except ValueError:
        return default


def gemm_flops_per_s() -> float:
    """Sustained bf16 rate of the GEMM core that sizing heuristics assume (how many comm CTAs an
    all-gather GEMM needs to keep up). Measured on B200 under the power cap: about 1.45 PFLOP/s.
    KRAKEN_GEMM_TFLOPS overrides (TFLOP/s)."""
    return _env_float("KRAKEN_GEMM_TFLOPS", 1450.0) * 1e12


def comm_cta_bytes_per_s(engine: str) -> float:
    """What one comm CTA of an in-kernel all-gather engine moves over NVLink, as measured at 2 and 8
    GPUs: "pull" (bulk async copies from a peer) about 15 GB/s, "push" (bulk stores to one peer)
    about 20 GB/s, "multicast" (multimem.st from registers) about 10 GB/s. Bounded by what the CTA
    keeps in flight over the link latency. KRAKEN_COMM_CTA_GBS_<ENGINE> overrides (GB/s)."""
    default = {"pull": 15.0, "push": 20.0, "multicast": 10.0}[engine]
    return _env_float("KRAKEN_COMM_CTA_GBS_" + engine.upper(), default) * 1e9


def push_tagged_max_bytes(world_size: int = 8) -> int:
    """Messages up to this size take the tagged form of the push-style one-shot all-reduce (data and
    a per-call tag in one 8-byte store, no barrier at all); larger ones the flag form (one barrier).
    Measured at 2 ranks: the tagged form wins up to 512 KB (15.4 us against 18.5 us) and loses at
    1 MB (20.4 against 18.5); with more peers every byte goes out once per peer and twice as wide, so
    the default stays at 64 KB there. KRAKEN_PUSH_TAGGED_KB overrides; 0 turns the tagged form off."""
    return _env_int("KRAKEN_PUSH_TAGGED_KB", 512 if world_size <= 2 else 64) << 10


def dump_kernel() -> bool:
    return os.environ.get("KRAKEN_DUMP_KERNEL", "0") == "1"


def nvtx_enabled() -> bool:
    return os.environ.get("KRAKEN_NVTX", "0") == "1"


def symm_backend() -> str:
    v = os.environ.get("KRAKEN_SYMM_BACKEND", "native").strip().lower()
    return v if v in ("native", "torch") else "native"


# Signal-pad layout (uint32 words). Words [0, BARRIER_WORDS) are per-block barrier slots
# (slot = block_id * world_size + src_rank, the reference's layout); the fused GEMM kernels keep
# their per-tile flags from TILE_FLAG_BASE on. A 9216-byte pad (torch's default) only has the
# barrier region, which is all the memory-bound kernels need.
BARRIER_WORDS = 2304
TILE_FLAG_BASE = 4096
