"""Fused GEMM + collective ops on the tcgen05 kernels.

Signatures follow the reference: kraken/fused/all_gather_matmul.py:222-325,
kraken/fused/gemm_one_shot_all_reduce_fused.py:106-178,
kraken/fused/gemm_reduce_scatter_fused.py:152-235,
kraken/fused/gemm_reduce_scatter_ce_persistent.py:326-375. The Triton tiling kwargs
(``block_size_*``, ``BLOCK_SIZE_*``, ``group_size_m``, ``num_stages``, ``num_warps``) are accepted and
ignored: tile shapes are chosen by the library (128 x 256 x 64, or 128 x {16..128} with the
operands swapped for decode-sized M).
"""
from __future__ import annotations

import ctypes

import torch

from .. import _reference as ref
from .. import config
from .._logging import utils as _log
from ..ops import lib as _lib
from ..parallel import symm_mem
from .gemm_common import as_k_major_a, as_k_major_bt, use_tf32


def matmul(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16, **kwargs) -> torch.Tensor:
    """Single-GPU C = A @ B on the library's tcgen05 kernel (bf16 inputs, or fp32 inputs multiplied as
    tf32; fp32 accumulate).
    Not in the reference's API; it is the compute core of every fused op, exposed for tests and
    roofline measurements. kwargs: swap_ab (-1 auto / 0 / 1), bn (column-tile override), max_ctas,
    pair (0 forces the single-CTA kernel; default lets large shapes use CTA pairs)."""
    if a.device.type != "cuda":
        return ref.matmul_f32(a, b).to(out_dtype)
    tf32 = use_tf32(a, b) and kwargs.get("tf32", True)
    a2, lda = as_k_major_a(a, tf32)
    bt, ldb = as_k_major_bt(b, tf32)
    M, K = a2.shape
    N = bt.shape[0]
    if bt.shape[1] != K:
        raise ValueError("inner dimensions differ")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("output must be bfloat16 or float32")
    out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _lib.check(_lib.lib().kr_gemm_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, out.data_ptr(), N, M, N, K,
                                       1 if out_dtype == torch.float32 else 0, int(kwargs.get("swap_ab", -1)),
                                       int(kwargs.get("bn", 0)), int(kwargs.get("max_ctas", 0)),
                                       int(kwargs.get("pair", 1)), 1 if tf32 else 0, _lib.current_stream_ptr()))
    return out


_ag_counters: dict[int, torch.Tensor] = {}


def _zero_counters(device: torch.device, n: int, emu) -> torch.Tensor:
    if emu is not None:
        t = torch.zeros(n, dtype=torch.int32, device=device)
        emu._keep.append(t)
        return t
    t = _ag_counters.get(device.index)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 1024), dtype=torch.int32, device=device)
        _ag_counters[device.index] = t
    return t


def _default_comm_ctas(n_local: int, ws: int) -> int:
    """Comm CTAs of the in-kernel PULL engine. The first remote shard must land by the time the MMA
    CTAs finish the local one, which needs M*K*2 bytes per GEMM time = (tensor rate) / N_local bytes
    per second whatever the world size; one comm CTA was measured to pull about 15 GB/s over NVLink
    (its copies in flight cover only a fraction of the link's latency-bandwidth product).
    KRAKEN_NUM_COMM_SMS overrides."""
    import os

    if "KRAKEN_NUM_COMM_SMS" in os.environ:
        return config.num_comm_sms()
    if ws == 1:
        return 2
    rate = config.gemm_flops_per_s() / max(1, n_local)            # bytes per second needed
    n = int(-(-rate // config.comm_cta_bytes_per_s("pull")))
    n = (n + 1) & ~1
    return max(2, min(32, n))


def _default_push_ctas(shard_bytes: int, ws: int, flops: float, multicast: bool) -> int:
    """Comm CTAs of the PUSH engine. Unicast: each rank writes ws copies of its shard during the GEMM
    and a comm CTA (local memory -> shared memory -> peer, bounded by what its shared memory keeps
    in flight) was measured at about 20 GB/s. Multicast: one copy, forwarded from registers at about
    10 GB/s per comm CTA. KRAKEN_NUM_COMM_SMS overrides."""
    import os

    if "KRAKEN_NUM_COMM_SMS" in os.environ:
        return config.num_comm_sms()
    t_gemm = flops / config.gemm_flops_per_s()
    if multicast:
        return 8           # measured at 8 GPUs: 4 starve the GEMM, 16 cost more SMs than they save (M = 2048 and 8192)
    else:
        rate = ws * shard_bytes / max(t_gemm, 1e-6)
        n = int(-(-rate // config.comm_cta_bytes_per_s("push")))
    n = (n + 1) & ~1
    return max(2, min(16, n))


_AG_FLAG_BANK = 2048      # chunk flags per bank in the signal pad (two banks from TILE_FLAG_BASE on)


def all_gather_matmul(a_shared: torch.Tensor, b: torch.Tensor, a_out: torch.Tensor | None = None,
                      progress: torch.Tensor | None = None, **kwargs) -> tuple[torch.Tensor, torch.Tensor]:
    """(gathered A [M, K], C [M, N] = gathered A @ b). `a_shared` is this rank's [M/ws, K] shard in
    symmetric memory. The persistent tcgen05 GEMM starts on the local shard (rank pivot) and
    consumes remote chunks as their flags appear. Engines that move the shards (kwarg ``backend``):

    * ``"push"`` (default): comm CTAs of the same launch write this rank's shard into every rank's
      gathered buffer and raise the chunk's flag in the signal pads: once, through the NVSwitch
      (``multimem.st`` / ``multimem.red``), when the gathered buffer has a multicast mapping — the
      tile order after the own shard then goes chunk by chunk over all peers, as the data arrives —
      else peer by peer with posted bulk stores, the rank that needs the shard first served first
      (``multicast=False`` forces this form). One launch, no barrier, no second stream. The
      gathered buffer must be symmetric: with ``a_out=None`` the op returns a view of a
      double-buffered library workspace, valid until the second next call on the same group; a
      symmetric ``a_out`` is written in place (at the price of an entry barrier); an ordinary
      ``a_out`` receives a device copy of the workspace afterwards.
    * ``"ce"``: copy engines on a backend stream, one stream memory operation per chunk (the
      reference's recipe, kraken/fused/all_gather_matmul.py:296-304).
    * ``"sm"``: comm CTAs pull the peers' shards with bulk async copies.

    kwargs: splits_per_rank=1, num_comm_sms, backend, group."""
    group = kwargs.get("group")
    if a_shared.device.type != "cuda":
        a, c = ref.all_gather_matmul(a_shared, b, group)
        if progress is not None:
            progress.fill_(1)
        if a_out is not None:
            a_out.copy_(a)
            a = a_out
        return a, c
    if a_shared.dtype != torch.bfloat16 or not a_shared.is_contiguous():
        raise TypeError("a_shared must be a contiguous bfloat16 symmetric tensor")
    hdl = symm_mem.rendezvous(a_shared, group)
    ws, rank = hdl.world_size, hdl.rank
    shard_rows, K = a_shared.shape
    M = shard_rows * ws
    bt, ldb = as_k_major_bt(b)
    N = bt.shape[0]
    if bt.shape[1] != K or K % 8:
        raise ValueError("inner dimensions must match and be a multiple of 8")
    splits = int(kwargs.get("splits_per_rank", 1))
    if shard_rows % splits:
        splits = 1
    dev = a_shared.device
    backend = kwargs.get("backend", config.ag_mode())
    emu = hdl.group.emu
    if backend == "auto":
        # Measured: a comm CTA moves 10-20 GB/s (what its shared memory keeps in flight). Pushing
        # ws - 1 copies of a shard peer by peer needs 8 CTAs at 2 ranks and far too many at 8; ONE
        # multicast copy through the NVSwitch needs 8 at any world size and was the fastest engine at
        # 8 GPUs. Without a multicast mapping the copy engines take over above 2 ranks.
        mc_ok = config.nvls_enabled() and config.ag_multicast(ws) and emu is None and bool(_lib.lib().kr_symm_multicast_supported())
        backend = "push" if (ws <= 2 or mc_ok) else "ce"
    if backend not in ("push", "ce", "sm"):
        raise ValueError("backend must be 'push', 'ce' or 'sm'")
    if backend == "ce" and (emu is not None or ws == 1):
        backend = "sm"
    if backend == "push" and (ws == 1 or ws * splits > _AG_FLAG_BANK):
        backend = "sm"
    if hdl.offset_of(a_shared):
        raise ValueError("a_shared must start at the beginning of its symmetric buffer")
    c = torch.empty((M, N), dtype=a_shared.dtype, device=dev)
    counters = _zero_counters(dev, ws * splits + 1, emu)
    L = _lib.lib()
    _log.log_kernel_choice("all_gather_matmul", f"M={M} N={N} K={K} ws={ws} splits={splits} engine={backend}")
    stream = _lib.current_stream_ptr()
    if progress is not None:
        progress.zero_()

    if backend == "push":
        user_out = a_out
        if a_out is not None and symm_mem.is_symm_tensor(a_out):
            oh = symm_mem.rendezvous(a_out, group)            # caller-owned symmetric buffer: written in place
            off, gathered, barrier, user_out = oh.offset_of(a_out), a_out, 1, None
        else:
            half = -(-M * K * 2 // 1024) * 1024
            oh = symm_mem.get_symm_mem_workspace(group, 2 * half, dev, kind="ag_out")
            barrier = 0
            off = None
        calls = getattr(oh, "_ag_calls", 0)
        oh._ag_calls = calls + 1
        if symm_mem.capturing():
            calls, barrier = 0, 1       # a replayed graph repeats one half / flag bank: protect it with the entry barrier
        if off is None:
            off = (calls & 1) * half
            gathered = oh.get_buffer(rank, (M, K), torch.bfloat16, storage_offset=off // 2)
        flag_base = config.TILE_FLAG_BASE + (calls & 1) * _AG_FLAG_BANK
        use_mc = bool(oh.multicast_ptr) and bool(kwargs.get("multicast", config.ag_multicast(ws)))
        if use_mc and progress is None and "splits_per_rank" not in kwargs:
            # all shards arrive at the same pace: finer chunks let the GEMM start sooner
            splits = 4 if shard_rows % 1024 == 0 else (2 if shard_rows % 256 == 0 else 1)
        mc_out = oh.multicast_ptr + off if use_mc else None
        mc_flags = oh.multicast_ptr + oh.buffer_size + 4 * flag_base if use_mc else None
        n_comm = int(kwargs.get("num_comm_sms", 0)) or _default_push_ctas(shard_rows * K * 2, ws, 2.0 * M * N * K, use_mc)
        _lib.check(L.kr_ag_gemm_bf16(oh.buffer_ptrs_dev, oh.signal_pad_ptrs_dev, a_shared.data_ptr(), rank, ws,
                                     gathered.data_ptr(), bt.data_ptr(), ldb, c.data_ptr(), N, shard_rows, N, K, splits,
                                     progress.data_ptr() if progress is not None else None, counters.data_ptr(), n_comm,
                                     0, 1, off, flag_base, oh.signal_pad_words, barrier, mc_out, mc_flags, stream))
        if user_out is not None:
            user_out.copy_(gathered)
            gathered = user_out
        return gathered, c

    if a_out is None:
        a_out = torch.empty((M, K), dtype=a_shared.dtype, device=dev)
    if progress is None:
        progress = torch.zeros(ws * splits, dtype=torch.uint32, device=dev)
    args_tail = (0, 0, 0, 0, 0, None, None, stream)     # the push arguments (unused)
    if ws == 1 and emu is None:
        # nothing to gather: a device copy fills a_out while the GEMM reads the shard in place
        a_out.copy_(a_shared)
        progress.fill_(1)
        n_comm = -1
    elif backend == "ce":
        from ..comm.all_gather import _copy_engine_all_gather_w_progress

        ce_stream = _copy_engine_all_gather_w_progress(a_out, a_shared, progress, splits)
        n_comm = -1
    else:
        n_comm = int(kwargs.get("num_comm_sms", 0)) or _default_comm_ctas(N, ws)
    _lib.check(L.kr_ag_gemm_bf16(hdl.buffer_ptrs_dev, hdl.signal_pad_ptrs_dev, a_shared.data_ptr(), rank, ws,
                                 a_out.data_ptr(), bt.data_ptr(), ldb, c.data_ptr(), N, shard_rows, N, K, splits,
                                 progress.data_ptr(), counters.data_ptr(), n_comm, 0, *args_tail))
    if backend == "ce" and n_comm == -1 and ws > 1:
        torch.cuda.current_stream().wait_stream(ce_stream)
    return a_out, c


_AR_ALGOS = {"one_shot": 0, "two_shot": 1, "push": 2, "push_two_shot": 3}


def gemm_one_shot_all_reduce(a: torch.Tensor, b: torch.Tensor, **kwargs) -> torch.Tensor:
    """fp32 [M, N] = all_reduce(a @ b): each rank holds a K-shard of both operands. One kernel:
    the GEMM epilogue exchanges fp32 partial tiles; there is no grid-wide barrier. Three exchanges:
    "push" (decode-sized M) — the epilogue writes every partial element, paired with a per-call tag
    in one 8-byte store, straight into a slot of every rank's staging; each rank then sums its own
    slots as the tagged pairs land (no flag, no fence, one NVLink crossing); "one_shot" — the
    partial tile goes to the own staging, a flag to every peer, and every rank sums the tile from
    all ranks (in the NVSwitch when the staging buffer has a multicast mapping); "two_shot" (larger
    outputs) — tile owner t % ws receives all partials, sums them in rank order and publishes the
    result, which moves ws/2 times fewer bytes; "push_two_shot" — the two-shot exchange with tagged
    pairs instead of flags in both directions (decode rows at larger world sizes, where pushing
    every partial to every rank is too many bytes). Small M also splits K over several CTAs per tile so
    that more SMs stream the weights; the splits are extra slots of the same exchange. The launcher
    picks exchange and split count by a cost model. Every rank gets identical bits. Decode-sized M
    puts the weights on the 128-row side of the MMA. bf16 operands use the bf16 tensor-core path;
    fp32 x fp32 operands are multiplied as tf32 (what ``tl.dot`` does for the reference's fp32
    tests); anything else is cast to bf16.
    kwargs: group, swap_ab, algo="push"|"push_two_shot"|"one_shot"|"two_shot", k_splits=1..4."""
    group = kwargs.get("group")
    if a.device.type != "cuda":
        return ref.gemm_all_reduce(a, b, group)
    tf32 = use_tf32(a, b)
    a2, lda = as_k_major_a(a, tf32)
    bt, ldb = as_k_major_bt(b, tf32)
    M, K = a2.shape
    N = bt.shape[0]
    if bt.shape[1] != K or (K * a2.element_size()) % 16:
        raise ValueError("inner dimensions must match and K rows must be whole 16-byte units")
    info = symm_mem.resolve_group(group)
    out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    L = _lib.lib()
    if info.world_size == 1:
        _lib.check(L.kr_gemm_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, out.data_ptr(), N, M, N, K, 1, -1, 0, 0, 1,
                                  1 if tf32 else 0, _lib.current_stream_ptr()))
        return out
    ws = info.world_size
    mn4 = M * N * 4
    # one-shot: an eighth of the buffer per staging half; two-shot: ws partial slots + the result in
    # the upper half (twice the slots for decode-sized outputs, so that K can be split in two)
    need = max(8 * mn4, 2 * (ws + 1) * mn4, 2 * (2 * ws + 1) * mn4 if mn4 <= (4 << 20) else 0)
    # tagged push: ws * k_splits slots of {value, tag} pairs in an eighth of the buffer; sized for when
    # it is asked for, and up to 64 MB so that the cost model may pick it for decode-sized outputs
    ll = 8 * ws * max(int(kwargs.get("k_splits", 0)), 1) * M * N * 8
    need = max(need, ll if kwargs.get("algo") == "push" else min(2 * ll, 64 << 20) if M <= 64 else 0)
    if kwargs.get("algo") == "push_two_shot":       # (splits + 1) arrays of M x N pairs, slots padded to whole tiles
        need = max(need, 8 * (max(int(kwargs.get("k_splits", 0)), 1) + 2) * max(M, 16) * N * 8)
    hdl = symm_mem.get_symm_mem_workspace(group, need, a.device, kind="gemm_ar")
    calls = getattr(hdl, "_gemm_ar_calls", 0)      # per staging buffer: selects the staging half, flag bank and tag
    hdl._gemm_ar_calls = calls + 1
    want = kwargs.get("algo", config.force_algo() or "")
    algo = _AR_ALGOS.get(str(want), -1)
    if symm_mem.capturing():
        algo = 1                        # the others alternate staging halves (and tags) call by call: not replayable
    host = getattr(hdl, "_host_ptr_array", None)
    mc = hdl.multicast_ptr or None
    if _log.dump_enabled():
        plan = (ctypes.c_int * 5)()
        _lib.check(L.kr_gemm_ar_plan(M, N, K, ws, 1 if tf32 else 0, algo, int(kwargs.get("k_splits", 0)),
                                     hdl.buffer_size // 1024 * 1024, 1 if host is not None else 0, plan))
        _log.log_kernel_choice("gemm_one_shot_all_reduce", f"M={M} N={N} K={K} ws={ws} "
                               f"exchange={('one_shot', 'two_shot', 'push', 'push_two_shot')[plan[0]]} k_splits={plan[1]} "
                               f"bn={plan[2]} ctas={plan[3]} nvls={bool(mc)}")
    _lib.check(L.kr_gemm_ar_bf16(hdl.buffer_ptrs_dev, host, hdl.signal_pad_ptrs_dev, mc, hdl.rank, ws,
                                 a2.data_ptr(), lda, bt.data_ptr(), ldb, out.data_ptr(), N, M, N, K,
                                 int(kwargs.get("swap_ab", -1)), algo, int(kwargs.get("k_splits", 0)),
                                 calls & 0xFFFFFFFF, config.TILE_FLAG_BASE,
                                 hdl.signal_pad_words, hdl.buffer_size // 1024 * 1024, 1 if tf32 else 0,
                                 _lib.current_stream_ptr()))
    return out


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, **kwargs) -> torch.Tensor:
    """[M/ws, N] = reduce_scatter(a @ b) along M, in one kernel. Three exchange algorithms:
    "pull" — every rank TMA-stores its partial tiles into its own symmetric staging and bumps a
    per-tile counter at the tile's owner; reducer warps inside the same kernel sum each owned tile
    over all ranks (peer loads in rank order, or ``multimem.ld_reduce`` with KRAKEN_RS_NVLS=1) as
    soon as all ranks have stored it, while the MMAs of later tiles run; "scatter" — the same, but
    the epilogue TMA-stores each tile into the owner's staging over NVLink so the reducer warps sum
    local memory; "push" — the epilogue TMA-stores remote tiles into the owner's staging slab and
    the owner adds them to its accumulator in the epilogue of its own tiles (computed last). All
    are bit-reproducible from call to call.
    Shapes whose slab is not a multiple of 128 rows, or N < 256, run GEMM -> symmetric staging ->
    reduce-scatter kernel. kwargs: group, algo="pull"|"scatter"|"push" (default KRAKEN_RS_ALGO)."""
    group = kwargs.get("group")
    if a.device.type != "cuda":
        return ref.gemm_reduce_scatter(a, b, group)
    a2, lda = as_k_major_a(a)
    bt, ldb = as_k_major_bt(b)
    M, K = a2.shape
    N = bt.shape[0]
    if bt.shape[1] != K or K % 8:
        raise ValueError("inner dimensions must match and be a multiple of 8")
    info = symm_mem.resolve_group(group)
    ws = info.world_size
    if M % ws:
        raise ValueError("M must be divisible by the world size")
    out = torch.empty((M // ws, N), dtype=torch.bfloat16, device=a.device)
    algo = str(kwargs.get("algo", config.rs_algo()))
    if algo not in ("pull", "push", "scatter"):
        raise ValueError("algo must be 'pull', 'scatter' or 'push'")
    if symm_mem.capturing() and algo != "push":
        algo = "push"                   # pull and scatter alternate staging halves call by call: not replayable
    fused_ok = (M // ws) % 128 == 0 and N % 8 == 0 and N >= 256
    force = bool(kwargs.get("_force_fused", False))           # tests: run the fused kernel at world size 1
    if _log.dump_enabled():
        path = "plain GEMM" if ws == 1 and not force else (f"fused, {algo}" if fused_ok
                                                           else "GEMM + reduce-scatter kernel")
        _log.log_kernel_choice("gemm_reduce_scatter", f"M={M} N={N} K={K} ws={ws}: {path}")
    L = _lib.lib()
    s = _lib.current_stream_ptr()
    if ws == 1 and not (force and fused_ok):
        _lib.check(L.kr_gemm_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, out.data_ptr(), N, M, N, K, 0, -1, 0, 0, 1, 0, s))
    elif fused_ok:
        if algo in ("pull", "scatter"):
            hdl = symm_mem.get_symm_mem_workspace(group, 2 * M * N * 2 + 2048, a.device, kind="gemm_rs")
            calls = getattr(hdl, "_gemm_rs_calls", 0)        # per staging buffer: selects the half / counter bank
            hdl._gemm_rs_calls = calls + 1
        else:
            hdl = symm_mem.get_symm_mem_workspace(group, M * N * 2, a.device)
            calls = 0
        mc = hdl.multicast_ptr if (algo == "pull" and config.rs_nvls()) else 0
        pads_host = getattr(hdl, "_host_pad_array", None)
        if pads_host is None:
            pads_host = hdl._host_pad_array = (ctypes.c_void_p * ws)(*hdl.signal_pad_ptrs)
        _lib.check(L.kr_gemm_rs_bf16(hdl.buffer_ptrs_dev, hdl._host_ptr_array, hdl.signal_pad_ptrs_dev, pads_host,
                                     mc or None, hdl.rank, ws, a2.data_ptr(), lda, bt.data_ptr(), ldb,
                                     out.data_ptr(), N, M, N, K, {"push": 0, "pull": 1, "scatter": 2}[algo], calls & 1, 0,
                                     config.TILE_FLAG_BASE, hdl.signal_pad_words, hdl.buffer_size, s))
    else:
        if (M * N) % (8 * ws):
            raise ValueError("M * N must be a multiple of 8 * world size")
        hdl = symm_mem.get_symm_mem_workspace(group, M * N * 2, a.device)
        stage = hdl.buffer_ptrs[hdl.rank]
        _lib.check(L.kr_gemm_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, stage, N, M, N, K, 0, 0, 0, 0, 1, 0, s))
        _lib.check(L.kr_reduce_scatter(hdl.buffer_ptrs_dev, 0, hdl.signal_pad_ptrs_dev, hdl.rank, ws, None,
                                       out.data_ptr(), M * N, 0, 0, s))
    return out if a.dtype != torch.float32 else out.to(a.dtype)


_ce_state: dict[int, tuple] = {}


def gemm_reduce_scatter_ce_persistent(a: torch.Tensor, b: torch.Tensor, reduce_op: str = "sum", group=None,
                                      **kwargs) -> torch.Tensor:
    """Copy-engine variant of GEMM -> reduce-scatter (the reference's recipe): a persistent producer
    GEMM writes the local product slab by slab (next rank's slab first) and raises a signal word
    per finished slab; on a backend stream, stream waits on those words gate copy-engine transfers
    of each slab to its owner's workspace; after a cross-device barrier a local kernel sums the ws
    received slabs."""
    if reduce_op != "sum":
        raise ValueError("only reduce_op='sum' is supported")
    if a.device.type != "cuda":
        return ref.gemm_reduce_scatter(a, b, group)
    a2, lda = as_k_major_a(a)
    bt, ldb = as_k_major_bt(b)
    M, K = a2.shape
    N = bt.shape[0]
    info = symm_mem.resolve_group(group)
    ws, rank = info.world_size, info.rank
    if M % ws or (M // ws) % 128:
        raise ValueError("copy-engine GEMM reduce-scatter needs (M / world_size) % 128 == 0")
    L = _lib.lib()
    dev = a.device
    out = torch.empty((M // ws, N), dtype=torch.bfloat16, device=dev)
    if ws == 1:
        _lib.check(L.kr_gemm_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, out.data_ptr(), N, M, N, K, 0, -1, 0, 0, 1, 0,
                                  _lib.current_stream_ptr()))
        return out
    gemm_out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    _log.log_kernel_choice("gemm_reduce_scatter_ce_persistent", f"M={M} N={N} K={K} ws={ws}: producer GEMM + copy engines + slab reduction")
    hdl = symm_mem.get_symm_mem_workspace(group, M * N * 2, dev)
    backend = symm_mem._get_backend_stream(priority=-1)
    cur = torch.cuda.current_stream()
    signals = torch.zeros(ws, dtype=torch.uint32, device=dev)
    counters = torch.zeros(ws, dtype=torch.uint32, device=dev)
    backend.wait_stream(cur)
    _lib.check(L.kr_gemm_ce_producer_bf16(a2.data_ptr(), lda, bt.data_ptr(), ldb, gemm_out.data_ptr(), N, M, N, K,
                                          rank, ws, signals.data_ptr(), counters.data_ptr(), cur.cuda_stream))
    slab_bytes = (M // ws) * N * 2
    ptrs = (ctypes.c_void_p * ws)(*hdl.buffer_ptrs)
    with torch.cuda.stream(backend):
        _lib.check(L.kr_ce_scatter_slabs(ptrs, rank, ws, gemm_out.data_ptr(), signals.data_ptr(), slab_bytes,
                                         backend.cuda_stream))
    cur.wait_stream(backend)
    hdl.barrier()                       # every rank's slabs have landed everywhere
    _lib.check(L.kr_reduce_slabs(hdl.buffer_ptrs[rank], out.data_ptr(), ws, (rank + 1) % ws, (M // ws) * N,
                                 cur.cuda_stream))
    hdl.barrier()                       # workspace free for the next op
    for t in (gemm_out, signals, counters):
        t.record_stream(backend)
    return out
