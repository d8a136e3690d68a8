"""All-gather with per-chunk progress flags.

Reference: kraken/comm/copy_engine_all_gather.py:6-126. Two engines produce the same result and
the same flag layout (chunk index = src_rank * splits + split; flag becomes non-zero when the
chunk has fully landed in ``a_out``):
  * ``ce``: copy-engine DMA (``cudaMemcpyAsync`` peer -> local) on a backend stream, each chunk
    followed by a stream memory operation that sets its flag — the reference's recipe;
  * ``sm``: one kernel whose blocks pull the chunks with 16-byte loads and publish the flags with
    ``st.release.gpu`` — no second stream, usable inside CUDA graphs without stream mem-ops.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _reference as ref
from .._logging import utils as _log
from ..ops import lib as _lib
from ..parallel import symm_mem


def _copy_engine_all_gather_w_progress(output: torch.Tensor, inp: torch.Tensor, progress: torch.Tensor,
                                       splits_per_rank: int, backend_stream: torch.cuda.Stream | None = None):
    """Copy-engine all-gather of the symmetric shard `inp` into `output` on a backend stream.
    Returns the backend stream; the caller decides when the current stream waits for it."""
    assert inp.is_contiguous() and output.is_contiguous()
    hdl = symm_mem.rendezvous(inp)
    ws, rank = hdl.world_size, hdl.rank
    if output.numel() != inp.numel() * ws:
        raise ValueError("output must hold world_size shards")
    if inp.shape[0] % splits_per_rank:
        raise ValueError("shard rows must divide into splits_per_rank")
    if backend_stream is None:
        backend_stream = symm_mem._get_backend_stream(priority=-1)
    off = hdl.offset_of(inp)
    ptrs = (ctypes.c_void_p * ws)(*[p + off for p in hdl.buffer_ptrs])
    hdl.barrier()                                   # every rank's shard is complete
    backend_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(backend_stream):
        _lib.check(_lib.lib().kr_ce_all_gather(ptrs, rank, ws, output.data_ptr(), progress.data_ptr(),
                                               splits_per_rank, inp.numel() * inp.element_size(),
                                               backend_stream.cuda_stream))
        hdl.barrier()                               # peers are done reading this rank's shard
    return backend_stream


_sm_counters: dict[int, torch.Tensor] = {}


def _counters(device: torch.device, n: int) -> torch.Tensor:
    t = _sm_counters.get(device.index)
    if t is None or t.numel() < n:
        t = torch.zeros(max(n, 2048), dtype=torch.int32, device=device)
        _sm_counters[device.index] = t
    return t


def _sm_all_gather_w_progress(output: torch.Tensor, inp: torch.Tensor, progress: torch.Tensor, splits_per_rank: int,
                              max_num_blocks: int = 0, counters: torch.Tensor | None = None) -> None:
    hdl = symm_mem.rendezvous(inp)
    if (inp.numel() * inp.element_size()) % (16 * splits_per_rank):
        raise ValueError("shard bytes must be a multiple of 16 * splits_per_rank")
    if counters is None:
        if hdl.group.emu is not None:
            counters = torch.zeros(hdl.world_size * splits_per_rank, dtype=torch.int32, device=inp.device)
            hdl.group.emu._keep.append(counters)
        else:
            counters = _counters(inp.device, hdl.world_size * splits_per_rank)
    # the kernel counts in 2-byte elements
    numel16 = inp.numel() * inp.element_size() // 2
    _lib.check(_lib.lib().kr_all_gather_sm(
        hdl.buffer_ptrs_dev, hdl.offset_of(inp), hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, output.data_ptr(),
        progress.data_ptr(), counters.data_ptr(), splits_per_rank, numel16, max_num_blocks, 0,
        _lib.current_stream_ptr()))


def all_gather_w_progress(a_shared: torch.Tensor, a_out: torch.Tensor | None = None,
                          progress: torch.Tensor | None = None, **kwargs) -> torch.Tensor:
    """Gathers every rank's symmetric shard `a_shared` along dim 0 into `a_out`; `progress`
    (uint32 [world_size * splits_per_rank]) is zeroed on entry and every slot is non-zero on return.
    kwargs: splits_per_rank=1, backend="ce"|"sm" (default from KRAKEN_AG_MODE, "ce" matching the
    reference when unset here), max_num_blocks."""
    splits = int(kwargs.get("splits_per_rank", 1))
    if a_shared.device.type != "cuda":
        out = ref.all_gather(a_shared, kwargs.get("group"))
        if a_out is not None:
            a_out.copy_(out)
            out = a_out
        if progress is not None:
            progress.fill_(1)
        return out
    hdl = symm_mem.rendezvous(a_shared, kwargs.get("group"))
    shape = list(a_shared.shape)
    shape[0] *= hdl.world_size
    if a_out is None:
        a_out = torch.empty(shape, dtype=a_shared.dtype, device=a_shared.device)
    if progress is None:
        progress = torch.zeros(hdl.world_size * splits, dtype=torch.uint32, device=a_shared.device)
    else:
        progress.zero_()
    backend = kwargs.get("backend", "ce" if hdl.group.emu is None else "sm")
    _log.log_kernel_choice("all_gather_w_progress", f"numel={a_shared.numel()} ws={hdl.world_size} splits={splits} engine={backend}")
    if backend == "sm":
        _sm_all_gather_w_progress(a_out, a_shared, progress, splits, int(kwargs.get("max_num_blocks", 0) or 0))
    else:
        stream = _copy_engine_all_gather_w_progress(a_out, a_shared, progress, splits, kwargs.get("backend_stream"))
        torch.cuda.current_stream().wait_stream(stream)
    return a_out
