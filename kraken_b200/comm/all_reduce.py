"""All-reduce and reduce-scatter over symmetric memory.

Public functions keep the reference's signatures (kraken/comm/one_shot_all_reduce.py:57-113,
kraken/comm/two_shot_all_reduce.py:100-157); ``multimem_all_reduce`` and ``reduce_scatter`` are
named by the reference's README but have no reference code — their semantics follow
``torch.ops.symm_mem.multimem_all_reduce_`` and ``reduce_scatter_tensor``. Triton tuning kwargs
(``num_warps``, ``BLOCK_SIZE``) are accepted and ignored; ``max_num_blocks`` caps the grid.
CPU tensors run the pure-PyTorch backend over the process group.
"""
from __future__ import annotations

import torch

from .. import _reference as ref
from .. import config
from .._logging import utils as _log
from ..ops import lib as _lib
from ..parallel import symm_mem


def _dump(msg: str, hdl=None) -> None:
    op, _, detail = msg.partition(" ")
    _log.log_kernel_choice(op, detail)


# ---- push-style one-shot (small messages) ---------------------------------------------------------
_PUSH_WORKSPACE_BYTES = 64 << 20     # four quarters (flag form even / odd calls, tagged form even / odd) of world_size slots


def push_limit_bytes(ws: int) -> int:
    """Largest message the push-style one-shot kernels take: (ws - 1) x S leaves each rank, so the
    limit shrinks with the world size: 2 MiB at 2 ranks (measured: pushing 4 MB takes 30.8 us against
    26.7 us for the pull form, 2 MB and less are equal or faster), 1 MiB above; beyond it the one-shot
    ops pull."""
    fits = (_PUSH_WORKSPACE_BYTES // 4 // max(1, ws)) // 1024 * 1024
    return min(fits, (2 << 20) if ws <= 2 else (1 << 20))


def push_eligible(nbytes: int, numel: int, ws: int, kwargs=None) -> bool:
    mode = (kwargs or {}).get("algo") or config.one_shot_mode()
    if symm_mem.capturing():
        return False          # the push form alternates workspace halves call by call: not replayable
    return mode == "push" and 1 <= ws <= 8 and numel % 8 == 0 and 16 <= nbytes <= push_limit_bytes(ws)


def push_workspace(group, device):
    """(handle, host array of signal-pad addresses, number of calls made on it so far) of the push
    workspace. The call number picks the workspace half and is the tag of the tagged form."""
    import ctypes

    hdl = symm_mem.get_symm_mem_workspace(group, _PUSH_WORKSPACE_BYTES, device, kind="push")
    pads = getattr(hdl, "_host_pad_array", None)
    if pads is None:
        pads = hdl._host_pad_array = (ctypes.c_void_p * hdl.world_size)(*hdl.signal_pad_ptrs)
    calls = getattr(hdl, "_push_calls", 0)
    hdl._push_calls = calls + 1
    return hdl, pads, calls & 0xFFFFFFFF


def _push_all_reduce(inp: torch.Tensor, bias, out: torch.Tensor, group) -> None:
    hdl, pads, seq = push_workspace(group, inp.device)
    bias_ptr, bias_n = _bias_args(bias, inp)
    tagged = config.push_tagged_max_bytes(hdl.world_size)
    _dump(f"one_shot_all_reduce push numel={inp.numel()} ws={hdl.world_size} nvls={bool(hdl.multicast_ptr)} "
          f"tagged={inp.numel() * 2 <= tagged}")
    _lib.check(_lib.lib().kr_push_all_reduce(
        hdl._host_ptr_array, pads, hdl.multicast_ptr or None, hdl.rank, hdl.world_size, inp.data_ptr(), out.data_ptr(),
        bias_ptr, bias_n, inp.numel(), seq, tagged, hdl.buffer_size, 0, _lib.current_stream_ptr()))


def _check_bf16(t: torch.Tensor) -> None:
    if t.dtype != torch.bfloat16:
        raise TypeError("only bfloat16 is supported")
    if not t.is_contiguous():
        raise ValueError("tensor must be contiguous")
    if t.data_ptr() % 16:
        raise ValueError("tensor must be 16-byte aligned")


def _bias_args(bias: torch.Tensor | None, like: torch.Tensor):
    """bias may have the input's full shape (the reference's tests) or be one row [D]."""
    if bias is None:
        return None, 0
    _check_bf16(bias)
    if bias.numel() != like.numel() and (like.dim() == 0 or bias.numel() != like.shape[-1]):
        raise ValueError("bias must have the input's shape or its last dimension")
    return bias.data_ptr(), bias.numel()


def _max_blocks(kwargs) -> int:
    # The reference caps its grid at 24 blocks by default, a Triton-era tuning; here 0 = up to one
    # block per SM and an explicit max_num_blocks still caps it.
    return int(kwargs.get("max_num_blocks", 0) or 0)


def one_shot_all_reduce(tensor: torch.Tensor, **kwargs) -> torch.Tensor:
    """output = sum over ranks of `tensor`. `tensor` must live in symmetric memory
    (``symm_mem.empty``). Small messages are pushed: every rank writes its data into a slot of each
    peer's workspace, one barrier, local sum. Larger ones are pulled: every rank reads all peers'
    copies directly. fp32 accumulation in rank order. kwargs: group, max_num_blocks,
    algo="push"|"pull" (default KRAKEN_ONE_SHOT)."""
    if tensor.device.type != "cuda":
        return ref.all_reduce(tensor, kwargs.get("group"))
    _check_bf16(tensor)
    hdl = symm_mem.rendezvous(tensor, kwargs.get("group"))
    out = torch.empty_like(tensor)
    if push_eligible(tensor.numel() * 2, tensor.numel(), hdl.world_size, kwargs):
        _push_all_reduce(tensor, None, out, kwargs.get("group"))
        return out
    _dump(f"one_shot_all_reduce pull numel={tensor.numel()} ws={hdl.world_size}", hdl)
    _lib.check(_lib.lib().kr_one_shot_all_reduce(
        hdl.buffer_ptrs_dev, hdl.offset_of(tensor), hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, None,
        out.data_ptr(), None, 0, tensor.numel(), _max_blocks(kwargs), 0, _lib.current_stream_ptr()))
    return out


def _two_shot(tensor: torch.Tensor, bias, out: torch.Tensor | None, kwargs, use_mc: bool) -> torch.Tensor:
    group = kwargs.get("group")
    hdl = symm_mem.get_symm_mem_workspace(group, tensor.numel() * tensor.element_size(), tensor.device)
    if out is None:
        out = torch.empty_like(tensor)
    bias_ptr, bias_n = _bias_args(bias, tensor)
    # in-switch reduction pays from 4 ranks on: at 2 ranks the peer-load form was measured faster
    # (731 us against 1007 us at 256 MB), at 8 it is 1.8x slower than the NVLS form
    mc = hdl.multicast_ptr if (use_mc and hdl.multicast_ptr and hdl.world_size > 2) else None
    _dump(f"two_shot_all_reduce numel={tensor.numel()} ws={hdl.world_size} nvls={bool(mc)}", hdl)
    _lib.check(_lib.lib().kr_two_shot_all_reduce(
        hdl.buffer_ptrs_dev, 0, hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, tensor.data_ptr(), out.data_ptr(),
        bias_ptr, bias_n, tensor.numel(), mc, _max_blocks(kwargs), 0, _lib.current_stream_ptr()))
    return out


def two_shot_all_reduce(tensor: torch.Tensor, **kwargs) -> torch.Tensor:
    """output = sum over ranks of `tensor` (an ordinary tensor: it is staged through the group's
    symmetric workspace). Each rank reduces 1/ws of the data and publishes it to all ranks — with
    ``multimem.ld_reduce`` / ``multimem.st`` through the NVSwitch when the workspace has a multicast
    mapping and there are more than 2 ranks (measured 1.8x the peer-load form at 256 MB on 8 GPUs,
    but slower than it on 2), else with peer loads and stores.
    kwargs: group, max_num_blocks, nvls=False forces the peer-load form (as does
    KRAKEN_FORCE_ALGO=two_shot)."""
    if tensor.device.type != "cuda":
        return ref.all_reduce(tensor, kwargs.get("group"))
    _check_bf16(tensor)
    if tensor.numel() % 8:
        raise ValueError("numel must be a multiple of 8")
    use_mc = bool(kwargs.get("nvls", True)) and config.force_algo() != "two_shot"
    return _two_shot(tensor, None, None, kwargs, use_mc)


def multimem_all_reduce(tensor: torch.Tensor, **kwargs) -> torch.Tensor:
    """In-place all-reduce of a symmetric tensor through NVLS: each rank reduces its 1/ws with
    ``multimem.ld_reduce`` (the NVSwitch adds) and broadcasts it with ``multimem.st``. Returns
    `tensor`. Falls back to the P2P two-shot form (still in place) when the buffer has no
    multicast mapping (NVLS disabled or unsupported)."""
    if tensor.device.type != "cuda":
        tensor.copy_(ref.all_reduce(tensor, kwargs.get("group")))
        return tensor
    _check_bf16(tensor)
    if tensor.numel() % 8:
        raise ValueError("numel must be a multiple of 8")
    hdl = symm_mem.rendezvous(tensor, kwargs.get("group"))
    mc = hdl.multicast_ptr or None
    _dump(f"multimem_all_reduce numel={tensor.numel()} ws={hdl.world_size} nvls={bool(mc)}", hdl)
    _lib.check(_lib.lib().kr_two_shot_all_reduce(
        hdl.buffer_ptrs_dev, hdl.offset_of(tensor), hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, None,
        tensor.data_ptr(), None, 0, tensor.numel(), mc, _max_blocks(kwargs), 0, _lib.current_stream_ptr()))
    return tensor


def reduce_scatter(tensor: torch.Tensor, **kwargs) -> torch.Tensor:
    """`tensor` is [ws * n, ...] on every rank; rank r returns sum over ranks of rows
    [r*n, (r+1)*n). A symmetric `tensor` is read in place; an ordinary one is staged through the
    group workspace. fp32 accumulation in rank order (bitwise identical run to run)."""
    group = kwargs.get("group")
    if tensor.device.type != "cuda":
        return ref.reduce_scatter(tensor, group)
    _check_bf16(tensor)
    info = symm_mem.resolve_group(group)
    ws = info.world_size
    if tensor.shape[0] % ws or tensor.numel() % (8 * ws):
        raise ValueError("dim 0 must divide by the world size and numel by 8 * world size")
    out = torch.empty((tensor.shape[0] // ws, *tensor.shape[1:]), dtype=tensor.dtype, device=tensor.device)
    if symm_mem.is_symm_tensor(tensor):
        hdl = symm_mem.rendezvous(tensor, group)
        off, inp = hdl.offset_of(tensor), None
    else:
        hdl = symm_mem.get_symm_mem_workspace(group, tensor.numel() * 2, tensor.device)
        off, inp = 0, tensor.data_ptr()
    _dump(f"reduce_scatter numel={tensor.numel()} ws={ws} staged={inp is not None}")
    _lib.check(_lib.lib().kr_reduce_scatter(
        hdl.buffer_ptrs_dev, off, hdl.signal_pad_ptrs_dev, hdl.rank, ws, inp, out.data_ptr(), tensor.numel(),
        _max_blocks(kwargs), 0, _lib.current_stream_ptr()))
    return out


def all_reduce(tensor: torch.Tensor, **kwargs) -> torch.Tensor:
    """Size-based choice among the algorithms (not in the reference). Measured crossovers on B200:
    the one-shot pull wins while (ws-1) x S of pull traffic is cheaper than two barriers more —
    up to about 16 MB at 2 GPUs and 1-2 MB at 8 — hence a threshold of 64 MiB / ws^2; above it the
    two-shot form runs, through NVLS when the workspace has a multicast mapping. One-shot needs the
    input itself in symmetric memory; ordinary tensors always take the staged two-shot form."""
    if tensor.device.type != "cuda":
        return ref.all_reduce(tensor, kwargs.get("group"))
    algo = config.force_algo()
    nbytes = tensor.numel() * tensor.element_size()
    info = symm_mem.resolve_group(kwargs.get("group"))
    if algo is None:
        algo = "one_shot" if nbytes <= (64 << 20) // max(1, info.world_size ** 2) else "two_shot"
    if algo == "one_shot" and symm_mem.is_symm_tensor(tensor):
        return one_shot_all_reduce(tensor, **kwargs)
    return _two_shot(tensor, None, None, kwargs, True)
