"""All-reduce fused with a bias add, and with bias add + RMSNorm (the tensor-parallel decode
epilogue). Signatures follow the reference: kraken/fused/one_shot_all_reduce_bias.py:105-173,
kraken/fused/two_shot_all_reduce_bias.py:123-193,
kraken/fused/one_shot_all_reduce_bias_rms_norm.py:102-169,
kraken/fused/two_shot_all_reduce_bias_rms_norm.py:132-223.

``symm_mem_buffer`` / ``symm_mem_input`` is a symmetric scratch tensor at least as large as the
input; the input itself is an ordinary tensor. ``bias`` may have the input's shape (as in the
reference's tests) or be a single row [D] shared by all rows. ``max_num_blocks`` caps the grid;
``BLOCK_SIZE`` is accepted and ignored.
"""
from __future__ import annotations

import torch

from .. import _reference as ref
from .. import config
from ..comm.all_reduce import _bias_args, _check_bf16, _dump, _push_all_reduce, push_eligible, push_workspace
from ..ops import lib as _lib
from ..parallel import symm_mem


def _scratch(symm_buf: torch.Tensor, x: torch.Tensor, group):
    hdl = symm_mem.rendezvous(symm_buf, group)
    if symm_buf.numel() * symm_buf.element_size() < x.numel() * x.element_size():
        raise ValueError("symmetric buffer is smaller than the input")
    return hdl, hdl.offset_of(symm_buf)


def one_shot_all_reduce_bias(symm_mem_buffer: torch.Tensor, input_tensor: torch.Tensor, bias: torch.Tensor | None,
                             output: torch.Tensor, max_num_blocks: int = 0, BLOCK_SIZE: int = 4096,
                             group=None, algo: str | None = None) -> None:
    """output = all_reduce(input) (+ bias). Small messages: every rank writes its data into the
    peers' workspace, one barrier, local sum (`symm_mem_buffer` is then not touched). Larger ones:
    copy into `symm_mem_buffer`, barrier, every rank pulls all peers' copies and sums."""
    if input_tensor.device.type != "cuda":
        output.copy_(ref.all_reduce_bias(input_tensor, bias, group))
        return None
    _check_bf16(input_tensor)
    _check_bf16(output)
    hdl, off = _scratch(symm_mem_buffer, input_tensor, group)
    if push_eligible(input_tensor.numel() * 2, input_tensor.numel(), hdl.world_size, {"algo": algo}):
        _push_all_reduce(input_tensor, bias, output, group)
        return None
    bias_ptr, bias_n = _bias_args(bias, input_tensor)
    _dump(f"one_shot_all_reduce_bias pull numel={input_tensor.numel()} ws={hdl.world_size}")
    _lib.check(_lib.lib().kr_one_shot_all_reduce(
        hdl.buffer_ptrs_dev, off, hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, input_tensor.data_ptr(),
        output.data_ptr(), bias_ptr, bias_n, input_tensor.numel(), int(max_num_blocks or 0), 0,
        _lib.current_stream_ptr()))
    return None


def two_shot_all_reduce_bias(symm_mem_input: torch.Tensor, input_tensor: torch.Tensor, bias: torch.Tensor | None,
                             output: torch.Tensor, max_num_blocks: int = 0, BLOCK_SIZE: int = 2048,
                             group=None) -> torch.Tensor:
    """output = all_reduce(input) (+ bias): each rank reduces 1/ws of the elements, adds the bias
    and publishes the result to every rank (through NVLS when the buffer has a multicast mapping)."""
    if input_tensor.device.type != "cuda":
        output.copy_(ref.all_reduce_bias(input_tensor, bias, group))
        return output
    _check_bf16(input_tensor)
    _check_bf16(output)
    if input_tensor.numel() % 8:
        raise ValueError("numel must be a multiple of 8")
    hdl, off = _scratch(symm_mem_input, input_tensor, group)
    bias_ptr, bias_n = _bias_args(bias, input_tensor)
    mc = hdl.multicast_ptr if (hdl.multicast_ptr and config.force_algo() != "two_shot") else None
    _dump(f"two_shot_all_reduce_bias numel={input_tensor.numel()} ws={hdl.world_size} nvls={bool(mc)}")
    _lib.check(_lib.lib().kr_two_shot_all_reduce(
        hdl.buffer_ptrs_dev, off, hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, input_tensor.data_ptr(),
        output.data_ptr(), bias_ptr, bias_n, input_tensor.numel(), mc, int(max_num_blocks or 0), 0,
        _lib.current_stream_ptr()))
    return output


def _ar_bias_rms_norm(symm_buf, x, bias, w, y, eps, group, algo: int, one_shot: str | None = None) -> None:
    if x.device.type != "cuda":
        y.copy_(ref.all_reduce_bias_rms_norm(x, bias, w, eps, group))
        return
    for t in (x, y, w):
        _check_bf16(t)
    D = x.shape[-1]
    rows = x.numel() // D
    if w.numel() != D:
        raise ValueError("RMSNorm weight must have the last dimension's size")
    hdl, off = _scratch(symm_buf, x, group)
    bias_ptr, bias_n = _bias_args(bias, x)
    if algo == 0 and push_eligible(x.numel() * 2, x.numel(), hdl.world_size, {"algo": one_shot}):
        ph, pads, seq = push_workspace(group, x.device)
        _dump(f"one_shot_all_reduce_bias_rms_norm push rows={rows} D={D} ws={ph.world_size} nvls={bool(ph.multicast_ptr)}")
        _lib.check(_lib.lib().kr_push_all_reduce_bias_rms_norm(
            ph._host_ptr_array, pads, ph.multicast_ptr or None, ph.rank, ph.world_size, x.data_ptr(), bias_ptr, bias_n,
            w.data_ptr(), y.data_ptr(), rows, D, float(eps), seq, config.push_tagged_max_bytes(ph.world_size), ph.buffer_size, 0,
            _lib.current_stream_ptr()))
        return
    mc = None
    if algo == 1 and hdl.multicast_ptr and config.force_algo() != "two_shot":
        algo, mc = 2, hdl.multicast_ptr
    _dump(f"all_reduce_bias_rms_norm {('one_shot pull', 'two_shot', 'two_shot nvls')[algo]} rows={rows} D={D} ws={hdl.world_size}")
    _lib.check(_lib.lib().kr_all_reduce_bias_rms_norm(
        hdl.buffer_ptrs_dev, off, hdl.signal_pad_ptrs_dev, hdl.rank, hdl.world_size, x.data_ptr(), bias_ptr, bias_n,
        w.data_ptr(), y.data_ptr(), rows, D, float(eps), algo, mc, 0, _lib.current_stream_ptr()))


def one_shot_all_reduce_bias_rms_norm(symm_mem_input: torch.Tensor, x: torch.Tensor, bias: torch.Tensor | None,
                                      w: torch.Tensor, y: torch.Tensor, eps: float = 1e-5, BLOCK_SIZE: int = 1024,
                                      group=None, algo: str | None = None) -> None:
    """y = rms_norm(all_reduce(x) + bias) * w; the summed row never leaves registers. Small inputs
    take the push form (one barrier), larger ones the pull form; algo="push"|"pull" overrides."""
    _ar_bias_rms_norm(symm_mem_input, x, bias, w, y, eps, group, 0, algo)


def two_shot_all_reduce_bias_rms_norm(symm_mem_input: torch.Tensor, x: torch.Tensor, bias: torch.Tensor | None,
                                      w: torch.Tensor, y: torch.Tensor, eps: float = 1e-5, group=None) -> None:
    """Same result with the two-shot exchange: rank k reduces columns [k*D/ws, (k+1)*D/ws) of each
    row and publishes them, then every rank normalises. Needs D % (8 * world_size) == 0."""
    D = x.shape[-1]
    info = symm_mem.resolve_group(group)
    algo = 1 if D % (8 * info.world_size) == 0 else 0
    _ar_bias_rms_norm(symm_mem_input, x, bias, w, y, eps, group, algo)
