"""Synchronisation primitives.

In the reference these are ``@triton.jit`` device functions (kraken/_ptx_utils/__init__.py:1-19:
``symm_mem_sync``, ``send_signal``, ``get_flat_tid``, ``arrive_gmem_barrier``, ``wait_gmem_barrier``)
that user kernels inline. Here the device functions live in the CUDA header
``csrc/include/kraken/ptx_sync.cuh`` (same names; every wait bounded by a deadline) for user CUDA
kernels to include, and this module offers host-callable launches of them — what a Python user can
do with a device primitive: run it as a barrier, or run the library's self-test kernels.
"""
from __future__ import annotations

import os

import torch

from ..ops import lib as _lib
from ..parallel import symm_mem

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                      "csrc", "include", "kraken", "ptx_sync.cuh")


def symm_mem_sync(signal_pad_ptrs, block_id=None, rank: int = 0, world_size: int = 1,
                  hasPreviousMemAccess: bool | None = None, hasSubsequentMemAccess: bool | None = None,
                  num_blocks: int = 1) -> torch.Tensor:
    """Launches `num_blocks` blocks on the current stream that each meet the blocks of the same id
    on all ranks in the per-block cross-device barrier. With both pattern arguments left at None
    every block runs the three patterns the library's kernels use, (F,T), (T,T), (T,F), back to
    back (a self-test); with either given, every block runs ONE barrier of exactly that pattern
    (hasPreviousMemAccess: release before signalling; hasSubsequentMemAccess: acquire after
    waiting) — which, launched between two kernels of a stream, orders their symmetric-memory
    accesses across ranks the way the device function does inside a kernel. `signal_pad_ptrs` is a
    handle (or its ``signal_pad_ptrs_dev``); `block_id` is implied by the launch (block i uses slot
    i) and accepted for signature parity. Returns a tensor with 1 per block whose waits completed."""
    dev_ptr = getattr(signal_pad_ptrs, "signal_pad_ptrs_dev", signal_pad_ptrs)
    out = torch.zeros(num_blocks, dtype=torch.int32, device="cuda")
    if hasPreviousMemAccess is None and hasSubsequentMemAccess is None:
        mode = 0
    else:
        mode = 4 | (2 if hasPreviousMemAccess else 0) | (1 if hasSubsequentMemAccess else 0)
    _lib.check(_lib.lib().kr_sync_test(dev_ptr, rank, world_size, None, out.data_ptr(), mode, num_blocks, 1,
                                       _lib.current_stream_ptr()))
    return out


def send_signal(handle, dst_rank: int, slot: int, value: int = 1) -> None:
    """Stream-ordered write of `value` into word `slot` of `dst_rank`'s signal pad (the host-side
    counterpart of the device function; uses a stream memory operation)."""
    addr = handle.signal_pad_ptrs[dst_rank] + 4 * slot
    _lib.check(_lib.lib().kr_stream_write_value32(_lib.current_stream_ptr(), addr, value))


def get_flat_tid() -> str:
    """A device function in the reference (the flattened thread index inside a block). Python has no
    device code, so this returns the C expression for it, for user CUDA sources that are assembled
    as text; kernels that include ``ptx_sync.cuh`` use the same expression inside ``symm_mem_sync``."""
    return "threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z)"


def gmem_barrier_test(num_producers: int, num_blocks: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Runs the arrive/wait self-test: blocks [0, num_producers) publish a value and arrive on their
    flag; the other blocks wait on flag (block % num_producers) and read the value.
    Returns (flags, values-seen-per-block)."""
    flags = torch.zeros(num_producers, dtype=torch.int32, device="cuda")
    out = torch.zeros(num_blocks, dtype=torch.int32, device="cuda")
    pads = torch.zeros(1, dtype=torch.int64, device="cuda")
    _lib.check(_lib.lib().kr_sync_test(pads.data_ptr(), 0, 1, flags.data_ptr(), out.data_ptr(), 1, num_blocks,
                                       num_producers, _lib.current_stream_ptr()))
    return flags, out


def arrive_gmem_barrier(flag: torch.Tensor, index: int = 0, update: int = 1) -> None:
    """Stream-ordered flag write (host counterpart of the device function)."""
    _lib.check(_lib.lib().kr_stream_write_value32(_lib.current_stream_ptr(), flag.data_ptr() + 4 * index, update))


def wait_gmem_barrier(flag: torch.Tensor, index: int = 0, expect: int = 1) -> None:
    """Stream-ordered wait until flag[index] == expect (host counterpart of the device function)."""
    _lib.check(_lib.lib().kr_stream_wait_value32(_lib.current_stream_ptr(), flag.data_ptr() + 4 * index, expect))


def wait_timeout_test(num_blocks: int = 4) -> torch.Tensor:
    """Blocks wait on flags nothing sets; with a short deadline they give up, record a status word
    and return. Returns per-block results (2 = gave up)."""
    flags = torch.zeros(num_blocks, dtype=torch.int32, device="cuda")
    out = torch.zeros(num_blocks, dtype=torch.int32, device="cuda")
    pads = torch.zeros(1, dtype=torch.int64, device="cuda")
    _lib.check(_lib.lib().kr_sync_test(pads.data_ptr(), 0, 1, flags.data_ptr(), out.data_ptr(), 2, num_blocks, 1,
                                       _lib.current_stream_ptr()))
    return out


def bounds_check_selftest() -> tuple[int, bool]:
    """Runs a kernel whose one store is guarded by a bounds check that must fail. Returns
    (value stored, whether a bounds error was recorded). With the debug build (KRAKEN_DEBUG=1) the
    store is skipped and the status word carries the bounds code; the regular build compiles the
    check away. The status word is cleared again."""
    import ctypes

    L = _lib.lib()
    out = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    pads = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = _lib.current_stream_ptr()
    _lib.check(L.kr_sync_test(pads.data_ptr(), 0, 1, flags.data_ptr(), out.data_ptr(), 3, 1, 4, stream))
    word = ctypes.c_uint32(0)
    _lib.check(L.kr_read_status(stream, ctypes.byref(word)))
    _lib.check(L.kr_clear_status(stream))
    torch.cuda.synchronize()
    return int(out[4].item()), (word.value & 0xFF) == 4


__all__ = ["symm_mem_sync", "bounds_check_selftest", "send_signal", "get_flat_tid", "arrive_gmem_barrier", "wait_gmem_barrier",
           "gmem_barrier_test", "wait_timeout_test", "HEADER"]
