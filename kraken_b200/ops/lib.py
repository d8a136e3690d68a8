"""ctypes binding of ``libkraken_b200.so`` — the one place where C prototypes are declared.

``lib()`` returns the loaded library (building it first when the sources are newer and nvcc is
available). ``check(rc)`` turns a non-zero return code into ``KrakenError`` carrying the native
error string. There is no Python fallback for CUDA tensors: if the library cannot be loaded the
import error propagates.
"""
from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_char_p, c_double, c_float, c_int, c_longlong, c_uint32, c_ulonglong, c_void_p, POINTER

from . import _build


class KrakenError(RuntimeError):
    pass


class KrakenSyncTimeout(KrakenError):
    """A bounded device-side wait ran out (a peer never arrived, or a pipeline stalled)."""


_lock = threading.Lock()
_lib = None

_P = c_void_p
_PROTOS = {
    "kr_last_error": (c_char_p, []),
    "kr_num_sms": (c_int, []),
    "kr_is_debug_build": (c_int, []),
    "kr_set_timeout_ms": (c_int, [c_double]),
    "kr_get_timeout_ms": (c_double, []),
    "kr_status_ptr": (_P, []),
    "kr_read_status": (c_int, [_P, POINTER(c_uint32)]),
    "kr_clear_status": (c_int, [_P]),
    "kr_emu_begin": (c_int, [c_int]),
    "kr_emu_abort": (c_int, []),
    "kr_emu_end": (c_int, [_P]),
    # symmetric memory
    "kr_symm_multicast_supported": (c_int, []),
    "kr_symm_alloc": (c_int, [c_ulonglong, c_ulonglong, POINTER(_P)]),
    "kr_symm_local_ptr": (_P, [_P]),
    "kr_symm_set_group": (c_int, [_P, c_int, c_int]),
    "kr_symm_total_bytes": (c_ulonglong, [_P]),
    "kr_symm_data_bytes": (c_ulonglong, [_P]),
    "kr_symm_pad_bytes": (c_ulonglong, [_P]),
    "kr_symm_export_fd": (c_int, [_P, POINTER(c_int)]),
    "kr_symm_import_fd": (c_int, [_P, c_int, c_int]),
    "kr_symm_finalize": (c_int, [_P]),
    "kr_symm_ptr": (_P, [_P, c_int]),
    "kr_symm_pad_ptr": (_P, [_P, c_int]),
    "kr_symm_bufs_dev": (_P, [_P]),
    "kr_symm_pads_dev": (_P, [_P]),
    "kr_symm_mc_ptr": (_P, [_P]),
    "kr_symm_mc_create": (c_int, [_P, POINTER(c_int)]),
    "kr_symm_mc_import": (c_int, [_P, c_int]),
    "kr_symm_mc_add_device": (c_int, [_P]),
    "kr_symm_mc_bind": (c_int, [_P]),
    "kr_symm_free": (c_int, [_P]),
    "kr_ipc_open": (c_int, [c_char_p, POINTER(c_int)]),
    "kr_ipc_close": (c_int, [c_int]),
    "kr_ipc_send_fd": (c_int, [c_int, c_char_p, c_int, c_int]),
    "kr_ipc_recv_fd": (c_int, [c_int, c_int, POINTER(c_int), POINTER(c_int)]),
    "kr_stream_write_value32": (c_int, [_P, _P, c_uint32]),
    "kr_stream_wait_value32": (c_int, [_P, _P, c_uint32]),
    "kr_ce_all_gather": (c_int, [POINTER(_P), c_int, c_int, _P, _P, c_int, c_ulonglong, _P]),
    "kr_ce_scatter_slabs": (c_int, [POINTER(_P), c_int, c_int, _P, _P, c_ulonglong, _P]),
    # comm kernels
    "kr_one_shot_all_reduce": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, _P, c_ulonglong, c_ulonglong, c_int, c_uint32, _P]),
    "kr_two_shot_all_reduce": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, _P, c_ulonglong, c_ulonglong, _P, c_int, c_uint32, _P]),
    "kr_reduce_scatter": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, c_ulonglong, c_int, c_uint32, _P]),
    "kr_all_gather_sm": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, _P, c_int, c_ulonglong, c_int, c_uint32, _P]),
    "kr_all_gather_sm_noalloc": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, c_int, c_ulonglong, c_int, c_uint32,
                                         _P, _P]),
    "kr_noalloc_read_status": (c_int, [_P, POINTER(c_uint32), c_int]),
    "kr_noalloc_set_timeout_ms": (c_int, [c_double]),
    "kr_symm_barrier": (c_int, [_P, c_int, c_int, c_int, _P]),
    "kr_sync_test": (c_int, [_P, c_int, c_int, _P, _P, c_int, c_int, c_int, _P]),
    # host model of the barrier protocol
    "kr_host_barrier": (c_uint32, [_P, c_ulonglong, c_int, c_int, c_int, c_double, c_int, c_int]),
    "kr_host_pad_nonzero": (c_ulonglong, [_P, c_ulonglong, c_int]),
    # push-style one-shot kernels (host pointer arrays)
    "kr_push_all_reduce": (c_int, [_P, _P, _P, c_int, c_int, _P, _P, _P, c_ulonglong, c_ulonglong, c_uint32, c_ulonglong,
                                   c_ulonglong, c_uint32, _P]),
    "kr_push_all_reduce_bias_rms_norm": (c_int, [_P, _P, _P, c_int, c_int, _P, _P, c_ulonglong, _P, _P, c_int, c_int,
                                                 c_float, c_uint32, c_ulonglong, c_ulonglong, c_uint32, _P]),
    # norm kernels
    "kr_rms_norm": (c_int, [_P, _P, _P, c_int, c_int, c_float, _P]),
    "kr_all_reduce_bias_rms_norm": (c_int, [_P, c_ulonglong, _P, c_int, c_int, _P, _P, c_ulonglong, _P, _P, c_int, c_int, c_float,
                                            c_int, _P, c_uint32, _P]),
    # gemm kernels
    "kr_tmap_cache_stats": (c_int, [POINTER(c_ulonglong), POINTER(c_ulonglong)]),
    "kr_gemm_bf16": (c_int, [_P, c_longlong, _P, c_longlong, _P, c_longlong, c_int, c_int, c_int, c_int, c_int, c_int,
                             c_int, c_int, c_int, _P]),
    "kr_ag_gemm_bf16": (c_int, [_P, _P, _P, c_int, c_int, _P, _P, c_longlong, _P, c_longlong, c_int, c_int, c_int,
                                c_int, _P, _P, c_int, c_uint32, c_int, c_ulonglong, c_uint32, c_ulonglong, c_int, _P, _P, _P]),
    "kr_gemm_rs_bf16": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, _P, c_longlong, _P, c_longlong, _P, c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_uint32, c_uint32, c_ulonglong, c_ulonglong, _P]),
    "kr_gemm_rs_set_trace": (c_int, [_P, c_ulonglong]),
    "kr_rs_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "kr_gemm_ar_bf16": (c_int, [_P, _P, _P, _P, c_int, c_int, _P, c_longlong, _P, c_longlong, _P, c_longlong, c_int, c_int,
                                c_int, c_int, c_int, c_int, c_uint32, c_uint32, c_ulonglong, c_ulonglong, c_int, _P]),
    "kr_gemm_ar_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_ulonglong, c_int, _P]),
    "kr_gemm_ce_producer_bf16": (c_int, [_P, c_longlong, _P, c_longlong, _P, c_longlong, c_int, c_int, c_int, c_int,
                                         c_int, _P, _P, _P]),
    "kr_tile_order_ag": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, _P]),
    "kr_tile_order": (c_int, [c_int, c_int, c_int, c_int, c_int, _P]),
    "kr_reduce_slabs": (c_int, [_P, _P, c_int, c_int, c_ulonglong, _P]),
}


def debug_build_selected() -> bool:
    return os.environ.get("KRAKEN_DEBUG", "0") == "1"


def lib_path() -> str:
    return str(_build.lib_path(debug_build_selected()))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        debug = debug_build_selected()
        target = _build.lib_path(debug)
        if os.environ.get("KRAKEN_NO_BUILD", "0") != "1" and _build.is_stale(debug):
            try:
                _build.build(debug=debug)
            except Exception:
                if not target.exists():
                    raise
        handle = ctypes.CDLL(str(target), mode=ctypes.RTLD_GLOBAL)
        for name, (res, args) in _PROTOS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().kr_last_error()
    return msg.decode() if msg else ""


def check(rc: int) -> None:
    if rc != 0:
        raise KrakenError(f"kraken_b200 native call failed (code {rc}): {last_error()}")


_STATUS_CODES = {1: "cross-device signal wait", 2: "intra-GPU flag wait", 3: "mbarrier wait", 4: "bounds check",
                 5: "CAS send"}


def decode_status(word: int) -> str:
    code, site, peer, block = word & 0xFF, (word >> 8) & 0xFF, (word >> 16) & 0xFF, (word >> 24) & 0xFF
    return f"{_STATUS_CODES.get(code, 'code %d' % code)} timed out at site {site} (peer {peer}, block {block})"


def current_stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def check_status(stream: int | None = None, clear: bool = True) -> None:
    """Synchronises the stream and raises KrakenSyncTimeout if a device wait gave up."""
    word = c_uint32(0)
    s = current_stream_ptr() if stream is None else stream
    check(lib().kr_read_status(s, ctypes.byref(word)))
    if word.value != 0:
        if clear:
            check(lib().kr_clear_status(s))
        raise KrakenSyncTimeout(decode_status(word.value))
