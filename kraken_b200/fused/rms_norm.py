"""Row RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, fp32 math (reference: kraken/fused/rms_norm.py:46-72)."""
from __future__ import annotations

import torch

from .. import _reference as ref
from .._logging import utils as _log
from ..ops import lib as _lib


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if x.device.type != "cuda":
        return ref.rms_norm(x, w, eps)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise TypeError("rms_norm supports bfloat16 input and weight")
    D = x.shape[-1]
    if w.numel() != D or D % 8:
        raise ValueError("weight must have the last dimension's size, which must be a multiple of 8")
    xc = x.contiguous()
    _log.log_kernel_choice("rms_norm", f"rows={xc.numel() // D} D={D}")
    y = torch.empty_like(xc)
    _lib.check(_lib.lib().kr_rms_norm(xc.data_ptr(), w.contiguous().data_ptr(), y.data_ptr(), xc.numel() // D, D,
                                      float(eps), _lib.current_stream_ptr()))
    return y
