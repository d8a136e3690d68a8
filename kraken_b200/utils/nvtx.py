"""Optional NVTX ranges around the public ops (``KRAKEN_NVTX=1``), so that timeline tools show one
named range per call. The reference gives profilers per-launch names through Triton launch
metadata hooks (kraken/fused/all_gather_matmul.py:12-25); here the op name is the range name."""
from __future__ import annotations

import functools

from .. import config


def nvtx_range(fn):
    """Decorator: pushes/pops an NVTX range named after the function when enabled; free when not."""
    if not config.nvtx_enabled():
        return fn

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        import torch

        if not torch.cuda.is_available():
            return fn(*args, **kwargs)
        torch.cuda.nvtx.range_push(f"kraken_b200.{fn.__name__}")
        try:
            return fn(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()

    return wrapped
