"""Communication fused with compute (reference: kraken/fused/__init__.py:1-27; like the reference,
``gemm_one_shot_all_reduce`` is also exported as ``gemm_one_shot_all_reduce_fused``)."""
from .all_reduce_bias import (
    one_shot_all_reduce_bias,
    one_shot_all_reduce_bias_rms_norm,
    two_shot_all_reduce_bias,
    two_shot_all_reduce_bias_rms_norm,
)
from .gemm_ops import (
    all_gather_matmul,
    gemm_one_shot_all_reduce,
    gemm_reduce_scatter,
    gemm_reduce_scatter_ce_persistent,
    matmul,
)
from .rms_norm import rms_norm

gemm_one_shot_all_reduce_fused = gemm_one_shot_all_reduce

__all__ = [
    "all_gather_matmul",
    "gemm_one_shot_all_reduce",
    "gemm_one_shot_all_reduce_fused",
    "gemm_reduce_scatter",
    "gemm_reduce_scatter_ce_persistent",
    "matmul",
    "one_shot_all_reduce_bias",
    "one_shot_all_reduce_bias_rms_norm",
    "rms_norm",
    "two_shot_all_reduce_bias",
    "two_shot_all_reduce_bias_rms_norm",
]

# optional NVTX ranges (KRAKEN_NVTX=1): wrap the public callables of this module
from ..utils.nvtx import nvtx_range as _nvtx_range  # noqa: E402

for _name in list(__all__):
    _obj = globals()[_name]
    if callable(_obj):
        globals()[_name] = _nvtx_range(_obj)
