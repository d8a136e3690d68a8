"""Pure communication ops over symmetric memory (reference: kraken/comm/__init__.py:1-17, plus the
two ops its README names without shipping: ``multimem_all_reduce`` and ``reduce_scatter``)."""
from .all_gather import _copy_engine_all_gather_w_progress, _sm_all_gather_w_progress, all_gather_w_progress
from .all_reduce import all_reduce, multimem_all_reduce, one_shot_all_reduce, reduce_scatter, two_shot_all_reduce

__all__ = [
    "_copy_engine_all_gather_w_progress",
    "_sm_all_gather_w_progress",
    "all_gather_w_progress",
    "all_reduce",
    "multimem_all_reduce",
    "one_shot_all_reduce",
    "reduce_scatter",
    "two_shot_all_reduce",
]

# optional NVTX ranges (KRAKEN_NVTX=1): wrap the public callables of this module
from ..utils.nvtx import nvtx_range as _nvtx_range  # noqa: E402

for _name in list(__all__):
    _obj = globals()[_name]
    if callable(_obj):
        globals()[_name] = _nvtx_range(_obj)
