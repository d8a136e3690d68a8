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
