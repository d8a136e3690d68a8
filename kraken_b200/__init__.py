"""kraken_b200 — symmetric-memory communication and fused comm+compute operators, hand-written
for NVIDIA B200 (sm_100a): tcgen05/TMEM/TMA GEMMs fused with in-kernel NVLink collectives.

Subpackages mirror the reference's layout (kraken/__init__.py:1-13): ``comm``, ``fused``,
``_ptx_utils``, ``_logging``; plus ``parallel`` (symmetric memory, groups, rank emulation), ``ops``
(native library), ``models`` (tensor-parallel MLP block), ``_reference`` (pure-PyTorch oracle and
CPU backend), ``utils``.
"""
from . import config  # noqa: F401
from . import _logging, _ptx_utils, _reference, comm, fused, models, ops, parallel, utils  # noqa: F401
from .ops import KrakenError, KrakenSyncTimeout, check_status
from .parallel import symm_mem

__version__ = "0.1.0"
__all__ = ["_logging", "_ptx_utils", "_reference", "comm", "fused", "models", "ops", "parallel", "utils", "config",
           "symm_mem", "KrakenError", "KrakenSyncTimeout", "check_status"]
