"""Host utilities: device-clock sampling for benchmarks, distributed bootstrap helpers, NVTX ranges
and the per-tile device timeline of the fused GEMM kernels."""
from .clocks import ClockSampler
from .dist import init_from_env
from .nvtx import nvtx_range
from .tile_trace import TileTrace

__all__ = ["ClockSampler", "TileTrace", "init_from_env", "nvtx_range"]
