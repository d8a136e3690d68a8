"""Host utilities: device-clock sampling for benchmarks, distributed bootstrap helpers."""
from .clocks import ClockSampler
from .dist import init_from_env
from .nvtx import nvtx_range

__all__ = ["ClockSampler", "init_from_env", "nvtx_range"]
