"""Host utilities: device-clock sampling for benchmarks, distributed bootstrap helpers."""
from .clocks import ClockSampler
from .dist import init_from_env

__all__ = ["ClockSampler", "init_from_env"]
