from .benchmarking import benchmark_with_event, benchmark_with_profiler, bus_bandwidth_gbs
from .utils import log_kernel, log_triton_kernel, plot_experiment_comparison

__all__ = ["benchmark_with_event", "benchmark_with_profiler", "bus_bandwidth_gbs", "log_kernel",
           "log_triton_kernel", "plot_experiment_comparison"]
