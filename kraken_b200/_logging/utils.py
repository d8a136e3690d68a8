"""Kernel-choice logging and result plotting (reference: kraken/_logging/utils.py:9-57).

The reference dumps the PTX Triton generated for a kernel at exit; these kernels are compiled ahead
of time, so ``log_triton_kernel`` (name kept for drop-in use) records what there is to record: the
variant each launch picked, written to a text file at exit by rank 0.
``plot_experiment_comparison`` draws the same line chart to a PNG when matplotlib is installed and
is a no-op otherwise.
"""
from __future__ import annotations

import atexit
import os
import tempfile

_records: list[str] = []
_registered = False


def log_triton_kernel(kernel) -> None:
    """Registers a description of a launched kernel; all records are written to
    ``<tmp>/kraken_b200_kernels.txt`` at interpreter exit."""
    global _registered
    _records.append(str(kernel))
    if not _registered:
        _registered = True

        def _flush():
            path = os.path.join(tempfile.gettempdir(), "kraken_b200_kernels.txt")
            with open(path, "w") as f:
                f.write("\n".join(_records) + "\n")

        atexit.register(_flush)


log_kernel = log_triton_kernel


def plot_experiment_comparison(sizes, series: dict, save_path: str, title: str = "", xlabel: str = "size",
                               ylabel: str = "latency (us)") -> bool:
    """series: name -> list of values aligned with `sizes`. Returns True when a PNG was written."""
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except Exception:
        return False
    fig, ax = plt.subplots(figsize=(8, 5))
    for name, vals in series.items():
        ax.plot(range(len(sizes)), vals, marker="o", label=name)
    ax.set_xticks(range(len(sizes)))
    ax.set_xticklabels([str(s) for s in sizes], rotation=45)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    ax.set_title(title)
    ax.legend()
    ax.grid(True, alpha=0.3)
    fig.tight_layout()
    fig.savefig(save_path)
    plt.close(fig)
    return True
