"""Kernel-choice logging and result plotting (reference: kraken/_logging/utils.py:9-57).

The reference's ops call ``log_triton_kernel(kernel)`` under ``SYMM_DUMP_KERNEL=1`` and dump the
PTX Triton generated at exit. The kernels here are compiled ahead of time and nothing is
disassembled, so what there is to record per launch is the variant the op picked (algorithm,
tiling, engine). Every public op reports it through ``log_kernel_choice``; with
``KRAKEN_DUMP_KERNEL=1`` (or the reference's ``SYMM_DUMP_KERNEL=1``) rank 0 prints each distinct
choice once and writes all of them to ``<tmp>/kraken_b200_kernels.txt`` at interpreter exit.
``log_triton_kernel`` is kept under the reference's name for drop-in use and takes any object.

``plot_experiment_comparison(sizes, experiments, data, filename)`` has the reference's signature:
``data[i][j]`` is the time of experiment ``j`` at size ``i``. It draws one line per experiment into
a PNG when matplotlib is installed; without matplotlib it writes the same table as CSV next to
the requested file name and returns False.
"""
from __future__ import annotations

import atexit
import os
import tempfile

_records: list[str] = []
_seen: set[str] = set()
_registered = False


def _is_rank0() -> bool:
    try:
        import torch.distributed as dist

        return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0
    except Exception:
        return True


def dump_enabled() -> bool:
    return os.environ.get("KRAKEN_DUMP_KERNEL", "0") == "1" or os.environ.get("SYMM_DUMP_KERNEL", "0") == "1"


def _flush() -> None:
    path = os.path.join(tempfile.gettempdir(), "kraken_b200_kernels.txt")
    with open(path, "w") as f:
        f.write("\n".join(_records) + "\n")


def log_triton_kernel(kernel) -> None:
    """Registers a description of a launched kernel (rank 0 only); the records are written to
    ``<tmp>/kraken_b200_kernels.txt`` at interpreter exit."""
    global _registered
    if not _is_rank0():
        return
    text = str(kernel)
    if text in _seen:
        return
    _seen.add(text)
    _records.append(text)
    if not _registered:
        _registered = True
        atexit.register(_flush)


log_kernel = log_triton_kernel


def log_kernel_choice(op: str, detail: str) -> None:
    """Called by every public op with the variant it is about to launch. Costs one environment
    lookup when dumping is off."""
    if not dump_enabled() or not _is_rank0():
        return
    text = f"{op}: {detail}"
    if text not in _seen:
        print(f"[kraken_b200] {text}", flush=True)
    log_triton_kernel(text)


def recorded_kernels() -> list[str]:
    return list(_records)


def plot_experiment_comparison(sizes, experiments, data, filename: str) -> bool:
    """One line per experiment over the input sizes. ``data`` has one row per size and one column
    per experiment (a ``None`` entry leaves a gap). Returns True when a PNG was written."""
    sizes = [str(s) for s in sizes]
    experiments = list(experiments)
    rows = [list(r) for r in data]
    if len(rows) != len(sizes) or any(len(r) != len(experiments) for r in rows):
        raise ValueError("data must have one row per size and one column per experiment")
    try:
        import matplotlib

        matplotlib.use("Agg")
        from matplotlib import pyplot
    except Exception:
        csv_path = os.path.splitext(filename)[0] + ".csv"
        with open(csv_path, "w") as f:
            f.write("size," + ",".join(experiments) + "\n")
            for s, r in zip(sizes, rows):
                f.write(s + "," + ",".join("" if v is None else f"{v:.3f}" for v in r) + "\n")
        return False
    fig, ax = pyplot.subplots(figsize=(11, 5.5))
    xs = list(range(len(sizes)))
    for j, name in enumerate(experiments):
        ys = [float("nan") if r[j] is None else float(r[j]) for r in rows]
        ax.plot(xs, ys, marker="o", linewidth=1.5, label=name)
    ax.set_xticks(xs)
    ax.set_xticklabels(sizes, rotation=30, ha="right")
    ax.set_xlabel("input size")
    ax.set_ylabel("time per call (us)")
    ax.set_yscale("log")
    ax.grid(True, which="both", axis="y", alpha=0.3)
    ax.legend()
    fig.tight_layout()
    fig.savefig(filename, dpi=200)
    pyplot.close(fig)
    return True
