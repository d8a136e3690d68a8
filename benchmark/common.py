"""Shared plumbing of the benchmark scripts: process-group start-up, timing with the library's
harness (CUDA events, L2 flush, median, max over ranks), optional import of the reference package
installed under baseline/_ref, and result tables (markdown on stdout, JSON/markdown files)."""
from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from kraken_b200._logging import benchmark_with_event, bus_bandwidth_gbs  # noqa: E402
from kraken_b200.utils import init_from_env  # noqa: E402

NVLINK_GBS_MEASURED = 770.0     # peer copy per direction on this pool's B200s
NVLINK_GBS_NOMINAL = 900.0


def setup():
    rank, local_rank, ws = init_from_env()
    if ws == 1 and not dist.is_initialized():
        # a 1-rank group keeps torch's symmetric memory and the reference usable at N=1
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29544")
        dist.init_process_group("nccl", rank=0, world_size=1,
                                device_id=torch.device("cuda", torch.cuda.current_device()))
    torch.manual_seed(42 + rank)
    return rank, ws, torch.device("cuda", torch.cuda.current_device())


def peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def load_reference():
    """The unmodified reference package (its Triton kernels), or None with the reason."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "kraken")):
        return None, "reference not installed under baseline/_ref"
    try:
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        import kraken

        return kraken, ""
    except Exception as e:
        return None, f"{type(e).__name__}: {e}"


def time_us(fn, iters: int = 25, warmup: int = 20, flush_l2: bool = True) -> float:
    return benchmark_with_event(fn, warmup_iters=warmup, benchmark_iters=iters, flush_l2=flush_l2, max_over_ranks=True)


def try_time(fn, **kw):
    """Times fn; a backend that cannot run a shape yields (None, reason) instead of aborting."""
    try:
        fn()
        torch.cuda.synchronize()
        return time_us(fn, **kw), ""
    except Exception as e:
        try:
            torch.cuda.synchronize()
        except Exception:
            pass
        return None, f"{type(e).__name__}: {str(e)[:120]}"


def print_table(rows: list[dict], columns: list[str], title: str, save_prefix: str | None = None) -> None:
    if dist.is_initialized() and dist.get_rank() != 0:
        return
    def fmt(v):
        if v is None:
            return "n/a"
        if isinstance(v, float):
            return f"{v:.1f}" if abs(v) >= 10 else f"{v:.3g}"
        return str(v)
    lines = [f"### {title}", "", "| " + " | ".join(columns) + " |", "|" + "---|" * len(columns)]
    for r in rows:
        lines.append("| " + " | ".join(fmt(r.get(c)) for c in columns) + " |")
    text = "\n".join(lines)
    print(text, flush=True)
    if save_prefix:
        os.makedirs(os.path.dirname(save_prefix) or ".", exist_ok=True)
        with open(save_prefix + ".md", "w") as f:
            f.write(text + "\n")
        with open(save_prefix + ".json", "w") as f:
            json.dump({"title": title, "rows": rows}, f, indent=1)


def shape_triple(text: str) -> tuple[int, int, int]:
    """"M,N,K" or "MxNxK" -> (M, N, K): the `--shape` argument of the GEMM benchmarks (the reference
    takes the same three numbers, benchmark/benchmark_all_gather_matmul.py:222-232)."""
    parts = [t for t in text.replace("x", ",").replace("(", "").replace(")", "").split(",") if t.strip()]
    if len(parts) != 3:
        raise ValueError("a shape is three integers: M,N,K")
    return tuple(int(t) for t in parts)


def check_dtype(name: str) -> None:
    """`-dtype` is accepted for command-line compatibility with the reference's scripts; the
    tensor-core and collective kernels of this library are bf16 (fp32 inputs would be cast)."""
    if name not in ("bfloat16", "bf16"):
        raise SystemExit(f"-dtype {name}: this library's kernels are bfloat16; run with -dtype bfloat16")


def plot_rows(rows: list[dict], label_keys: list[str], save_prefix: str | None) -> None:
    """Line chart of every *_us column over the rows (rank 0), as the reference's bias benchmarks do."""
    if not save_prefix or (dist.is_initialized() and dist.get_rank() != 0) or not rows:
        return
    from kraken_b200._logging import plot_experiment_comparison

    names = sorted({k for r in rows for k in r if k.endswith("_us") and k != "roofline_us"})
    sizes = [" ".join(f"{k}:{r[k]}" for k in label_keys) for r in rows]
    data = [[r.get(n) for n in names] for r in rows]
    plot_experiment_comparison(sizes, [n[:-3] for n in names], data, save_prefix + ".png")


def finish():
    if dist.is_initialized():
        dist.barrier(device_ids=[torch.cuda.current_device()])
        dist.destroy_process_group()
