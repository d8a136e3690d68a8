"""Headline benchmark: the tensor-parallel MLP block made of the two fused GEMM + collective ops
the baseline names — all_gather_matmul (A shard [M/ws, 8192], B [8192, 28672/ws]) followed by
gemm_reduce_scatter (A [M, 28672/ws], B [28672/ws, 8192]) at M = 8192, bf16, synthetic data,
random-initialised weights. One "step" = both ops back to back on one stream.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the unmodified reference (baseline/_ref)

For N > 1 launch with torchrun (one rank per GPU); RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* are
read from the environment. Rank 0 prints ONE JSON line. `value` is the whole-job dense bf16
throughput in TFLOP/s (sum over all ranks of 2*M*N*K per GEMM divided by the step time, device-timed
with CUDA events, max over ranks); total work is fixed as N grows (strong scaling). Per-op
microseconds, NVLink bytes and roofline fractions are in `ops`. Between timed iterations nothing is
flushed: the step's working set (weights + activations, > 280 MB per rank at every N) exceeds the
126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_TOKENS = 8192
HIDDEN = 8192
FFN = 28672


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", 0)),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    except Exception:
        return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def _event_times(fn, steps, sync):
    import torch

    begins = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    sync()
    for i in range(steps):
        begins[i].record()
        fn()
        ends[i].record()
    sync()
    return [b.elapsed_time(e) for b, e in zip(begins, ends)]


def run_ours(args):
    import torch
    import torch.distributed as dist

    import kraken_b200
    from kraken_b200 import fused
    from kraken_b200.parallel import symm_mem
    from kraken_b200.utils import ClockSampler, init_from_env

    rank, local_rank, ws = init_from_env()
    dev = torch.device("cuda", torch.cuda.current_device())
    M, H, F = M_TOKENS, HIDDEN, FFN
    assert F % ws == 0 and M % ws == 0
    Fl, Ml = F // ws, M // ws
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    # weights K-major (nn.Linear layout): w_up_t [F/ws, H], w_down_t [H, F/ws]
    w_up_t = (0.02 * torch.randn(Fl, H, generator=g)).to(torch.bfloat16).to(dev)
    w_down_t = (0.02 * torch.randn(H, Fl, generator=g)).to(torch.bfloat16).to(dev)
    x_host = torch.randn(Ml, H, generator=g).to(torch.bfloat16).pin_memory()
    x_bufs = []
    for _ in range(2):                      # double-buffered symmetric input: step i+1's H2D overlaps step i
        xb = symm_mem.empty(Ml, H, dtype=torch.bfloat16, device=dev)
        symm_mem.rendezvous(xb)
        xb.copy_(x_host)
        x_bufs.append(xb)
    x_symm = x_bufs[0]
    copy_stream = torch.cuda.Stream()

    def sync():
        if ws > 1:
            dist.barrier(device_ids=[dev.index])
        torch.cuda.synchronize()

    def step(x=None):
        _, h = fused.all_gather_matmul(x_symm if x is None else x, w_up_t.t())
        return fused.gemm_reduce_scatter(h, w_down_t.t())

    def run_e2e(k):
        """k serving steps through the public API. Every step's input goes host (pinned) -> device
        and every step's result metric comes back device -> host inside the timed region. The copy
        of step i+1's input runs on a second stream while step i computes, and the host reads step
        i's result while step i+1 runs: the loop is never more than one step ahead of the results it
        has read (a serving loop that overlaps post-processing with the next forward)."""
        cur = torch.cuda.current_stream()
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        done = [torch.cuda.Event(), torch.cuda.Event()]
        got = [torch.cuda.Event(), torch.cuda.Event()]
        results = [torch.empty(1, dtype=torch.float32).pin_memory() for _ in range(2)]
        sink = 0.0
        t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync()
        t_begin.record(cur)
        copy_stream.wait_event(t_begin)
        with torch.cuda.stream(copy_stream):
            x_bufs[0].copy_(x_host, non_blocking=True)
            ready[0].record(copy_stream)
        for i in range(k):
            b = i & 1
            if i + 1 < k:
                with torch.cuda.stream(copy_stream):
                    if i >= 1:
                        copy_stream.wait_event(done[1 - b])      # step i-1 has finished with that buffer
                    x_bufs[1 - b].copy_(x_host, non_blocking=True)
                    ready[1 - b].record(copy_stream)
            cur.wait_event(ready[b])
            y = step(x_bufs[b])
            done[b].record(cur)
            results[b].copy_(y.float().abs().mean().reshape(1), non_blocking=True)   # the step's metric, D2H
            got[b].record(cur)
            if i >= 1:
                got[1 - b].synchronize()                         # step i-1's result is on the host
                sink += float(results[1 - b][0])
        got[(k - 1) & 1].synchronize()
        sink += float(results[(k - 1) & 1][0])
        t_end.record(cur)
        sync()
        assert sink == sink                                        # the results were read (and are numbers)
        return t_begin.elapsed_time(t_end) / k

    def op_ag():
        fused.all_gather_matmul(x_symm, w_up_t.t())

    h_fixed = (torch.randn(M, Fl, generator=g).to(torch.bfloat16)).to(dev)

    def op_rs():
        fused.gemm_reduce_scatter(h_fixed, w_down_t.t())

    def op_rs_ce():
        fused.gemm_reduce_scatter_ce_persistent(h_fixed, w_down_t.t())

    sampler = ClockSampler(gpu_index=dev.index).start() if rank == 0 else None
    for _ in range(max(3, args.warmup)):
        step()
    sync()
    kraken_b200.check_status()

    t_mark0 = time.perf_counter()
    times = _event_times(step, args.steps, sync)
    t_mark1 = time.perf_counter()
    wall = t_mark1 - t_mark0
    kraken_b200.check_status()

    def maxr(v):
        if ws == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ms_step = maxr(sum(times) / len(times))
    # per-op numbers (median, max over ranks)
    ops = {}
    for name, fn in (("all_gather_matmul", op_ag), ("gemm_reduce_scatter", op_rs),
                     ("gemm_reduce_scatter_ce_persistent", op_rs_ce)):
        for _ in range(3):
            fn()
        ts = sorted(_event_times(fn, max(3, args.steps), sync))
        ops[name] = {"us": maxr(ts[len(ts) // 2] * 1000.0)}
    # end to end through the public API, with the H2D input copy and the D2H result read every step
    run_e2e(3)
    ms_e2e = maxr(run_e2e(args.steps))
    kraken_b200.check_status()
    clocks = sampler.stop(t_mark0, t_mark1) if sampler is not None else None

    flops_step = 2.0 * M * F * H * 2          # whole job: two GEMMs of 2*M*(F)*(H) each
    peaks = _peaks()
    value = flops_step / (ms_step * 1e-3) / 1e12
    e2e_value = flops_step / (ms_e2e * 1e-3) / 1e12
    per_gemm_flops_rank = 2.0 * M * F * H / ws
    link = 770e9
    for name, nv_bytes in (("all_gather_matmul", (ws - 1) * Ml * H * 2), ("gemm_reduce_scatter", (ws - 1) * Ml * H * 2),
                           ("gemm_reduce_scatter_ce_persistent", (ws - 1) * Ml * H * 2)):
        t_mma = per_gemm_flops_rank / (peaks["bf16_tflops"] * 1e12)
        t_link = nv_bytes / link
        roof = max(t_mma, t_link)
        ops[name].update({"nvlink_bytes": nv_bytes, "roofline_us": roof * 1e6,
                          "frac_of_roofline": roof * 1e6 / ops[name]["us"],
                          "tflops_per_gpu": per_gemm_flops_rank / (ops[name]["us"] * 1e-6) / 1e12})
    if rank == 0:
        out = {
            "metric": "tp_mlp_fused_ag_matmul_plus_gemm_rs_tflops",
            "value": value, "unit": "TFLOP/s (bf16 dense, whole job)", "n_gpus": ws, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random activations, random-init weights)",
            "impl": "kraken_b200",
            "config": {"model": "tp_mlp_block(all_gather_matmul -> gemm_reduce_scatter)", "global_batch": M,
                       "seq_len": 1, "hidden": H, "ffn": F, "parallelism": f"tp{ws}",
                       "l2": "no flush: per-step working set exceeds the 126 MB L2",
                       "timing": "CUDA events per step on the launching stream, mean over steps, max over ranks"},
            "ops": ops,
            "roofline_denominators": peaks,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s (bf16 dense, whole job)", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": Ml * H * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": 2 * args.steps,   # per step: the all-gather GEMM kernel and the reduce-scatter GEMM kernel
            "wall_s": wall,
        }
        print(json.dumps(out), flush=True)
    if ws > 1:
        dist.barrier(device_ids=[dev.index])
        dist.destroy_process_group()


def run_reference(args):
    from baseline import reference_arm

    reference_arm.main(args, M_TOKENS, HIDDEN, FFN)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
