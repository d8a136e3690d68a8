"""Reference arm of bench.py: runs the UNMODIFIED reference package installed under
baseline/_ref (``pip install --target baseline/_ref <reference checkout>``) through its own public
API on the same metric and config as the library's arm:

    kraken.fused.all_gather_matmul(a_shared [M/ws, 8192], b [8192, 28672/ws])
    kraken.fused.gemm_reduce_scatter_ce_persistent(a [M, 28672/ws], b [28672/ws, 8192])

The reference has two GEMM + reduce-scatter ops. Its single-kernel ``gemm_reduce_scatter`` launches
one block per 64 x 64 tile (16384 blocks at this shape) and indexes the signal pad by block id, far
past the pad's 2304 slots, so it is not run on this shape; the persistent copy-engine variant is
the one its own tests use for large shapes (test/test_gemm_reduce_scatter.py, M=8192 N=4096 K=14336).
Nothing from kraken_b200 is imported here.
"""
from __future__ import annotations

import datetime
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", 0)) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}), flush=True)


def main(args, M, H, F) -> None:
    if not os.path.isdir(os.path.join(REF_DIR, "kraken")):
        _unavailable("reference package not installed under baseline/_ref")
        return
    try:
        _run(args, M, H, F)
    except Exception as e:  # the reference could not run on this box: report, exit 0
        _unavailable(f"{type(e).__name__}: {e}")


def _run(args, M, H, F) -> None:
    import torch
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm_mem

    sys.path.insert(0, REF_DIR)
    import kraken  # the reference

    assert os.path.realpath(kraken.__file__).startswith(os.path.realpath(REF_DIR))
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    ws = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=600),
                            device_id=dev)
    Fl, Ml = F // ws, M // ws
    g = torch.Generator(device="cpu").manual_seed(1234 + rank)
    w_up_t = (0.02 * torch.randn(Fl, H, generator=g)).to(torch.bfloat16).to(dev)
    w_down_t = (0.02 * torch.randn(H, Fl, generator=g)).to(torch.bfloat16).to(dev)
    x_host = torch.randn(Ml, H, generator=g).to(torch.bfloat16).pin_memory()
    x_bufs = []
    for _ in range(2):
        xb = symm_mem.empty(Ml, H, dtype=torch.bfloat16, device=dev)
        symm_mem.rendezvous(xb, group=dist.group.WORLD)
        xb.copy_(x_host)
        x_bufs.append(xb)
    x_symm = x_bufs[0]
    a_out = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    progress = torch.zeros(ws, dtype=torch.uint32, device=dev)
    copy_stream = torch.cuda.Stream()
    b_up = w_up_t.t()        # [H, F/ws] with b.T contiguous, as the reference requires
    b_down = w_down_t.t()

    def sync():
        dist.barrier(device_ids=[dev.index])
        torch.cuda.synchronize()

    def step(x=None):
        _, h = kraken.fused.all_gather_matmul(x_symm if x is None else x, b_up, a_out=a_out, progress=progress)
        return kraken.fused.gemm_reduce_scatter_ce_persistent(h, b_down)

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
            bb = i & 1
            if i + 1 < k:
                with torch.cuda.stream(copy_stream):
                    if i >= 1:
                        copy_stream.wait_event(done[1 - bb])      # step i-1 has finished with that buffer
                    x_bufs[1 - bb].copy_(x_host, non_blocking=True)
                    ready[1 - bb].record(copy_stream)
            cur.wait_event(ready[bb])
            y = step(x_bufs[bb])
            done[bb].record(cur)
            results[bb].copy_(y.float().abs().mean().reshape(1), non_blocking=True)   # the step's metric, D2H
            got[bb].record(cur)
            if i >= 1:
                got[1 - bb].synchronize()                         # step i-1's result is on the host
                sink += float(results[1 - bb][0])
        got[(k - 1) & 1].synchronize()
        sink += float(results[(k - 1) & 1][0])
        t_end.record(cur)
        sync()
        assert sink == sink                                        # the results were read (and are numbers)
        return t_begin.elapsed_time(t_end) / k

    def timed(fn, n):
        begins = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(n)]
        sync()
        for i in range(n):
            begins[i].record()
            fn()
            ends[i].record()
        sync()
        return [b.elapsed_time(e) for b, e in zip(begins, ends)]

    def maxr(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(3, args.warmup)):
        step()
    sync()
    t0 = time.perf_counter()
    times = timed(step, args.steps)
    wall = time.perf_counter() - t0
    ms_step = maxr(sum(times) / len(times))
    run_e2e(3)
    ms_e2e = maxr(run_e2e(args.steps))
    ops = {}
    h_fixed = torch.randn(M, Fl, generator=g).to(torch.bfloat16).to(dev)
    for name, fn in (("all_gather_matmul", lambda: kraken.fused.all_gather_matmul(x_symm, b_up, a_out=a_out, progress=progress)),
                     ("gemm_reduce_scatter_ce_persistent", lambda: kraken.fused.gemm_reduce_scatter_ce_persistent(h_fixed, b_down))):
        for _ in range(3):
            fn()
        ts = sorted(timed(fn, max(3, args.steps)))
        ops[name] = {"us": maxr(ts[len(ts) // 2] * 1000.0)}
    flops_step = 2.0 * M * F * H * 2
    if rank == 0:
        print(json.dumps({
            "metric": "tp_mlp_fused_ag_matmul_plus_gemm_rs_tflops", "impl": "reference",
            "value": flops_step / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s (bf16 dense, whole job)", "n_gpus": ws,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (random activations, random-init weights)",
            "config": {"model": "tp_mlp_block(all_gather_matmul -> gemm_reduce_scatter_ce_persistent)",
                       "global_batch": M, "seq_len": 1, "hidden": H, "ffn": F, "parallelism": f"tp{ws}",
                       "l2": "no flush: per-step working set exceeds the 126 MB L2"},
            "ops": ops,
            "e2e": {"value": flops_step / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s (bf16 dense, whole job)",
                    "ms_per_step": ms_e2e, "h2d_bytes_per_step": Ml * H * 2, "d2h_bytes_per_step": 4},
            "wall_s": wall,
        }), flush=True)
    dist.barrier(device_ids=[dev.index])
    dist.destroy_process_group()
