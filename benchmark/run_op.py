"""Runs ONE op a few times on one GPU — the small, self-terminating workload used for ncu captures
and quick timing (`python benchmark/run_op.py --op gemm --M 8192 --N 8192 --K 8192 --iters 3`).
Ops: gemm, gemm_swap (decode shape, operands swapped), gemm_tf32, rms_norm, ag_matmul (world size 1),
rs_pull / rs_scatter / rs_push (the fused reduce-scatter GEMM kernels at world size 1: CTA pairs,
reducer warps, counters), the memory-bound collectives at world size 1 (one_shot_ar, one_shot_ar_pull,
two_shot_ar, reduce_scatter, all_gather: M x K bf16 elements; ar_bias_norm_one_shot / _pull /
_two_shot: M rows of K), cublas (torch.matmul, for comparison). Prints the CUDA-event time of each
iteration; with --flush-l2 a 256 MB buffer is overwritten before each timed call."""
from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm")
    ap.add_argument("--M", type=int, default=8192)
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--pair", type=int, default=1, help="0: single-CTA GEMM kernel, 1: CTA-pair kernel when eligible")
    ap.add_argument("--flush-l2", action="store_true")
    args = ap.parse_args()
    import kraken_b200
    from kraken_b200 import comm, fused
    from kraken_b200.parallel import symm_mem

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    M, N, K = args.M, args.N, args.K
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    bt = (0.02 * torch.randn(N, K, device=dev)).to(torch.bfloat16)
    if args.op == "gemm":
        fn = lambda: fused.matmul(a, bt.t(), swap_ab=0, pair=args.pair)
    elif args.op == "gemm_swap":
        fn = lambda: fused.matmul(a, bt.t(), out_dtype=torch.float32, swap_ab=1)
    elif args.op == "cublas":
        fn = lambda: torch.matmul(a, bt.t())
    elif args.op == "rms_norm":
        w = torch.ones(K, device=dev, dtype=torch.bfloat16)
        fn = lambda: fused.rms_norm(a, w)
    elif args.op == "ag_matmul":
        xs = symm_mem.empty(M, K, dtype=torch.bfloat16, device=dev)
        xs.copy_(a)
        fn = lambda: fused.all_gather_matmul(xs, bt.t())
    elif args.op == "gemm_tf32":
        af, bf = a.float(), bt.float()
        fn = lambda: fused.matmul(af, bf.t(), out_dtype=torch.float32)
    elif args.op in ("rs_pull", "rs_scatter", "rs_push"):
        fn = lambda: fused.gemm_reduce_scatter(a, bt.t(), algo=args.op[3:], _force_fused=True)
    elif args.op in ("one_shot_ar", "one_shot_ar_pull", "two_shot_ar", "reduce_scatter", "all_gather"):
        xs = symm_mem.empty(M, K, dtype=torch.bfloat16, device=dev)
        xs.copy_(a)
        symm_mem.rendezvous(xs)
        fn = {"one_shot_ar": lambda: comm.one_shot_all_reduce(xs),
              "one_shot_ar_pull": lambda: comm.one_shot_all_reduce(xs, algo="pull"),
              "two_shot_ar": lambda: comm.two_shot_all_reduce(a),
              "reduce_scatter": lambda: comm.reduce_scatter(xs),
              "all_gather": lambda: comm.all_gather_w_progress(xs, backend="sm")}[args.op]
    elif args.op.startswith("ar_bias_norm"):
        pad = symm_mem.empty(M, K, dtype=torch.bfloat16, device=dev)
        symm_mem.rendezvous(pad)
        w = torch.ones(K, device=dev, dtype=torch.bfloat16)
        bias = torch.zeros(K, device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(a)
        if args.op.endswith("two_shot"):
            fn = lambda: fused.two_shot_all_reduce_bias_rms_norm(pad, a, bias, w, y, 1e-5)
        else:
            algo = "pull" if args.op.endswith("pull") else None
            fn = lambda: fused.one_shot_all_reduce_bias_rms_norm(pad, a, bias, w, y, 1e-5, algo=algo)
    else:
        raise SystemExit(f"unknown op {args.op}")
    cache = torch.empty(64 << 20, dtype=torch.int32, device=dev) if args.flush_l2 else None
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    for i in range(args.iters):
        b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if cache is not None:
            cache.zero_()
        b.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ms = b.elapsed_time(e)
        flops = 2.0 * M * N * K
        print(f"{args.op} M={M} N={N} K={K} iter {i}: {ms * 1000:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s", flush=True)
    kraken_b200.check_status()


if __name__ == "__main__":
    main()
