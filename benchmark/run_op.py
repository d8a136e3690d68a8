"""Runs ONE op a few times on one GPU — the small, self-terminating workload used for ncu captures
and quick timing (`python benchmark/run_op.py --op gemm --M 8192 --N 8192 --K 8192 --iters 3`).
Ops: gemm, gemm_swap (decode shape, operands swapped), rms_norm, ag_matmul (world size 1),
cublas (torch.matmul, for comparison). Prints the CUDA-event time of each iteration."""
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
    args = ap.parse_args()
    import kraken_b200
    from kraken_b200 import fused
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
    else:
        raise SystemExit(f"unknown op {args.op}")
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    for i in range(args.iters):
        b, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
