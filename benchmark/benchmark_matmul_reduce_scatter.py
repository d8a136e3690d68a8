"""Matmul + reduce-scatter (reference: benchmark/benchmark_matmul_reduce_scatter.py). Per rank:
A bf16 [M, K/ws], B bf16 [K/ws, N] (b.T contiguous); output [M/ws, N]. Backends: this library's
fused kernel and its copy-engine variant, cuBLAS + NCCL reduce_scatter, torch's
fused_matmul_reduce_scatter, the reference's Triton kernels. ``--shape M,N,K`` (repeatable list)
follows the reference: per rank A [M, K] and B [K, N]; ``-dtype`` is accepted and must be bfloat16
(the reference's script defaults to float32 inputs, which this library would cast to bf16)."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import check_dtype, shape_triple, finish, load_reference, peaks, print_table, setup, try_time, NVLINK_GBS_MEASURED


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, nargs="*", default=[2048, 8192])
    ap.add_argument("--K", type=int, default=28672, help="global K; each rank holds K / world_size")
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--shape", type=shape_triple, nargs="+", default=None,
                    help="per-rank shapes M,N,K as in the reference's script (overrides --M/--N/--K)")
    ap.add_argument("-dtype", default="bfloat16")
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--save-path", default="results/bench_matmul_reduce_scatter")
    args = ap.parse_args()
    check_dtype(args.dtype)
    rank, ws, dev = setup()
    from kraken_b200 import fused

    ref, why = load_reference()
    pk = peaks()
    rows = []
    problems = [(m, k, n) for (m, n, k) in args.shape] if args.shape else [(M, args.K // ws, args.N) for M in args.M]
    for M, Kl, N in problems:
        a = torch.randn(M, Kl, device=dev).to(torch.bfloat16)
        bt = (0.02 * torch.randn(N, Kl, device=dev)).to(torch.bfloat16)
        b = bt.t()

        def cublas_nccl():
            c = torch.matmul(a, b)
            out = torch.empty(M // ws, N, dtype=torch.bfloat16, device=dev)
            dist.reduce_scatter_tensor(out, c)
            return out

        golden = cublas_nccl().float()
        backends = {
            "kraken_b200": lambda: fused.gemm_reduce_scatter(a, b),
            "kraken_b200_pull": lambda: fused.gemm_reduce_scatter(a, b, algo="pull"),
            "kraken_b200_scatter": lambda: fused.gemm_reduce_scatter(a, b, algo="scatter"),
            "kraken_b200_push": lambda: fused.gemm_reduce_scatter(a, b, algo="push"),
            "kraken_b200_ce": lambda: fused.gemm_reduce_scatter_ce_persistent(a, b),
            "cublas_nccl": cublas_nccl,
            "cublas_only": lambda: torch.matmul(a, b),
        }
        try:
            gname = dist.group.WORLD.group_name
            backends["torch_symm_mem"] = lambda: torch.ops.symm_mem.fused_matmul_reduce_scatter(a, b, "sum", 0, gname)
        except Exception as e:
            why = why or str(e)
        if ref is not None:
            backends["ref_triton_ce"] = lambda: ref.fused.gemm_reduce_scatter_ce_persistent(a, b)
            # the reference's single-kernel variant launches one block per 64x64 tile and indexes the
            # signal pad by block id: only run it where that stays inside torch's 2304-slot pad
            if (M // 64) * (N // 64) * ws <= 2304:
                backends["ref_triton"] = lambda: ref.fused.gemm_reduce_scatter(a, b)
        torch.testing.assert_close(fused.gemm_reduce_scatter(a, b).float(), golden, atol=2e-1, rtol=1e-1)
        flops = 2.0 * M * N * Kl
        nv_out = (ws - 1) * (M // ws) * N * 2
        roof_us = max(flops / (pk["bf16_tflops"] * 1e12), nv_out / (NVLINK_GBS_MEASURED * 1e9)) * 1e6
        row = {"M": M, "K_per_rank": Kl, "N": N, "roofline_us": roof_us}
        for name, fn in backends.items():
            us, err = try_time(fn, iters=args.iters, warmup=5)
            row[name + "_us"] = us
            if us is None and rank == 0:
                print(f"[{name}] n/a: {err}", flush=True)
        if row.get("kraken_b200_us"):
            row["frac_of_roofline"] = roof_us / row["kraken_b200_us"]
            row["tflops_per_gpu"] = flops / (row["kraken_b200_us"] * 1e-6) / 1e12
        rows.append(row)
    cols = ["M", "K_per_rank", "N", "roofline_us", "frac_of_roofline", "tflops_per_gpu"] + \
        sorted({k for r in rows for k in r if k.endswith("_us") and k != "roofline_us"})
    print_table(rows, cols, f"matmul_reduce_scatter, {ws} x B200 ({pk['source']} peaks)", f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
