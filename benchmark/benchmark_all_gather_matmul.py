"""All-gather + matmul (reference: benchmark/benchmark_all_gather_matmul.py). Per rank: A shard
bf16 [M/ws, K], B bf16 [K, N/ws] column-major (b.T contiguous). Backends: this library's fused
kernel (in-kernel pull and copy-engine engines), NCCL all_gather + cuBLAS, torch's
fused_all_gather_matmul, the reference's Triton kernel. Roofline = max(FLOPs / measured cuBLAS
peak, NVLink bytes in / 770 GB/s). ``--shape M,N,K`` (repeatable list) follows the reference: per
rank an A shard [M, K] and B [K, N], so the GEMM is [M * world_size, K] x [K, N]; ``-dtype`` is
accepted and must be bfloat16."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import check_dtype, shape_triple, finish, load_reference, peaks, print_table, setup, try_time, NVLINK_GBS_MEASURED


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, nargs="*", default=[2048, 8192])
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--N", type=int, default=28672, help="global N; each rank holds N / world_size columns")
    ap.add_argument("--shape", type=shape_triple, nargs="+", default=None,
                    help="per-rank shapes M,N,K as in the reference's script (overrides --M/--N/--K)")
    ap.add_argument("-dtype", default="bfloat16")
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--save-path", default="results/bench_all_gather_matmul")
    args = ap.parse_args()
    check_dtype(args.dtype)
    rank, ws, dev = setup()
    from kraken_b200 import fused
    from kraken_b200.parallel import symm_mem
    import torch.distributed._symmetric_memory as tsm

    ref, why = load_reference()
    pk = peaks()
    rows = []
    problems = [(m * ws, k, n) for (m, n, k) in args.shape] if args.shape else [(M, args.K, args.N // ws) for M in args.M]
    for M, K, Nl in problems:
        Ml = M // ws
        a = torch.randn(Ml, K, device=dev).to(torch.bfloat16)
        bt = (0.02 * torch.randn(Nl, K, device=dev)).to(torch.bfloat16)
        b = bt.t()
        a_sh = symm_mem.empty(Ml, K, dtype=torch.bfloat16, device=dev)
        a_sh.copy_(a)
        symm_mem.rendezvous(a_sh)
        a_out = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        prog = torch.zeros(ws, dtype=torch.uint32, device=dev)

        def nccl_cublas():
            full = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(full, a)
            return torch.matmul(full, b)

        golden = nccl_cublas().float()
        backends = {
            "kraken_b200": lambda: fused.all_gather_matmul(a_sh, b),
            "kraken_b200_sm": lambda: fused.all_gather_matmul(a_sh, b, a_out=a_out, progress=prog, backend="sm"),
            "kraken_b200_ce": lambda: fused.all_gather_matmul(a_sh, b, a_out=a_out, progress=prog, backend="ce"),
            "nccl_cublas": nccl_cublas,
            "cublas_only": lambda: torch.matmul(a_out, b),
        }
        try:
            ta = tsm.empty(Ml, K, dtype=torch.bfloat16, device=dev)
            ta.copy_(a)
            tsm.rendezvous(ta, group=dist.group.WORLD)
            gname = dist.group.WORLD.group_name
            backends["torch_symm_mem"] = lambda: torch.ops.symm_mem.fused_all_gather_matmul(ta, [b], 0, gname)
            if ref is not None:
                t_out = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
                t_prog = torch.zeros(ws, dtype=torch.uint32, device=dev)
                backends["ref_triton"] = lambda: ref.fused.all_gather_matmul(ta, b, a_out=t_out, progress=t_prog)
        except Exception as e:
            why = why or str(e)
        for be in ("push", "ce"):
            _, c = fused.all_gather_matmul(a_sh, b, backend=be)
            torch.testing.assert_close(c.float(), golden, atol=1e-1, rtol=1e-1)
        flops = 2.0 * M * Nl * K
        nv_in = (ws - 1) * Ml * K * 2
        roof_us = max(flops / (pk["bf16_tflops"] * 1e12), nv_in / (NVLINK_GBS_MEASURED * 1e9)) * 1e6
        row = {"M": M, "K": K, "N_per_rank": Nl, "roofline_us": roof_us}
        for name, fn in backends.items():
            us, err = try_time(fn, iters=args.iters, warmup=5)
            row[name + "_us"] = us
            if us is None and rank == 0:
                print(f"[{name}] n/a: {err}", flush=True)
        if row.get("kraken_b200_us"):
            row["frac_of_roofline"] = roof_us / row["kraken_b200_us"]
            row["tflops_per_gpu"] = flops / (row["kraken_b200_us"] * 1e-6) / 1e12
        rows.append(row)
    cols = ["M", "K", "N_per_rank", "roofline_us", "frac_of_roofline", "tflops_per_gpu"] + \
        sorted({k for r in rows for k in r if k.endswith("_us") and k != "roofline_us"})
    print_table(rows, cols, f"all_gather_matmul, {ws} x B200 ({pk['source']} peaks)", f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
