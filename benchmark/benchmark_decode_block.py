"""Decode-shaped chain (no reference script; the shapes come from the tensor-parallel decode use
case the reference's ops target): gemm_one_shot_all_reduce_fused with A bf16 [M, 8192/ws],
B bf16 [8192/ws, 8192], M in {1, 16, 64, 256}, then all-reduce + bias + RMSNorm on [M, 8192] (the
one-shot form up to M = 64, the two-shot form beyond).
Baselines: cuBLAS + NCCL all_reduce (fp32), and NCCL all_reduce + add + rms_norm."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import finish, load_reference, peaks, print_table, setup, try_time


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, nargs="*", default=[1, 16, 64, 256])
    ap.add_argument("--K", type=int, default=8192, help="global K; each rank holds K / world_size")
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--save-path", default="results/bench_decode_block")
    ap.add_argument("--variants", action="store_true",
                    help="also time every exchange (push / one_shot / two_shot) with 1 and 2 K splits")
    args = ap.parse_args()
    rank, ws, dev = setup()
    from kraken_b200 import fused
    from kraken_b200.parallel import symm_mem

    ref, why = load_reference()
    pk = peaks()
    Kl, N = args.K // ws, args.N
    bt = (0.02 * torch.randn(N, Kl, device=dev)).to(torch.bfloat16)
    b = bt.t()
    g = torch.Generator().manual_seed(3)
    bias = torch.randn(N, generator=g).to(torch.bfloat16).to(dev)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16).to(dev)
    pad = symm_mem.empty(max(args.M) * N, dtype=torch.bfloat16, device=dev)
    symm_mem.rendezvous(pad)
    rows = []
    for M in args.M:
        a = torch.randn(M, Kl, device=dev).to(torch.bfloat16)
        x = torch.randn(M, N, device=dev).to(torch.bfloat16)
        y = torch.empty_like(x)

        def cublas_nccl():
            c = torch.matmul(a, b).float()
            dist.all_reduce(c)
            return c

        def nccl_norm():
            t = x.clone()
            dist.all_reduce(t)
            return fused.rms_norm(t + bias, w, 1e-5)

        gold = cublas_nccl()
        o = fused.gemm_one_shot_all_reduce_fused(a, b)
        torch.testing.assert_close(o, gold, atol=5e-2, rtol=5e-2)
        backends = {
            "gemm_ar_fused": lambda: fused.gemm_one_shot_all_reduce_fused(a, b),
            "cublas_nccl": cublas_nccl,
            "ar_bias_norm_two_shot": lambda: fused.two_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5),
            "ar_bias_norm_one_shot": lambda: fused.one_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5),
            "nccl_add_norm": nccl_norm,
        }
        if args.variants:
            for algo in ("push", "push_two_shot", "one_shot", "two_shot"):
                for ks in (1, 2):
                    if algo == "one_shot" and ks == 2:
                        continue
                    backends[f"gemm_ar_{algo}_k{ks}"] = (
                        lambda algo=algo, ks=ks: fused.gemm_one_shot_all_reduce_fused(a, b, algo=algo, k_splits=ks))

        def chain():
            # the decode step this benchmark is about: GEMM + all-reduce, then the next layer's
            # all-reduce + bias + RMSNorm, back to back on one stream
            fused.gemm_one_shot_all_reduce_fused(a, b)
            if M <= 64:
                fused.one_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5)
            else:
                fused.two_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5)

        backends["chain_gemm_ar_then_ar_bias_norm"] = chain
        if ref is not None and ((M + 63) // 64) * (N // 64) * ws <= 2304:
            # same bf16 operands as this library's column; the fp32 column is how the reference's own
            # test feeds it (test/test_gemm_allreduce.py:57-58) and moves twice the bytes
            bc = b.contiguous()
            backends["ref_gemm_ar"] = lambda: ref.fused.gemm_one_shot_all_reduce_fused(a, bc)
            af, bf = a.float(), b.float().contiguous()
            backends["ref_gemm_ar_fp32"] = lambda: ref.fused.gemm_one_shot_all_reduce_fused(af, bf)
        row = {"M": M, "K_per_rank": Kl, "N": N,
               "weight_read_us": Kl * N * 2 / (pk["hbm_gbs"] * 1e9) * 1e6}
        for name, fn in backends.items():
            us, err = try_time(fn, iters=args.iters, warmup=20)
            row[name + "_us"] = us
            if us is None and rank == 0:
                print(f"[{name}] n/a: {err}", flush=True)
        rows.append(row)
    cols = ["M", "K_per_rank", "N", "weight_read_us"] + sorted({k for r in rows for k in r if k.endswith("_us") and k != "weight_read_us"})
    print_table(rows, cols, f"decode block, {ws} x B200", f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
