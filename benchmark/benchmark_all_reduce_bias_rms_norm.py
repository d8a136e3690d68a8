"""All-reduce + bias + RMSNorm (reference: benchmark/benchmark_all_reduce_bias_rms_norm.py):
x bf16 [b, d]; the fused one-shot and two-shot kernels against (a) NCCL all_reduce + add +
rms_norm kernel, (b) this library's all-reduce-bias kernel followed by its rms_norm kernel
(unfused), (c) the reference's Triton kernels."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import finish, load_reference, plot_rows, print_table, setup, try_time


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-b", "--max_b", dest="max_b", type=int, default=512)
    ap.add_argument("--d-size", "--d_size", dest="d_size", type=int, default=5120)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--save-path", default="results/bench_all_reduce_bias_rms_norm")
    args = ap.parse_args()
    rank, ws, dev = setup()
    from kraken_b200 import fused
    from kraken_b200.parallel import symm_mem
    import torch.distributed._symmetric_memory as tsm

    ref, why = load_reference()
    D = args.d_size
    pad = symm_mem.empty(args.max_b * D, dtype=torch.bfloat16, device=dev)
    symm_mem.rendezvous(pad)
    tpad = None
    try:
        tpad = tsm.empty(args.max_b * D, dtype=torch.bfloat16, device=dev)
        tsm.rendezvous(tpad, group=dist.group.WORLD)
    except Exception as e:
        why = why or str(e)
    g = torch.Generator().manual_seed(3)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).to(dev)
    rows = []
    b = 1
    while b <= args.max_b:
        x = torch.randn(b, D, device=dev).to(torch.bfloat16)
        bias = torch.randn(D, generator=g).to(torch.bfloat16).to(dev)
        full_bias = bias.expand(b, D).contiguous()
        y = torch.empty_like(x)
        tmp = torch.empty_like(x)
        s = x.float().clone()
        dist.all_reduce(s)
        s += bias.float()
        gold = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()

        def nccl_unfused():
            t = x.clone()
            dist.all_reduce(t)
            return fused.rms_norm(t + bias, w, 1e-5)

        def ours_unfused():
            fused.two_shot_all_reduce_bias(pad, x, bias, tmp)
            return fused.rms_norm(tmp, w, 1e-5)

        backends = {
            "one_shot_fused": lambda: fused.one_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5),
            "one_shot_pull_fused": lambda: fused.one_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5, algo="pull"),
            "two_shot_fused": lambda: fused.two_shot_all_reduce_bias_rms_norm(pad, x, bias, w, y, 1e-5),
            "ours_unfused": ours_unfused,
            "nccl_unfused": nccl_unfused,
        }
        if tpad is not None and ref is not None and b * ws * 4 <= 9216:
            # the reference's one-shot kernel launches one block per row: stay inside its signal pad
            backends["ref_one_shot_fused"] = lambda: ref.fused.one_shot_all_reduce_bias_rms_norm(tpad, x, full_bias, w, y, 1e-5)
            backends["ref_two_shot_fused"] = lambda: ref.fused.two_shot_all_reduce_bias_rms_norm(tpad, x, full_bias, w, y, 1e-5)
        for fn in (fused.two_shot_all_reduce_bias_rms_norm, fused.one_shot_all_reduce_bias_rms_norm):
            fn(pad, x, bias, w, y, 1e-5)
            torch.testing.assert_close(y.float(), gold, atol=1e-1, rtol=1e-1)
        row = {"b": b, "bytes": b * D * 2}
        for name, fn in backends.items():
            us, err = try_time(fn, iters=args.iters, warmup=20)
            row[name + "_us"] = us
        rows.append(row)
        b *= 2
    cols = ["b", "bytes"] + sorted({k for r in rows for k in r if k.endswith("_us")})
    print_table(rows, cols, f"all_reduce + bias + rms_norm, d={D}, {ws} x B200", f"{args.save_path}_ws{ws}")
    plot_rows(rows, ["b"], f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
