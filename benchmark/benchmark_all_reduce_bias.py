"""All-reduce + bias (reference: benchmark/benchmark_all_reduce_bias.py): x bf16 [b, 5120],
b = 1..512; one-shot and two-shot fused kernels against NCCL all_reduce + add, torch's
one_shot_all_reduce_copy_out + add, and the reference's Triton kernels. Flags follow the reference
(``--max_b``, ``--max_t``, ``--d_size``: input [b, t, d] for powers of two up to the maxima); a line
chart of all columns is written next to the tables, as the reference's script does."""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import finish, load_reference, plot_rows, print_table, setup, try_time


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-b", "--max_b", dest="max_b", type=int, default=512)
    ap.add_argument("--max-t", "--max_t", dest="max_t", type=int, default=1)
    ap.add_argument("--d-size", "--d_size", dest="d_size", type=int, default=5120)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--save-path", default="results/bench_all_reduce_bias")
    args = ap.parse_args()
    rank, ws, dev = setup()
    from kraken_b200 import fused
    from kraken_b200.parallel import symm_mem
    import torch.distributed._symmetric_memory as tsm

    ref, why = load_reference()
    D = args.d_size
    pad = symm_mem.empty(args.max_b * args.max_t * D, dtype=torch.bfloat16, device=dev)
    symm_mem.rendezvous(pad)
    tpad = None
    try:
        tpad = tsm.empty(args.max_b * args.max_t * D, dtype=torch.bfloat16, device=dev)
        tsm.rendezvous(tpad, group=dist.group.WORLD)
    except Exception as e:
        why = why or str(e)
    rows = []
    bt_sizes = [(b, t) for b in (2 ** k for k in range(args.max_b.bit_length()) if 2 ** k <= args.max_b)
                for t in (2 ** k for k in range(args.max_t.bit_length()) if 2 ** k <= args.max_t)]
    for b, t in bt_sizes:
        x = torch.randn(b, t, D, device=dev).to(torch.bfloat16)
        g = torch.Generator().manual_seed(3)
        bias = torch.randn(b, t, D, generator=g).to(torch.bfloat16).to(dev)
        out = torch.empty_like(x)
        gold = x.float().clone()
        dist.all_reduce(gold)
        gold += bias.float()

        def nccl():
            y = x.clone()
            dist.all_reduce(y)
            return y + bias

        backends = {
            "one_shot_bias": lambda: fused.one_shot_all_reduce_bias(pad, x, bias, out),
            "one_shot_pull_bias": lambda: fused.one_shot_all_reduce_bias(pad, x, bias, out, algo="pull"),
            "two_shot_bias": lambda: fused.two_shot_all_reduce_bias(pad, x, bias, out),
            "nccl_add": nccl,
        }
        if tpad is not None and ref is not None:
            backends["ref_one_shot_bias"] = lambda: ref.fused.one_shot_all_reduce_bias(tpad, x, bias, out)
            backends["ref_two_shot_bias"] = lambda: ref.fused.two_shot_all_reduce_bias(tpad, x, bias, out)
        fused.two_shot_all_reduce_bias(pad, x, bias, out)
        torch.testing.assert_close(out.float(), gold, atol=1e-1, rtol=1e-1)
        row = {"b": b, "t": t, "bytes": b * t * D * 2}
        for name, fn in backends.items():
            us, err = try_time(fn, iters=args.iters, warmup=20)
            row[name + "_us"] = us
        rows.append(row)
    cols = ["b", "t", "bytes"] + sorted({k for r in rows for k in r if k.endswith("_us")})
    print_table(rows, cols, f"all_reduce + bias, d={D}, {ws} x B200", f"{args.save_path}_ws{ws}")
    plot_rows(rows, ["b", "t"], f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
