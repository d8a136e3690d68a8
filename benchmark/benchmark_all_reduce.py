"""All-reduce sweep (reference: benchmark/benchmark_all_reduce.py): bf16 tensors from 4 KB to
256 MB, one-shot vs two-shot vs NVLS multimem (this library) against NCCL, torch's symmetric-memory
ops and the reference's Triton kernels. Reports device-timed median microseconds (max over ranks)
and bus bandwidth 2(n-1)/n * S / t.

    torchrun --nnodes 1 --nproc-per-node N --master-addr 127.0.0.1 benchmark/benchmark_all_reduce.py

The reference's flags are accepted: ``--size`` (tensor lengths in elements; overrides the byte sweep),
``-dtype`` (bfloat16 only), ``--backend`` (this script's column names, or the reference's
nccl / triton_1shot / triton_2shot / dist_multimem / dist_1shot / dist_2shot), ``--save-path``.
"""
from __future__ import annotations

import argparse

import torch
import torch.distributed as dist

from common import (bus_bandwidth_gbs, check_dtype, finish, load_reference, plot_rows, print_table, setup, try_time,
                    NVLINK_GBS_MEASURED)

_REF_NAMES = {"triton_1shot": "ref_triton_one_shot", "triton_2shot": "ref_triton_two_shot", "dist_multimem": "torch_multimem",
              "dist_1shot": "torch_one_shot", "dist_2shot": "torch_two_shot"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=256 << 20)
    ap.add_argument("--step", type=int, default=2, help="factor between consecutive sizes")
    ap.add_argument("--size", type=int, nargs="+", default=None, help="tensor lengths in elements (reference flag)")
    ap.add_argument("-dtype", default="bfloat16")
    ap.add_argument("--backend", nargs="*", default=None)
    ap.add_argument("--iters", type=int, default=25)
    ap.add_argument("--save-path", default="results/bench_all_reduce")
    args = ap.parse_args()
    check_dtype(args.dtype)
    if args.backend:
        args.backend = [_REF_NAMES.get(b, b) for b in args.backend]
    rank, ws, dev = setup()
    from kraken_b200 import comm
    from kraken_b200.parallel import symm_mem
    import torch.distributed._symmetric_memory as tsm

    ref, why = load_reference()
    rows = []
    if args.size:
        sizes = [2 * n for n in args.size]
    else:
        sizes, nb_ = [], args.min_bytes
        while nb_ <= args.max_bytes:
            sizes.append(nb_)
            nb_ *= max(2, args.step)
    for nbytes in sizes:
        numel = nbytes // 2
        x = torch.randn(numel, device=dev).to(torch.bfloat16)
        xs = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
        xs.copy_(x)
        symm_mem.rendezvous(xs)
        xm = symm_mem.empty(numel, dtype=torch.bfloat16, device=dev)
        xm.copy_(x)
        symm_mem.rendezvous(xm)
        golden = x.float().clone()
        dist.all_reduce(golden)
        backends = {
            "one_shot": lambda: comm.one_shot_all_reduce(xs),
            "one_shot_pull": lambda: comm.one_shot_all_reduce(xs, algo="pull"),
            "two_shot": lambda: comm.two_shot_all_reduce(x),
            "two_shot_p2p": lambda: comm.two_shot_all_reduce(x, nvls=False),
            "multimem": lambda: comm.multimem_all_reduce(xm),
            "nccl": lambda: dist.all_reduce(x.clone()),
        }
        try:
            tx = tsm.empty(numel, dtype=torch.bfloat16, device=dev)
            tx.copy_(x)
            tsm.rendezvous(tx, group=dist.group.WORLD)
            gname = dist.group.WORLD.group_name
            backends["torch_multimem"] = lambda: torch.ops.symm_mem.multimem_all_reduce_(tx, "sum", gname)
            backends["torch_one_shot"] = lambda: torch.ops.symm_mem.one_shot_all_reduce(tx, "sum", gname)
            backends["torch_two_shot"] = lambda: torch.ops.symm_mem.two_shot_all_reduce_(tx, "sum", gname)
            if ref is not None:
                backends["ref_triton_one_shot"] = lambda: ref.comm.one_shot_all_reduce(tx)
                backends["ref_triton_two_shot"] = lambda: ref.comm.two_shot_all_reduce(x)
        except Exception as e:   # torch symmetric memory unavailable on this box
            why = why or str(e)
        if nbytes > (32 << 20):
            backends.pop("one_shot", None)          # pull traffic (n-1)*S: pointless at this size
            backends.pop("one_shot_pull", None)
            backends.pop("torch_one_shot", None)
            backends.pop("ref_triton_one_shot", None)
        # correctness gate before timing, as the reference's benchmark does
        torch.testing.assert_close(comm.two_shot_all_reduce(x).float(), golden, atol=1e-1, rtol=1e-1)
        if "one_shot" in backends:
            torch.testing.assert_close(comm.one_shot_all_reduce(xs).float(), golden, atol=1e-1, rtol=1e-1)
        row = {"bytes": nbytes}
        for name, fn in backends.items():
            if args.backend and name not in args.backend:
                continue
            if name == "multimem":
                xm.copy_(x)
            us, err = try_time(fn, iters=args.iters)
            row[name + "_us"] = us
            if us:
                row[name + "_busGBs"] = bus_bandwidth_gbs("all_reduce", nbytes, ws, us)
        best = min((row[k] for k in ("one_shot_us", "two_shot_us", "multimem_us") if row.get(k)), default=None)
        if best:
            row["best_busGBs"] = bus_bandwidth_gbs("all_reduce", nbytes, ws, best)
            row["frac_of_link"] = row["best_busGBs"] / NVLINK_GBS_MEASURED
        rows.append(row)
    cols = ["bytes"] + sorted({k for r in rows for k in r if k != "bytes"})
    print_table(rows, cols, f"all_reduce sweep, {ws} x B200 (us = median, max over ranks)", f"{args.save_path}_ws{ws}")
    plot_rows(rows, ["bytes"], f"{args.save_path}_ws{ws}")
    finish()


if __name__ == "__main__":
    main()
