"""Shared helpers for the tests: multi-process launch over gloo/NCCL and tolerances."""
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world_size, backend, init_file, fn, args, errq):
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        store = dist.FileStore(init_file, world_size)
        import datetime

        dist.init_process_group(backend, store=store, rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=120))
        torch.manual_seed(42 + rank)
        fn(rank, world_size, *args)
        if backend == "nccl":
            torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_distributed(fn, world_size, backend="gloo", args=()):
    """Runs fn(rank, world_size, *args) in `world_size` processes; raises if any rank failed."""
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    with tempfile.TemporaryDirectory() as d:
        init_file = os.path.join(d, "store")
        procs = [ctx.Process(target=_worker, args=(r, world_size, backend, init_file, fn, args, errq))
                 for r in range(world_size)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=300)
        failed = []
        for r, p in enumerate(procs):
            if p.is_alive():
                p.kill()          # the exact child this test started
                failed.append((r, "timed out"))
            elif p.exitcode != 0:
                failed.append((r, f"exit code {p.exitcode}"))
        msgs = []
        while not errq.empty():
            msgs.append(errq.get())
        if failed or msgs:
            raise AssertionError(f"ranks failed: {failed}\n" + "\n".join(f"[rank {r}] {m}" for r, m in msgs))
