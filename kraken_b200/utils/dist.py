"""Process-group bootstrap from the environment torchrun sets (RANK, LOCAL_RANK, WORLD_SIZE,
MASTER_ADDR, MASTER_PORT). NCCL is used for rendezvous control traffic and baselines only."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def init_from_env(backend: str | None = None, timeout_s: int = 600) -> tuple[int, int, int]:
    """Returns (rank, local_rank, world_size); initialises the default group when WORLD_SIZE > 1."""
    rank = int(os.environ.get("RANK", 0))
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        torch.cuda.set_device(local_rank % max(1, torch.cuda.device_count()))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, local_rank, world
