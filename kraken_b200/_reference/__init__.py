"""Pure-PyTorch restatement of every op: fp32 math plus ``torch.distributed`` collectives.

Two jobs: (1) the CPU path — ops called with CPU tensors under a gloo group run this code, which is
how the multi-process plumbing is tested without a GPU; (2) the oracle and the "NCCL + cuBLAS"
baseline on GPUs (same functions with CUDA tensors over an NCCL group). The reference has no CPU
path; its tests use NCCL collectives as goldens (test/test_allreduce.py:61-65,
test/test_gemm_reduce_scatter.py:106) and these functions state the same math.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel.symm_mem import GroupInfo, resolve_group


def _pg(info: GroupInfo):
    return info.pg


def all_reduce_f32(x: torch.Tensor, info: GroupInfo) -> torch.Tensor:
    y = x.detach().to(torch.float32).clone()
    if info.world_size > 1:
        dist.all_reduce(y, group=_pg(info))
    return y


def all_reduce(x: torch.Tensor, group=None, out_dtype=None) -> torch.Tensor:
    info = resolve_group(group)
    return all_reduce_f32(x, info).to(out_dtype or x.dtype)


def reduce_scatter(x: torch.Tensor, group=None) -> torch.Tensor:
    """x: [ws * n, ...] on every rank -> rank r gets sum over ranks of slab r."""
    info = resolve_group(group)
    full = all_reduce_f32(x, info)
    n = x.shape[0] // info.world_size
    return full[info.rank * n:(info.rank + 1) * n].to(x.dtype).contiguous()


def all_gather(x: torch.Tensor, group=None) -> torch.Tensor:
    info = resolve_group(group)
    if info.world_size == 1:
        return x.clone()
    outs = [torch.empty_like(x) for _ in range(info.world_size)]
    dist.all_gather(outs, x.contiguous(), group=_pg(info))
    return torch.cat(outs, dim=0)


def _bias_term(bias: torch.Tensor | None, like: torch.Tensor) -> torch.Tensor | float:
    if bias is None:
        return 0.0
    b = bias.to(torch.float32)
    if b.numel() == like.numel():
        return b.reshape(like.shape)
    return b            # row-broadcast [D]


def all_reduce_bias(x: torch.Tensor, bias: torch.Tensor | None, group=None) -> torch.Tensor:
    info = resolve_group(group)
    y = all_reduce_f32(x, info)
    return (y + _bias_term(bias, y)).to(x.dtype)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    xf = x.to(torch.float32)
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * w.to(torch.float32)).to(x.dtype)


def all_reduce_bias_rms_norm(x: torch.Tensor, bias: torch.Tensor | None, w: torch.Tensor, eps: float = 1e-5,
                             group=None, round_sum_to_bf16: bool = False) -> torch.Tensor:
    info = resolve_group(group)
    y = all_reduce_f32(x, info)
    y = y + _bias_term(bias, y)
    if round_sum_to_bf16:
        y = y.to(x.dtype).to(torch.float32)
    inv = torch.rsqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (y * inv * w.to(torch.float32)).to(x.dtype)


def matmul_f32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return a.to(torch.float32) @ b.to(torch.float32)


def all_gather_matmul(a_shard: torch.Tensor, b: torch.Tensor, group=None):
    a = all_gather(a_shard, group)
    return a, matmul_f32(a, b).to(a_shard.dtype)


def gemm_all_reduce(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    info = resolve_group(group)
    return all_reduce_f32(matmul_f32(a, b), info)


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, group=None) -> torch.Tensor:
    info = resolve_group(group)
    full = all_reduce_f32(matmul_f32(a, b), info)
    n = a.shape[0] // info.world_size
    return full[info.rank * n:(info.rank + 1) * n].to(a.dtype).contiguous()
