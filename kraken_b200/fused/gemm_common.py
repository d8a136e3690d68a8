"""Operand preparation shared by the fused GEMM ops.

The tcgen05 kernels take both operands K-major: ``a`` as [M, K] with K contiguous and ``b`` as its
transpose ``bt`` [N, K] with K contiguous (the layout of an ``nn.Linear`` weight, and what the
reference's all-gather matmul insists on: kraken/fused/all_gather_matmul.py:158-160). A ``b`` that is
row-major [K, N] is transposed once and cached per (storage, version) — weights are static in
inference, whereas the reference's copy-engine variant re-transposes on every call
(kraken/fused/gemm_reduce_scatter_ce_persistent.py:192). Non-bf16 inputs are cast to bf16: the
tensor-core path of this library is bf16 with fp32 accumulation.
"""
from __future__ import annotations

import torch

_bt_cache: dict[tuple, tuple] = {}


def as_k_major_a(a: torch.Tensor) -> tuple[torch.Tensor, int]:
    """Returns (tensor, row stride in elements) with K contiguous, bf16, 16-byte aligned rows."""
    if a.dtype != torch.bfloat16:
        a = a.to(torch.bfloat16)
    if a.dim() != 2:
        raise ValueError("GEMM operands must be 2-D")
    if a.stride(1) != 1 or a.stride(0) % 8 or a.data_ptr() % 16 or a.stride(0) < a.shape[1]:
        a = a.contiguous()
    return a, a.stride(0)


def as_k_major_bt(b: torch.Tensor) -> tuple[torch.Tensor, int]:
    """b is [K, N]; returns (bt [N, K] with K contiguous, row stride in elements)."""
    if b.dim() != 2:
        raise ValueError("GEMM operands must be 2-D")
    if b.dtype == torch.bfloat16 and b.stride(0) == 1 and b.stride(1) % 8 == 0 and b.stride(1) >= b.shape[0] \
            and b.data_ptr() % 16 == 0:
        return b.t(), b.stride(1)
    key = (b.data_ptr(), tuple(b.shape), tuple(b.stride()), b.dtype, b._version)
    hit = _bt_cache.get(key)
    if hit is not None:
        return hit[0], hit[0].stride(0)
    bt = b.t().to(torch.bfloat16).contiguous()
    if len(_bt_cache) > 64:
        _bt_cache.clear()
    _bt_cache[key] = (bt, b)     # keep `b` alive so the key's data_ptr cannot be recycled
    return bt, bt.stride(0)
