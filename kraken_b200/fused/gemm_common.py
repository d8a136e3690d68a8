"""Operand preparation shared by the fused GEMM ops.

The tcgen05 kernels take both operands K-major: ``a`` as [M, K] with K contiguous and ``b`` as its
transpose ``bt`` [N, K] with K contiguous (the layout of an ``nn.Linear`` weight, and what the
reference's all-gather matmul insists on: kraken/fused/all_gather_matmul.py:158-160). A ``b`` that is
row-major [K, N] is transposed once and cached per (storage, version) — weights are static in
inference, whereas the reference's copy-engine variant re-transposes on every call
(kraken/fused/gemm_reduce_scatter_ce_persistent.py:192). bf16 operands run on the bf16 tensor-core
path; when BOTH operands are fp32 the plain GEMM and the GEMM all-reduce multiply them as tf32
(``keep_fp32=True`` below), as ``tl.dot`` does for the reference's fp32 tests; every other
combination is cast to bf16. Accumulation is always fp32.
"""
from __future__ import annotations

import torch

_bt_cache: dict[tuple, tuple] = {}


def use_tf32(a: torch.Tensor, b: torch.Tensor) -> bool:
    """fp32 x fp32 (and K rows of whole 16-byte units) takes the tf32 kernels."""
    return a.dtype == torch.float32 and b.dtype == torch.float32 and a.shape[-1] % 4 == 0


def as_k_major_a(a: torch.Tensor, keep_fp32: bool = False) -> tuple[torch.Tensor, int]:
    """Returns (tensor, row stride in elements) with K contiguous and 16-byte aligned rows; bf16,
    or fp32 when keep_fp32 and `a` is fp32."""
    want = torch.float32 if (keep_fp32 and a.dtype == torch.float32) else torch.bfloat16
    if a.dtype != want:
        a = a.to(want)
    if a.dim() != 2:
        raise ValueError("GEMM operands must be 2-D")
    unit = 16 // a.element_size()
    if a.stride(1) != 1 or a.stride(0) % unit or a.data_ptr() % 16 or a.stride(0) < a.shape[1]:
        a = a.contiguous()
    return a, a.stride(0)


def as_k_major_bt(b: torch.Tensor, keep_fp32: bool = False) -> tuple[torch.Tensor, int]:
    """b is [K, N]; returns (bt [N, K] with K contiguous, row stride in elements); bf16, or fp32
    when keep_fp32 and `b` is fp32."""
    if b.dim() != 2:
        raise ValueError("GEMM operands must be 2-D")
    want = torch.float32 if (keep_fp32 and b.dtype == torch.float32) else torch.bfloat16
    unit = 16 // torch.empty((), dtype=want).element_size()
    if b.dtype == want and b.stride(0) == 1 and b.stride(1) % unit == 0 and b.stride(1) >= b.shape[0] \
            and b.data_ptr() % 16 == 0:
        return b.t(), b.stride(1)
    key = (b.data_ptr(), tuple(b.shape), tuple(b.stride()), b.dtype, b._version, want)
    hit = _bt_cache.get(key)
    if hit is not None:
        return hit[0], hit[0].stride(0)
    bt = b.t().to(want).contiguous()
    if len(_bt_cache) > 64:
        _bt_cache.clear()
    _bt_cache[key] = (bt, b)     # keep `b` alive so the key's data_ptr cannot be recycled
    return bt, bt.stride(0)
