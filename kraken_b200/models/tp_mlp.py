"""Tensor-parallel transformer MLP block built from the library's fused ops — the end-to-end slice
the reference's ops exist for (its README calls itself a cookbook for tensor-parallel inference;
the ops are kraken/fused/all_gather_matmul.py, gemm_reduce_scatter_fused.py,
gemm_one_shot_all_reduce_fused.py and two_shot_all_reduce_bias_rms_norm.py).

Prefill (sequence-parallel activations, [M/ws, H] per rank):
    h = all_gather_matmul(x_shard, W_up[:, shard])        column-parallel up projection
    h = gelu(h)
    y_shard = gemm_reduce_scatter(h, W_down[shard, :])    row-parallel down projection
Decode (replicated activations, [M, H] per rank, M small):
    p = gemm_one_shot_all_reduce(h_local, W_down[shard, :])     fp32 [M, H]
    y = two_shot_all_reduce_bias_rms_norm(...)  is the next layer's input norm; here the already
        reduced p only needs bias + RMSNorm, so decode() applies them with the fused norm kernel
        on one rank's data (world size 1 semantics of the same kernel).
Weights are random-initialised bf16 (no checkpoints are involved anywhere in this library).
"""
from __future__ import annotations

import torch

from .. import fused
from ..parallel import symm_mem


class TPMLP:
    def __init__(self, hidden: int, ffn: int, group=None, device=None, dtype=torch.bfloat16, seed: int = 0):
        info = symm_mem.resolve_group(group)
        self.group = group
        self.rank, self.ws = info.rank, info.world_size
        if ffn % self.ws:
            raise ValueError("ffn size must divide by the world size")
        self.hidden, self.ffn = hidden, ffn
        self.device = torch.device(device) if device is not None else (
            torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
        g = torch.Generator(device="cpu").manual_seed(seed + 1000 * self.rank)
        f_local = ffn // self.ws
        # stored K-major for the tensor cores: w_up_t [F/ws, H], w_down_t [H, F/ws]
        self.w_up_t = (torch.randn(f_local, hidden, generator=g) * 0.02).to(dtype).to(self.device)
        self.w_down_t = (torch.randn(hidden, f_local, generator=g) * 0.02).to(dtype).to(self.device)
        g2 = torch.Generator(device="cpu").manual_seed(seed)        # replicated parameters
        self.bias = torch.randn(hidden, generator=g2).to(dtype).to(self.device)
        self.norm_w = (1.0 + 0.1 * torch.randn(hidden, generator=g2)).to(dtype).to(self.device)
        self._x_symm = None
        self._norm_buf = None

    # -- prefill -----------------------------------------------------------------------------------
    def stage_input(self, x_shard: torch.Tensor) -> torch.Tensor:
        """Copies this rank's activation shard into symmetric memory (allocated once per shape)."""
        if self._x_symm is None or self._x_symm.shape != x_shard.shape:
            self._x_symm = symm_mem.empty(*x_shard.shape, dtype=x_shard.dtype, device=x_shard.device)
            symm_mem.rendezvous(self._x_symm, self.group)
        self._x_symm.copy_(x_shard)
        return self._x_symm

    def prefill(self, x_symm_shard: torch.Tensor) -> torch.Tensor:
        """x_symm_shard: [M/ws, H] in symmetric memory -> [M/ws, H]."""
        _, h = fused.all_gather_matmul(x_symm_shard, self.w_up_t.t(), group=self.group)
        h = torch.nn.functional.gelu(h, approximate="tanh")
        return fused.gemm_reduce_scatter(h, self.w_down_t.t(), group=self.group)

    # -- decode ------------------------------------------------------------------------------------
    def decode(self, h_local: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        """h_local: [M, F/ws] (this rank's slice of the MLP activations) -> normalised [M, H]."""
        p = fused.gemm_one_shot_all_reduce(h_local, self.w_down_t.t(), group=self.group)     # fp32, replicated
        x = p.to(torch.bfloat16)
        if x.device.type != "cuda":
            from .. import _reference as ref

            return ref.rms_norm((x.float() + self.bias.float()).to(x.dtype), self.norm_w, eps)
        return fused.rms_norm((x.float() + self.bias.float()).to(x.dtype), self.norm_w, eps)

    def decode_partial_norm(self, partial: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
        """The reference's decode epilogue: `partial` [M, H] bf16 is this rank's un-reduced partial
        sum; returns rms_norm(all_reduce(partial) + bias) * w via the fused one-shot or two-shot kernel."""
        y = torch.empty_like(partial)
        if partial.device.type == "cuda":
            if self._norm_buf is None or self._norm_buf.numel() < partial.numel():
                self._norm_buf = symm_mem.empty(partial.numel(), dtype=partial.dtype, device=partial.device)
                symm_mem.rendezvous(self._norm_buf, self.group)
            buf = self._norm_buf
        else:
            buf = torch.empty_like(partial)
        # Measured: the one-shot (push) form wins while the rows fit its workspace slots (b <= 64 of 5120
        # at 8 GPUs: 22.7 us against 32.9 us; every b up to 512 at 2 GPUs), the two-shot form beyond.
        from ..comm.all_reduce import push_limit_bytes

        ws = symm_mem.resolve_group(self.group).world_size if partial.device.type == "cuda" else 1
        if partial.numel() * partial.element_size() <= push_limit_bytes(ws):
            fused.one_shot_all_reduce_bias_rms_norm(buf, partial, self.bias, self.norm_w, y, eps, group=self.group)
        else:
            fused.two_shot_all_reduce_bias_rms_norm(buf, partial, self.bias, self.norm_w, y, eps, group=self.group)
        return y
