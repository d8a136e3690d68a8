"""Per-tile device timeline of the fused reduce-scatter GEMM (a profiling aid; the reference has
only host-side timers and the torch profiler, kraken/_logging/benchmarking.py:37-163).

While a ``TileTrace`` is active, one thread per role of every CTA stamps ``%globaltimer`` at fixed
points of each tile it handles: the MMA issuer (accumulator free / first operands landed / last MMA
issued), the epilogue (accumulator complete / tile stored / completion hook done) and the reducer
warps (wait begins / wait over / tile reduced). ``summary()`` turns the stamps into the numbers
that matter when the kernel is slower than its roofline: how long the tensor pipe sat between
tiles, how long epilogues and hooks took, how long reducers waited for peers, and when each role
finished relative to the first stamp of the launch.

    with TileTrace() as tr:
        fused.gemm_reduce_scatter(a, b)
    print(tr.summary())
"""
from __future__ import annotations

import torch

from ..ops import lib as _lib

ROLES, TILES, FIELDS = 3, 64, 4


class TileTrace:
    def __init__(self, max_ctas: int = 160, device=None):
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.buf = torch.zeros(max_ctas * ROLES * TILES * FIELDS, dtype=torch.int64, device=self.device)
        self.max_ctas = max_ctas

    def __enter__(self):
        self.buf.zero_()
        _lib.check(_lib.lib().kr_gemm_rs_set_trace(self.buf.data_ptr(), self.buf.numel()))
        return self

    def __exit__(self, *exc):
        torch.cuda.synchronize(self.device)
        _lib.check(_lib.lib().kr_gemm_rs_set_trace(None, 0))
        return False

    def stamps(self) -> torch.Tensor:
        """[CTA, role, tile slot, field] nanoseconds (0 = not stamped)."""
        return self.buf.view(self.max_ctas, ROLES, TILES, FIELDS).cpu()

    def summary(self) -> dict:
        t = self.stamps().double()
        valid = t > 0
        if not bool(valid.any()):
            return {}
        t0 = float(t[valid].min())
        us = lambda x: round(float(x) / 1000.0, 1)      # noqa: E731
        out = {}
        mma, epi, red = t[:, 0], t[:, 1], t[:, 2]
        m_ok = (mma[..., 0] > 0) & (mma[..., 2] > 0)
        if bool(m_ok.any()):
            busy = (mma[..., 2] - mma[..., 0])[m_ok]
            out["mma_tiles"] = int(m_ok.sum())
            out["mma_issue_us_mean"] = us(busy.mean())
            wait_ops = (mma[..., 1] - mma[..., 0])[m_ok]
            out["mma_wait_first_stage_us_mean"] = us(wait_ops.mean())
            out["mma_wait_first_stage_us_max"] = us(wait_ops.max())
            # gap between the end of one tile's issue and the next tile's accumulator being free
            nxt = m_ok[:, 1:] & m_ok[:, :-1]
            if bool(nxt.any()):
                gap = (mma[:, 1:, 0] - mma[:, :-1, 2])[nxt]
                out["mma_gap_between_tiles_us_mean"] = us(gap.mean())
                out["mma_gap_between_tiles_us_max"] = us(gap.max())
            out["mma_first_start_us"] = us(mma[..., 0][m_ok].min() - t0)
            out["mma_last_issue_us"] = us(mma[..., 2][m_ok].max() - t0)
        e_ok = (epi[..., 0] > 0) & (epi[..., 2] > 0)
        if bool(e_ok.any()):
            out["epilogue_us_mean"] = us((epi[..., 1] - epi[..., 0])[e_ok].mean())
            out["epilogue_us_max"] = us((epi[..., 1] - epi[..., 0])[e_ok].max())
            out["hook_us_mean"] = us((epi[..., 2] - epi[..., 1])[e_ok].mean())
            out["hook_us_max"] = us((epi[..., 2] - epi[..., 1])[e_ok].max())
            out["epilogue_last_done_us"] = us(epi[..., 2][e_ok].max() - t0)
        r_ok = (red[..., 0] > 0) & (red[..., 2] > 0)
        if bool(r_ok.any()):
            out["reduce_units"] = int(r_ok.sum())
            out["reduce_wait_us_mean"] = us((red[..., 1] - red[..., 0])[r_ok].mean())
            out["reduce_work_us_mean"] = us((red[..., 2] - red[..., 1])[r_ok].mean())
            out["reduce_work_us_max"] = us((red[..., 2] - red[..., 1])[r_ok].max())
            out["reduce_last_done_us"] = us(red[..., 2][r_ok].max() - t0)
            # how far behind the last MMA the last reduction ends: the kernel's exposed tail
            if "mma_last_issue_us" in out:
                out["tail_after_last_mma_us"] = round(out["reduce_last_done_us"] - out["mma_last_issue_us"], 1)
        return out
