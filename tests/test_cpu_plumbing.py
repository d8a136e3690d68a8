"""CPU / gloo tests (no GPU): API surface, the pure-PyTorch backend over a 2-rank gloo group, the
native library's loadability and its argument checking."""
import inspect

import pytest
import torch

import kraken_b200
from kraken_b200 import _reference as ref
from kraken_b200 import comm, config, fused
from kraken_b200.ops import lib as klib
from helpers import run_distributed


def test_public_api_surface():
    for name in ["one_shot_all_reduce", "two_shot_all_reduce", "multimem_all_reduce", "all_gather_w_progress",
                 "reduce_scatter", "_copy_engine_all_gather_w_progress"]:
        assert callable(getattr(comm, name)), name
    for name in ["all_gather_matmul", "gemm_one_shot_all_reduce_fused", "gemm_one_shot_all_reduce",
                 "gemm_reduce_scatter", "gemm_reduce_scatter_ce_persistent", "one_shot_all_reduce_bias",
                 "one_shot_all_reduce_bias_rms_norm", "rms_norm", "two_shot_all_reduce_bias",
                 "two_shot_all_reduce_bias_rms_norm"]:
        assert callable(getattr(fused, name)), name
    for name in ["symm_mem_sync", "send_signal", "get_flat_tid", "arrive_gmem_barrier", "wait_gmem_barrier"]:
        assert hasattr(kraken_b200._ptx_utils, name), name
    for name in ["benchmark_with_event", "benchmark_with_profiler", "log_triton_kernel", "plot_experiment_comparison"]:
        assert hasattr(kraken_b200._logging, name), name
    sig = inspect.signature(fused.one_shot_all_reduce_bias_rms_norm)
    assert list(sig.parameters)[:6] == ["symm_mem_input", "x", "bias", "w", "y", "eps"]
    sig = inspect.signature(fused.gemm_reduce_scatter_ce_persistent)
    assert list(sig.parameters)[:4] == ["a", "b", "reduce_op", "group"]


def test_native_library_loads_and_validates():
    L = klib.lib()
    # no driver here: calls must fail with a message, not crash
    assert L.kr_num_sms() in (-1,) or L.kr_num_sms() > 0
    assert klib.decode_status(1 | (30 << 8) | (3 << 16) | (7 << 24)).startswith("cross-device signal wait")
    assert config.TILE_FLAG_BASE >= config.BARRIER_WORDS


def test_compat_alias():
    from kraken_b200 import compat

    compat.install_alias("kraken_alias_for_test")
    import kraken_alias_for_test.comm as c  # noqa

    assert c.one_shot_all_reduce is comm.one_shot_all_reduce


def test_single_process_cpu_ops():
    torch.manual_seed(0)
    x = torch.randn(8, 64, dtype=torch.bfloat16)
    w = (1 + 0.1 * torch.randn(64)).to(torch.bfloat16)
    bias = torch.randn(64, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    fused.one_shot_all_reduce_bias_rms_norm(torch.empty_like(x), x, bias, w, y, 1e-5)
    xf = x.float() + bias.float()
    expect = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    torch.testing.assert_close(y.float(), expect, atol=4e-2, rtol=4e-2)
    a = torch.randn(16, 32, dtype=torch.bfloat16)
    b = torch.randn(32, 24, dtype=torch.bfloat16)
    torch.testing.assert_close(fused.gemm_one_shot_all_reduce_fused(a, b), a.float() @ b.float())
    ag, c = fused.all_gather_matmul(a, b)
    torch.testing.assert_close(ag, a)
    assert c.shape == (16, 24)


def _gloo_config1(rank, ws):
    # x bf16 [128,1024] ~N(0,1) seeded by rank, shared bias [1024], w ~ N(1, 0.1), eps 1e-5
    g = torch.Generator().manual_seed(1234)
    bias = torch.randn(1024, generator=g).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(1024, generator=g)).to(torch.bfloat16)
    xs = [torch.randn(128, 1024, generator=torch.Generator().manual_seed(42 + r)).to(torch.bfloat16) for r in range(ws)]
    x = xs[rank]
    total = sum(t.float() for t in xs) + bias.float()
    expect = total * torch.rsqrt(total.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    for fn in (fused.one_shot_all_reduce_bias_rms_norm, fused.two_shot_all_reduce_bias_rms_norm):
        y = torch.empty_like(x)
        fn(torch.empty_like(x), x, bias, w, y, 1e-5)
        torch.testing.assert_close(y.float(), expect, atol=4e-2, rtol=4e-2)
    # all-reduce family
    s = sum(t.float() for t in xs)
    for fn in (comm.one_shot_all_reduce, comm.two_shot_all_reduce):
        torch.testing.assert_close(fn(x).float(), s, atol=1e-1, rtol=1e-1)
    z = x.clone()
    assert comm.multimem_all_reduce(z) is z
    torch.testing.assert_close(z.float(), s, atol=1e-1, rtol=1e-1)
    rs = comm.reduce_scatter(x)
    torch.testing.assert_close(rs.float(), s[rank * 64:(rank + 1) * 64], atol=1e-1, rtol=1e-1)
    prog = torch.zeros(ws * 2, dtype=torch.int32)
    ag = comm.all_gather_w_progress(x, progress=prog, splits_per_rank=2)
    torch.testing.assert_close(ag, torch.cat(xs, 0))
    assert bool((prog != 0).all())
    out = torch.empty_like(x)
    fused.two_shot_all_reduce_bias(torch.empty_like(x), x, bias, out)
    torch.testing.assert_close(out.float(), s + bias.float(), atol=1e-1, rtol=1e-1)
    fullbias = torch.randn(128, 1024, generator=g).to(torch.bfloat16)
    fused.one_shot_all_reduce_bias(torch.empty_like(x), x, fullbias, out)
    torch.testing.assert_close(out.float(), s + fullbias.float(), atol=1e-1, rtol=1e-1)
    # GEMM family: K sharded across ranks
    gk = torch.Generator().manual_seed(7)
    a_full = torch.randn(64, 96 * ws, generator=gk).to(torch.bfloat16)
    b_full = (0.02 * torch.randn(96 * ws, 48, generator=gk)).to(torch.bfloat16)
    a_loc = a_full[:, rank * 96:(rank + 1) * 96].contiguous()
    b_loc = b_full[rank * 96:(rank + 1) * 96].contiguous()
    full = a_full.float() @ b_full.float()
    torch.testing.assert_close(fused.gemm_one_shot_all_reduce_fused(a_loc, b_loc), full, atol=1e-2, rtol=1e-2)
    for fn in (fused.gemm_reduce_scatter, fused.gemm_reduce_scatter_ce_persistent):
        r = fn(a_loc, b_loc)
        torch.testing.assert_close(r.float(), full[rank * 32:(rank + 1) * 32], atol=2e-2, rtol=2e-2)
    # AG matmul: M sharded
    a_shard = a_full[rank * 32:(rank + 1) * 32].contiguous()
    gathered, c = fused.all_gather_matmul(a_shard, b_full)
    torch.testing.assert_close(gathered, a_full)
    torch.testing.assert_close(c.float(), full, atol=2e-2, rtol=2e-2)
    # model block
    mlp = kraken_b200.models.TPMLP(hidden=64, ffn=128 * ws, device="cpu", seed=3)
    xs2 = torch.randn(16, 64, generator=torch.Generator().manual_seed(5 + rank)).to(torch.bfloat16)
    yo = mlp.prefill(xs2)
    assert yo.shape == (16, 64) and torch.isfinite(yo.float()).all()


def test_gloo_world_size_2_plumbing():
    run_distributed(_gloo_config1, 2, "gloo")


def _gloo_rank_skips(rank, ws):
    # one rank never joins the collective: the others must get an error from the process-group
    # timeout, not hang
    import datetime

    import torch.distributed as dist

    pg = dist.new_group(timeout=datetime.timedelta(seconds=3))
    x = torch.ones(8, dtype=torch.bfloat16)
    if rank == 0:
        with pytest.raises(Exception):
            comm.two_shot_all_reduce(x, group=pg)
    # rank 1 skips the op on purpose


def test_gloo_missing_rank_times_out():
    run_distributed(_gloo_rank_skips, 2, "gloo")


def test_config_sizing_overrides(monkeypatch):
    from kraken_b200 import config
    from kraken_b200.comm.all_reduce import push_limit_bytes

    assert config.push_tagged_max_bytes() == 64 << 10 and config.push_tagged_max_bytes(2) == 512 << 10
    monkeypatch.setenv("KRAKEN_PUSH_TAGGED_KB", "0")
    assert config.push_tagged_max_bytes() == 0
    assert config.gemm_flops_per_s() == 1450e12
    monkeypatch.setenv("KRAKEN_GEMM_TFLOPS", "1000")
    assert config.gemm_flops_per_s() == 1000e12
    assert config.comm_cta_bytes_per_s("pull") == 15e9 and config.comm_cta_bytes_per_s("multicast") == 10e9
    monkeypatch.setenv("KRAKEN_COMM_CTA_GBS_PUSH", "33")
    assert config.comm_cta_bytes_per_s("push") == 33e9
    # push-style one-shot: the limit shrinks with the world size and stops where pulling was measured faster
    assert push_limit_bytes(2) == 2 << 20 and push_limit_bytes(8) == 1 << 20 and push_limit_bytes(4) == 1 << 20
