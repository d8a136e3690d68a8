"""Single-GPU numerics of the memory-bound collectives and the fused bias / RMSNorm epilogues,
at world size 1 and at emulated world sizes 2/4/8 (all ranks of a kernel run as ONE cooperative
launch on one GPU). Every result is compared with a plain PyTorch fp32 computation of the same op.
Shapes follow the reference's tests: [1024, 1024] bf16 for all-reduce (test/test_allreduce.py:52),
x/bias [b, 5120] for the bias ops (test/test_allreduce_bias.py:57-71)."""
import pytest
import torch

from kraken_b200 import comm, fused
from kraken_b200.parallel import EmuWorld, symm_mem

pytestmark = pytest.mark.gpu


def _inputs(ws, shape, seed=0):
    return [torch.randn(*shape, generator=torch.Generator().manual_seed(seed + 42 + r)).to(torch.bfloat16).cuda()
            for r in range(ws)]


def _poison(t):
    t.view(torch.int16).fill_(-1)     # NaN pattern: unwritten outputs are detected


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("shape", [(1024, 1024), (3, 40), (7, 1000)])
def test_one_shot_all_reduce(ws, shape):
    world = EmuWorld(ws)
    xs = _inputs(ws, shape)
    ts = world.symmetric(shape, torch.bfloat16)
    for r in range(ws):
        ts[r].copy_(xs[r])
    expect = sum(x.float() for x in xs)
    outs = world.run(lambda r: comm.one_shot_all_reduce(ts[r]))
    for r in range(ws):
        torch.testing.assert_close(outs[r].float(), expect, atol=1e-1, rtol=1e-1)
    # bitwise-identical across ranks? (rotated peer order -> not required); but repeatable:
    outs2 = world.run(lambda r: comm.one_shot_all_reduce(ts[r]))
    for r in range(ws):
        assert torch.equal(outs[r], outs2[r])


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("numel", [1024 * 1024, 8 * 4096 + 64, 40])
def test_two_shot_all_reduce(ws, numel):
    world = EmuWorld(ws)
    xs = _inputs(ws, (numel,))
    expect = sum(x.float() for x in xs)
    for _ in range(2):        # second round: staging workspace reused, pads must have reset
        outs = world.run(lambda r: comm.two_shot_all_reduce(xs[r]))
        for r in range(ws):
            torch.testing.assert_close(outs[r].float(), expect, atol=1e-1, rtol=1e-1)
        for r in range(1, ws):
            assert torch.equal(outs[0], outs[r])      # every rank receives the same bits


@pytest.mark.parametrize("ws", [1, 2, 4])
def test_multimem_all_reduce_falls_back_in_place(ws):
    world = EmuWorld(ws)          # emulated ranks have no multicast mapping: P2P form, same contract
    xs = _inputs(ws, (64, 1024))
    ts = world.symmetric((64, 1024), torch.bfloat16)
    for r in range(ws):
        ts[r].copy_(xs[r])
    expect = sum(x.float() for x in xs)
    outs = world.run(lambda r: comm.multimem_all_reduce(ts[r]))
    for r in range(ws):
        assert outs[r].data_ptr() == ts[r].data_ptr()
        torch.testing.assert_close(ts[r].float(), expect, atol=1e-1, rtol=1e-1)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("symmetric_input", [True, False])
def test_reduce_scatter(ws, symmetric_input):
    world = EmuWorld(ws)
    shape = (ws * 96, 256)
    xs = _inputs(ws, shape)
    expect = sum(x.float() for x in xs)
    if symmetric_input:
        ts = world.symmetric(shape, torch.bfloat16)
        for r in range(ws):
            ts[r].copy_(xs[r])
        src = ts
    else:
        src = xs
    outs = world.run(lambda r: comm.reduce_scatter(src[r]))
    for r in range(ws):
        torch.testing.assert_close(outs[r].float(), expect[r * 96:(r + 1) * 96], atol=1e-1, rtol=1e-1)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("splits", [1, 2, 4])
def test_all_gather_w_progress_sm(ws, splits):
    world = EmuWorld(ws)
    shape = (256, 1024)
    xs = _inputs(ws, shape)
    ts = world.symmetric(shape, torch.bfloat16)
    for r in range(ws):
        ts[r].copy_(xs[r])
    progs = [torch.zeros(ws * splits, dtype=torch.uint32, device="cuda") for _ in range(ws)]
    outs = world.run(lambda r: comm.all_gather_w_progress(ts[r], progress=progs[r], splits_per_rank=splits,
                                                          backend="sm"))
    expect = torch.cat(xs, 0)
    for r in range(ws):
        assert torch.equal(outs[r], expect)
        assert bool((progs[r].to(torch.int64) != 0).all())


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("b", [1, 2, 16, 64])
@pytest.mark.parametrize("full_bias", [True, False])
def test_all_reduce_bias(ws, b, full_bias):
    world = EmuWorld(ws)
    D = 5120
    xs = _inputs(ws, (b, D))
    bias = torch.randn(b, D).to(torch.bfloat16).cuda() if full_bias else torch.randn(D).to(torch.bfloat16).cuda()
    pads = world.symmetric((1024, 1024), torch.bfloat16)
    expect = sum(x.float() for x in xs) + bias.float()
    for fn in (fused.one_shot_all_reduce_bias, fused.two_shot_all_reduce_bias):
        outs = [torch.empty_like(xs[0]) for _ in range(ws)]
        for o in outs:
            _poison(o)
        world.run(lambda r: fn(pads[r], xs[r], bias, outs[r]))
        for r in range(ws):
            torch.testing.assert_close(outs[r].float(), expect, atol=5e-2, rtol=5e-2)
    # no bias
    outs = [torch.empty_like(xs[0]) for _ in range(ws)]
    world.run(lambda r: fused.one_shot_all_reduce_bias(pads[r], xs[r], None, outs[r]))
    torch.testing.assert_close(outs[0].float(), sum(x.float() for x in xs), atol=5e-2, rtol=5e-2)


def _rms_ref(x, w, eps):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


@pytest.mark.parametrize("rows,D", [(1, 5120), (64, 5120), (300, 8192), (5, 64), (2, 40000)])
def test_rms_norm(rows, D):
    x = torch.randn(rows, D).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(D)).to(torch.bfloat16).cuda()
    y = fused.rms_norm(x, w, 1e-5)
    torch.testing.assert_close(y.float(), _rms_ref(x, w, 1e-5), atol=4e-2, rtol=4e-2)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("b", [1, 4, 32, 200])
@pytest.mark.parametrize("D", [5120, 8192])
def test_all_reduce_bias_rms_norm(ws, b, D):
    world = EmuWorld(ws)
    xs = _inputs(ws, (b, D))
    bias = torch.randn(D).to(torch.bfloat16).cuda()
    fullbias = torch.randn(b, D).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(D)).to(torch.bfloat16).cuda()
    pads = world.symmetric((b * D + 64,), torch.bfloat16)
    for bb in (bias, fullbias):
        total = sum(x.float() for x in xs) + bb.float()
        expect = _rms_ref(total, w, 1e-5)
        for fn in (fused.one_shot_all_reduce_bias_rms_norm, fused.two_shot_all_reduce_bias_rms_norm):
            ys = [torch.empty_like(xs[0]) for _ in range(ws)]
            for y in ys:
                _poison(y)
            world.run(lambda r: fn(pads[r], xs[r], bb, w, ys[r], 1e-5))
            for r in range(ws):
                torch.testing.assert_close(ys[r].float(), expect, atol=4e-2, rtol=4e-2)


# ---- push-style one-shot kernels (small messages) ------------------------------------------------
@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("numel", [8, 2048, 5120 * 3, 64 * 1024])
@pytest.mark.parametrize("with_bias", [False, True])
def test_push_and_pull_one_shot_agree(ws, numel, with_bias):
    world = EmuWorld(ws)
    xs = _inputs(ws, (numel,), seed=31)
    bias = torch.randn(numel, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda() if with_bias else None
    expect = sum(x.float() for x in xs) + (bias.float() if with_bias else 0.0)
    pads = world.symmetric((numel,), torch.bfloat16)
    res = {}
    for algo in ("push", "pull"):
        for _ in range(3):          # three calls: both workspace halves, then the first again
            outs = [torch.empty_like(xs[r]) for r in range(ws)]
            for o in outs:
                _poison(o)
            world.run(lambda r: fused.one_shot_all_reduce_bias(pads[r], xs[r], bias, outs[r], algo=algo))
            for r in range(ws):
                torch.testing.assert_close(outs[r].float(), expect, atol=5e-2, rtol=5e-2)
        res[algo] = outs
    for r in range(ws):
        assert torch.equal(res["push"][0], res["push"][r])      # rank-order sums: same bits on every rank


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
@pytest.mark.parametrize("b,D", [(1, 5120), (3, 5120), (16, 1024), (40, 8192), (2, 64), (2, 8192), (4, 4096)])
def test_push_all_reduce_bias_rms_norm(ws, b, D):
    world = EmuWorld(ws)
    xs = _inputs(ws, (b, D), seed=33)
    g = torch.Generator().manual_seed(6)
    bias = torch.randn(D, generator=g).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(torch.bfloat16).cuda()
    s = sum(x.float() for x in xs) + bias.float()
    expect = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()
    pads = world.symmetric((b, D), torch.bfloat16)
    for algo in ("push", "pull"):
        for _ in range(2):
            ys = [torch.empty_like(xs[r]) for r in range(ws)]
            for y in ys:
                _poison(y)
            world.run(lambda r: fused.one_shot_all_reduce_bias_rms_norm(pads[r], xs[r], bias, w, ys[r], 1e-5, algo=algo))
            for r in range(ws):
                torch.testing.assert_close(ys[r].float(), expect, atol=4e-2, rtol=4e-2)


def test_push_tagged_and_flag_forms_share_a_workspace(monkeypatch):
    # small messages travel tagged (no barrier), larger ones behind one barrier; both forms alternate
    # workspace halves by the same call counter and must never read each other's leftovers
    ws, numel = 4, 4096
    world = EmuWorld(ws)
    pads = world.symmetric((numel,), torch.bfloat16)
    for i, kb in enumerate([64, 0, 64, 64, 0, 0, 64, 0, 64]):
        monkeypatch.setenv("KRAKEN_PUSH_TAGGED_KB", str(kb))
        xs = _inputs(ws, (numel,), seed=100 + i)
        expect = sum(x.float() for x in xs)
        outs = [torch.empty_like(xs[r]) for r in range(ws)]
        for o in outs:
            _poison(o)
        world.run(lambda r: fused.one_shot_all_reduce_bias(pads[r], xs[r], None, outs[r], algo="push"))
        for r in range(ws):
            torch.testing.assert_close(outs[r].float(), expect, atol=5e-2, rtol=5e-2)
            assert torch.equal(outs[0], outs[r])
