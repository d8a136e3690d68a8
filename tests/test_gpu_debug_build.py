"""The debug build of the native library (KRAKEN_DEBUG=1: device-side bounds checks that record
KR_ERR_BOUNDS and skip the access instead of faulting). Each case runs in a child process because
a process loads one build of the library. The checks must fire when an index is out of range (the
self-test kernel guards its only store with a check that cannot pass) and must stay silent on
correct runs of the kernels that carry them."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code: str, debug: bool) -> str:
    env = dict(os.environ)
    env["KRAKEN_DEBUG"] = "1" if debug else "0"
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout + r.stderr
    return r.stdout


SELFTEST = """
from kraken_b200 import _ptx_utils as ptx
from kraken_b200.ops import lib
print("debug", lib.lib().kr_is_debug_build())
print("selftest", ptx.bounds_check_selftest())
"""


def test_bounds_check_fires_only_in_the_debug_build():
    out = _run(SELFTEST, debug=True)
    assert "debug 1" in out and "selftest (0, True)" in out        # store skipped, error recorded
    out = _run(SELFTEST, debug=False)
    assert "debug 0" in out and "selftest (3, False)" in out       # check compiled away


OPS = """
import torch
import kraken_b200
from kraken_b200 import comm, fused
from kraken_b200.parallel import EmuWorld
ws = 4
world = EmuWorld(ws)
g = torch.Generator().manual_seed(1)
a_s = [torch.randn(1024, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(ws)]
bt_s = [(0.05 * torch.randn(520, 128, generator=g)).to(torch.bfloat16).cuda() for _ in range(ws)]
full = sum(a.float() @ bt.float().t() for a, bt in zip(a_s, bt_s))
for algo in ("pull", "scatter", "push"):
    outs = world.run(lambda r: fused.gemm_reduce_scatter(a_s[r], bt_s[r].t(), algo=algo))
    for r in range(ws):
        torch.testing.assert_close(outs[r].float(), full[r * 256:(r + 1) * 256], atol=6e-2, rtol=3e-2)
ts = world.symmetric((256, 256), torch.bfloat16)
for r in range(ws):
    ts[r].copy_(torch.randn(256, 256, generator=g).to(torch.bfloat16))
bt = (0.05 * torch.randn(384, 256, generator=g)).to(torch.bfloat16).cuda()
outs = world.run(lambda r: fused.all_gather_matmul(ts[r], bt.t(), backend="push", num_comm_sms=2, splits_per_rank=2))
gathered = torch.cat([t for t in ts], 0)
assert all(torch.equal(o[0], gathered) for o in outs)
outs = world.run(lambda r: comm.one_shot_all_reduce(ts[r]))
torch.testing.assert_close(outs[0].float(), sum(t.float() for t in ts), atol=1e-1, rtol=1e-1)
torch.cuda.synchronize()
kraken_b200.check_status()
print("ops ok")
"""


def test_debug_build_is_silent_on_correct_runs():
    assert "ops ok" in _run(OPS, debug=True)
