"""Ops are plain stream-ordered kernel launches with self-resetting flags, so they can be captured
in a CUDA graph and replayed (the reference's harness offers graph replay for its kernels:
kraken/_logging/benchmarking.py:99-108). Single GPU, world size 1."""
import pytest
import torch

from kraken_b200 import comm, fused
from kraken_b200.parallel import symm_mem

pytestmark = pytest.mark.gpu


def test_ops_replay_under_cuda_graph():
    dev = torch.device("cuda", torch.cuda.current_device())
    x = symm_mem.empty(256, 1024, dtype=torch.bfloat16, device=dev)
    symm_mem.rendezvous(x)
    w = (1 + 0.1 * torch.randn(1024, device=dev)).to(torch.bfloat16)
    bt = (0.05 * torch.randn(512, 1024, device=dev)).to(torch.bfloat16)
    x.copy_(torch.randn(256, 1024, device=dev).to(torch.bfloat16))

    def chain():
        y = comm.one_shot_all_reduce(x)           # world size 1: a copy through the kernel
        z = fused.rms_norm(y, w, 1e-5)
        return fused.matmul(z, bt.t())

    ref = chain()                                  # warm-up outside capture (first-use set-up happens here)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out = chain()
    for _ in range(3):
        x.copy_(torch.randn(256, 1024, device=dev).to(torch.bfloat16))
        g.replay()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), chain().float(), atol=2e-2, rtol=2e-2)
    assert ref.shape == out.shape
