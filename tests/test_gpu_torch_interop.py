"""Tensors allocated by torch.distributed._symmetric_memory are accepted by the ops: `rendezvous`
wraps torch's handle (same attribute names) when the tensor is not from the native allocator.
Runs as a 1-rank NCCL job on one GPU; skipped when torch's symmetric memory is unavailable."""
import pytest
import torch

from helpers import run_distributed

pytestmark = pytest.mark.gpu


def _interop(rank, ws):
    import torch.distributed as dist

    try:
        import torch.distributed._symmetric_memory as tsm

        t = tsm.empty(64, 1024, dtype=torch.bfloat16, device=f"cuda:{rank}")
        tsm.rendezvous(t, group=dist.group.WORLD)
    except Exception as e:      # torch build without CUDA symmetric memory
        print("torch symmetric memory unavailable:", e)
        return
    import kraken_b200
    from kraken_b200 import comm, fused
    from kraken_b200.parallel import symm_mem

    x = torch.randn(64, 1024, device=f"cuda:{rank}").to(torch.bfloat16)
    t.copy_(x)
    hdl = symm_mem.rendezvous(t)
    assert hdl.world_size == ws and hdl.rank == rank and hdl.alloc is None
    assert symm_mem.is_symm_tensor(t)
    out = comm.one_shot_all_reduce(t)
    torch.testing.assert_close(out.float(), x.float() * ws, atol=1e-1, rtol=1e-1)
    w = torch.ones(1024, device=x.device, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    fused.one_shot_all_reduce_bias_rms_norm(t, x, None, w, y, 1e-5)
    xf = x.float() * ws
    torch.testing.assert_close(y.float(), xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5), atol=4e-2, rtol=4e-2)
    torch.cuda.synchronize()
    kraken_b200.check_status()


def test_torch_symmetric_memory_tensors_are_accepted():
    run_distributed(_interop, 1, "nccl")
