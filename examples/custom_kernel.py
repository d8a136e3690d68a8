"""Builds and runs examples/custom_kernel.cu: a user kernel that uses the library's symmetric
memory (allocation + rendezvous from Python) and its device-side barrier (ptx_sync.cuh).

    python examples/custom_kernel.py                                   # one GPU
    torchrun --nnodes 1 --nproc-per-node 4 --master-addr 127.0.0.1 examples/custom_kernel.py
"""
import ctypes
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from kraken_b200.ops import lib as klib  # noqa: E402
from kraken_b200.parallel import symm_mem  # noqa: E402
from kraken_b200.utils import init_from_env  # noqa: E402


def build() -> str:
    src = os.path.join(ROOT, "examples", "custom_kernel.cu")
    out = os.path.join(ROOT, "examples", "libcustom_kernel.so")
    if not os.path.exists(out) or os.path.getmtime(out) < os.path.getmtime(src):
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-shared",
                               "-Xcompiler", "-fPIC", "-I", os.path.join(ROOT, "csrc", "include"), src, "-o", out])
    return out


def main():
    rank, _, ws = init_from_env()
    if rank == 0:
        build()
    if ws > 1:
        torch.distributed.barrier()
    so = ctypes.CDLL(build())
    dev = torch.device("cuda", torch.cuda.current_device())
    n = 1 << 20
    x = symm_mem.empty(n, dtype=torch.float32, device=dev)
    x.fill_(float(rank + 1))
    hdl = symm_mem.rendezvous(x)
    out = torch.empty(n, dtype=torch.float32, device=dev)
    status = ctypes.c_void_p(klib.lib().kr_status_ptr())
    rc = so.launch_sum_peers(ctypes.c_void_p(hdl.buffer_ptrs_dev), ctypes.c_void_p(hdl.signal_pad_ptrs_dev),
                             ctypes.c_void_p(out.data_ptr()), ctypes.c_size_t(n), rank, ws, status,
                             ctypes.c_double(2000.0), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    klib.check_status()
    expect = float(sum(range(1, ws + 1)))
    assert torch.all(out == expect), (out[:4], expect)
    print(f"rank {rank}: every element is {expect} as expected", flush=True)
    if ws > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
