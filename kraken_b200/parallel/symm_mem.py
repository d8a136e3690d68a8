"""Symmetric memory: allocation, rendezvous and the handle every kernel launch starts from.

Mirrors the slice of ``torch.distributed._symmetric_memory`` that the reference consumes
(``empty`` / ``rendezvous`` / ``get_symm_mem_workspace`` / ``_get_backend_stream`` and the handle's
``rank``, ``world_size``, ``buffer_ptrs_dev``, ``signal_pad_ptrs_dev``, ``multicast_ptr``,
``get_buffer``, ``get_signal_pad``, ``barrier``, ``stream_write_value32`` — e.g.
kraken/comm/one_shot_all_reduce.py:89-97, kraken/comm/copy_engine_all_gather.py:13-58,
kraken/fused/gemm_reduce_scatter_ce_persistent.py:146,338), on top of the library's own cuMem/fd
allocator. Tensors allocated by torch's symmetric memory are accepted too: ``rendezvous`` falls
back to torch's own rendezvous for tensors it does not own and wraps the result.

Three kinds of "world":
  * real: one process per GPU, ``torch.distributed`` initialised (any backend; control traffic only);
  * single: no process group — world size 1;
  * emulated: ``EmuWorld(n)`` keeps n virtual ranks on ONE GPU; inside ``with world.launch():`` the
    per-rank op calls are recorded and run as one cooperative kernel (used by single-GPU tests to
    exercise the multi-rank index math and barrier protocol).
CPU tensors get a handle with only ``rank``/``world_size``: the CPU path of every op is the
pure-PyTorch reference backend over the process group.
"""
from __future__ import annotations

import contextlib
import ctypes
import itertools
import os
import threading
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import config
from ..ops import lib as _lib


# ---------------------------------------------------------------------------------------------
# groups
# ---------------------------------------------------------------------------------------------
@dataclass
class GroupInfo:
    rank: int
    world_size: int
    name: str
    pg: object = None          # torch ProcessGroup, or None (single / emulated)
    emu: object = None         # EmuWorld when emulated


_tls = threading.local()


def _emu_ctx():
    return getattr(_tls, "emu", None)


def resolve_group(group=None) -> GroupInfo:
    """Group argument of an op -> (rank, world size, name). ``None`` means the default group."""
    emu = _emu_ctx()
    if emu is not None:
        world, rank = emu
        return GroupInfo(rank, world.world_size, world.name, None, world)
    if isinstance(group, GroupInfo):
        return group
    if not dist.is_available() or not dist.is_initialized():
        return GroupInfo(0, 1, "single")
    pg = group if group is not None and not isinstance(group, str) else dist.group.WORLD
    if isinstance(group, str):
        try:
            from torch.distributed.distributed_c10d import _resolve_process_group

            pg = _resolve_process_group(group)
        except Exception:
            pg = dist.group.WORLD
    name = getattr(pg, "group_name", None) or "world"
    return GroupInfo(dist.get_rank(pg), dist.get_world_size(pg), str(name), pg)


# ---------------------------------------------------------------------------------------------
# raw device memory as torch tensors
# ---------------------------------------------------------------------------------------------
class _DeviceSpan:
    """Exposes [ptr, ptr+nbytes) through the CUDA array interface; keeps `owner` alive."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


def _tensor_from_ptr(ptr: int, nbytes: int, device: torch.device, owner) -> torch.Tensor:
    return torch.as_tensor(_DeviceSpan(ptr, nbytes, owner), device=device)


def _view(raw_u8: torch.Tensor, shape, dtype) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    return raw_u8[:nbytes].view(dtype).view(*shape)


# ---------------------------------------------------------------------------------------------
# native allocation
# ---------------------------------------------------------------------------------------------
class SymmAllocation:
    """One block from the native allocator: [data | signal pad], local until rendezvous."""

    def __init__(self, nbytes: int, device: torch.device, pad_bytes: int | None = None):
        self.device = torch.device(device)
        self.pad_bytes = config.signal_pad_bytes() if pad_bytes is None else pad_bytes
        h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().kr_symm_alloc(int(nbytes), int(self.pad_bytes), ctypes.byref(h)))
        self.h = h
        self.data_bytes = int(_lib.lib().kr_symm_data_bytes(h))
        self.local_ptr = int(_lib.lib().kr_symm_local_ptr(h))
        self.handle: SymmHandle | None = None
        self._raw = _tensor_from_ptr(self.local_ptr, self.data_bytes, self.device, self)

    def contains(self, ptr: int) -> bool:
        return self.local_ptr <= ptr < self.local_ptr + self.data_bytes

    def tensor(self, shape, dtype) -> torch.Tensor:
        return _view(self._raw, shape, dtype)


_allocations: list[SymmAllocation] = []
_alloc_lock = threading.Lock()
_rdv_seq = itertools.count()


_alloc_by_ptr: dict[tuple, SymmAllocation | None] = {}


def _find_allocation(t: torch.Tensor) -> SymmAllocation | None:
    """Allocation that holds tensor `t` (ops call this on every invocation: hits are cached by
    data pointer; misses are not cached because ordinary memory is recycled by torch's allocator)."""
    ptr = t.data_ptr()
    key = (t.device.index, ptr)
    hit = _alloc_by_ptr.get(key)
    if hit is not None:
        return hit
    for a in _allocations:
        if a.device == t.device and a.contains(ptr):
            while len(_alloc_by_ptr) >= 4096:                    # evict the oldest entries, keep the hot ones
                _alloc_by_ptr.pop(next(iter(_alloc_by_ptr)))
            _alloc_by_ptr[key] = a
            return a
    return None


class SymmHandle:
    """What ``rendezvous`` returns. Attribute names follow torch's ``_SymmetricMemory``."""

    def __init__(self, alloc: SymmAllocation | None, info: GroupInfo, *, buffer_ptrs, signal_pad_ptrs,
                 buffer_ptrs_dev: int, signal_pad_ptrs_dev: int, multicast_ptr: int, buffer_size: int,
                 signal_pad_size: int, device, keepalive=None):
        self.alloc = alloc
        self.group = info
        self.rank = info.rank
        self.world_size = info.world_size
        self.buffer_ptrs = list(buffer_ptrs)
        self.signal_pad_ptrs = list(signal_pad_ptrs)
        self.buffer_ptrs_dev = buffer_ptrs_dev
        self.signal_pad_ptrs_dev = signal_pad_ptrs_dev
        self.multicast_ptr = multicast_ptr
        self.buffer_size = buffer_size
        self.signal_pad_size = signal_pad_size
        self.device = torch.device(device)
        self._keepalive = keepalive
        self._host_ptr_array = (ctypes.c_void_p * self.world_size)(*self.buffer_ptrs)

    # -- torch-compatible accessors
    def get_buffer(self, rank: int, sizes, dtype, storage_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        n = 1
        for s in sizes:
            n *= int(s)
        off = storage_offset * esz
        if off + n * esz > self.buffer_size:
            raise ValueError("get_buffer: view exceeds the symmetric buffer")
        raw = _tensor_from_ptr(self.buffer_ptrs[rank] + off, n * esz, self.device, self)
        return raw.view(dtype).view(*sizes)

    def get_signal_pad(self, rank: int, sizes=None, dtype=torch.uint32, storage_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        if sizes is None:
            sizes = (self.signal_pad_size // esz - storage_offset,)
        n = 1
        for s in sizes:
            n *= int(s)
        raw = _tensor_from_ptr(self.signal_pad_ptrs[rank] + storage_offset * esz, n * esz, self.device, self)
        return raw.view(dtype).view(*sizes)

    def barrier(self, channel: int = 0) -> None:
        """Cross-device barrier of all ranks on the current stream (one tiny kernel)."""
        slot = config.BARRIER_WORDS // self.world_size - 1 - channel
        _lib.check(_lib.lib().kr_symm_barrier(self.signal_pad_ptrs_dev, self.rank, self.world_size, slot,
                                              _lib.current_stream_ptr()))

    def stream_write_value32(self, tensor: torch.Tensor, offset: int, val: int) -> None:
        addr = tensor.data_ptr() + offset * tensor.element_size()
        _lib.check(_lib.lib().kr_stream_write_value32(_lib.current_stream_ptr(), addr, int(val)))

    def stream_wait_value32(self, tensor: torch.Tensor, offset: int, val: int) -> None:
        addr = tensor.data_ptr() + offset * tensor.element_size()
        _lib.check(_lib.lib().kr_stream_wait_value32(_lib.current_stream_ptr(), addr, int(val)))

    @property
    def signal_pad_words(self) -> int:
        return self.signal_pad_size // 4

    def offset_of(self, t: torch.Tensor) -> int:
        """Byte offset of tensor `t` inside this rank's symmetric buffer."""
        off = t.data_ptr() - self.buffer_ptrs[self.rank]
        if off < 0 or off >= self.buffer_size:
            raise ValueError("tensor does not live in this symmetric buffer")
        return off


class CpuHandle:
    """Handle for CPU tensors: the CPU path of every op only needs rank and world size."""

    def __init__(self, info: GroupInfo):
        self.group = info
        self.rank = info.rank
        self.world_size = info.world_size
        self.multicast_ptr = 0

    def barrier(self, channel: int = 0) -> None:
        if self.group.pg is not None:
            dist.barrier(self.group.pg)


# ---------------------------------------------------------------------------------------------
# public API
# ---------------------------------------------------------------------------------------------
def is_cuda_device(device) -> bool:
    return torch.device(device).type == "cuda"


def empty(*shape, dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
    """Allocates a tensor in symmetric memory (local until ``rendezvous``). CPU: a plain tensor."""
    if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
        shape = tuple(shape[0])
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    device = torch.device(device)
    if device.type != "cuda":
        return torch.empty(*shape, dtype=dtype, device=device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    emu = _emu_ctx()
    if emu is not None:
        return emu[0].empty(emu[1], shape, dtype)
    if config.symm_backend() == "torch":
        import torch.distributed._symmetric_memory as tsm

        return tsm.empty(*shape, dtype=dtype, device=device)
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    alloc = SymmAllocation(nbytes, device)
    with _alloc_lock:
        _allocations.append(alloc)
    return alloc.tensor(shape, dtype)


def _exchange_and_map(alloc: SymmAllocation, info: GroupInfo) -> SymmHandle:
    L = _lib.lib()
    ws, rank = info.world_size, info.rank
    with torch.cuda.device(alloc.device):
        _lib.check(L.kr_symm_set_group(alloc.h, rank, ws))
        mc_ptr = 0
        if ws > 1:
            seq = next(_rdv_seq)
            my_name = f"kraken-b200-{os.getpid()}-{seq}-{rank}".encode()
            sock = ctypes.c_int(-1)
            _lib.check(L.kr_ipc_open(my_name, ctypes.byref(sock)))
            try:
                names = [None] * ws
                dist.all_gather_object(names, my_name, group=info.pg)   # also: every socket is bound
                fd = ctypes.c_int(-1)
                _lib.check(L.kr_symm_export_fd(alloc.h, ctypes.byref(fd)))
                for peer in range(ws):
                    if peer != rank:
                        _lib.check(L.kr_ipc_send_fd(sock.value, names[peer], fd.value, rank))
                os.close(fd.value)
                for _ in range(ws - 1):
                    rfd, tag = ctypes.c_int(-1), ctypes.c_int(-1)
                    _lib.check(L.kr_ipc_recv_fd(sock.value, 60000, ctypes.byref(rfd), ctypes.byref(tag)))
                    _lib.check(L.kr_symm_import_fd(alloc.h, tag.value, rfd.value))
                use_mc = config.nvls_enabled() and bool(L.kr_symm_multicast_supported())
                flags = [None] * ws
                dist.all_gather_object(flags, bool(use_mc), group=info.pg)
                use_mc = all(flags)
                if use_mc:
                    if rank == 0:
                        mfd = ctypes.c_int(-1)
                        _lib.check(L.kr_symm_mc_create(alloc.h, ctypes.byref(mfd)))
                        for peer in range(1, ws):
                            _lib.check(L.kr_ipc_send_fd(sock.value, names[peer], mfd.value, 1000))
                        os.close(mfd.value)
                    else:
                        rfd, tag = ctypes.c_int(-1), ctypes.c_int(-1)
                        _lib.check(L.kr_ipc_recv_fd(sock.value, 60000, ctypes.byref(rfd), ctypes.byref(tag)))
                        _lib.check(L.kr_symm_mc_import(alloc.h, rfd.value))
                    _lib.check(L.kr_symm_mc_add_device(alloc.h))
                    dist.barrier(group=info.pg)        # every device added before anyone binds
                    _lib.check(L.kr_symm_mc_bind(alloc.h))
                    mc_ptr = int(L.kr_symm_mc_ptr(alloc.h) or 0)
                dist.barrier(group=info.pg)
            finally:
                L.kr_ipc_close(sock.value)
        _lib.check(L.kr_symm_finalize(alloc.h))
        bufs = [int(L.kr_symm_ptr(alloc.h, r)) for r in range(ws)]
        pads = [int(L.kr_symm_pad_ptr(alloc.h, r)) for r in range(ws)]
        return SymmHandle(alloc, info, buffer_ptrs=bufs, signal_pad_ptrs=pads,
                          buffer_ptrs_dev=int(L.kr_symm_bufs_dev(alloc.h)),
                          signal_pad_ptrs_dev=int(L.kr_symm_pads_dev(alloc.h)), multicast_ptr=mc_ptr,
                          buffer_size=alloc.data_bytes, signal_pad_size=alloc.pad_bytes, device=alloc.device)


_torch_handles: dict[int, SymmHandle] = {}


def _wrap_torch_handle(t: torch.Tensor, info: GroupInfo) -> SymmHandle:
    import torch.distributed._symmetric_memory as tsm

    key = t.untyped_storage().data_ptr()
    if key in _torch_handles:
        return _torch_handles[key]
    hdl = tsm.rendezvous(t, group=info.pg if info.pg is not None else dist.group.WORLD)
    h = SymmHandle(None, info, buffer_ptrs=list(hdl.buffer_ptrs), signal_pad_ptrs=list(hdl.signal_pad_ptrs),
                   buffer_ptrs_dev=int(hdl.buffer_ptrs_dev), signal_pad_ptrs_dev=int(hdl.signal_pad_ptrs_dev),
                   multicast_ptr=int(getattr(hdl, "multicast_ptr", 0) or 0), buffer_size=int(hdl.buffer_size),
                   signal_pad_size=int(hdl.signal_pad_size), device=t.device, keepalive=(hdl, t))
    _torch_handles[key] = h
    return h


def rendezvous(t: torch.Tensor, group=None):
    """Collective on first use per block (handle exchange and peer mapping); cached afterwards, so
    ops may call it on every invocation as the reference does (kraken/comm/one_shot_all_reduce.py:89)."""
    info = resolve_group(group)
    if t.device.type != "cuda":
        return CpuHandle(info)
    if info.emu is not None:
        return info.emu.handle_for(t, info.rank)
    alloc = _find_allocation(t)
    if alloc is None:
        if dist.is_available() and dist.is_initialized():
            try:
                return _wrap_torch_handle(t, info)
            except Exception as e:   # not a symmetric tensor of either allocator
                raise ValueError("tensor was not allocated in symmetric memory "
                                 "(use kraken_b200.parallel.symm_mem.empty)") from e
        raise ValueError("tensor was not allocated in symmetric memory (use kraken_b200.parallel.symm_mem.empty)")
    if alloc.handle is None:
        alloc.handle = _exchange_and_map(alloc, info)
    return alloc.handle


def is_symm_tensor(t: torch.Tensor) -> bool:
    if t.device.type != "cuda":
        return False
    emu = _emu_ctx()
    if emu is not None:
        return emu[0].owns(t)
    return _find_allocation(t) is not None or t.untyped_storage().data_ptr() in _torch_handles


# -- per-group growable workspace (torch: get_symm_mem_workspace) ---------------------------------
_workspaces: dict[tuple, SymmHandle] = {}


def get_symm_mem_workspace(group=None, min_size: int = 0, device=None, kind: str = "shared") -> SymmHandle:
    """Per-group symmetric scratch of at least `min_size` bytes. Growth is collective: all ranks
    must ask for the same size at the same time (they do — ops size it from the op's shape).
    `kind` selects a pool: ops that keep state in their scratch between calls (the GEMM all-reduce
    alternates staging halves) use a pool of their own."""
    info = resolve_group(group)
    if info.emu is not None:
        return info.emu.workspace(info.rank, min_size, kind)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    key = (info.name, device.index, kind)
    hdl = _workspaces.get(key)
    if hdl is not None and hdl.buffer_size >= min_size:
        return hdl
    if capturing():
        raise RuntimeError(f"the '{kind}' symmetric workspace ({min_size} bytes) has to exist before CUDA-graph capture: "
                           "growing it is a collective with host synchronisation. Call "
                           "symm_mem.get_symm_mem_workspace(group, size, kind=...) or run the op once eagerly first "
                           "(note that under capture some ops use another variant, see symm_mem.capturing)")
    size = max(int(min_size), int(os.environ.get("KRAKEN_WS_MIN_MB", "32")) << 20)
    size = 1 << (size - 1).bit_length()      # geometric growth: few re-rendezvous
    pre = int(os.environ.get("KRAKEN_WS_PREALLOC_MB", "0"))
    if pre > 0 and hdl is None:
        dummy = SymmAllocation(pre << 20, device)
        with _alloc_lock:
            _allocations.append(dummy)
        dummy.handle = _exchange_and_map(dummy, info)
    alloc = SymmAllocation(size, device)
    with _alloc_lock:
        _allocations.append(alloc)
    alloc.handle = _exchange_and_map(alloc, info)
    _workspaces[key] = alloc.handle           # the old block stays mapped: views of it may be alive
    return alloc.handle


_backend_streams: dict[tuple, torch.cuda.Stream] = {}


def _get_backend_stream(priority: int = 0) -> torch.cuda.Stream:
    """Cached side stream per (device, priority) for copy-engine work."""
    key = (torch.cuda.current_device(), priority)
    s = _backend_streams.get(key)
    if s is None:
        s = torch.cuda.Stream(priority=priority)
        _backend_streams[key] = s
    return s


# ---------------------------------------------------------------------------------------------
# emulated world: n virtual ranks on one GPU
# ---------------------------------------------------------------------------------------------
class EmuWorld:
    _ids = itertools.count()

    def __init__(self, world_size: int, device=None, pad_bytes: int | None = None):
        self.world_size = world_size
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.name = f"emu{next(EmuWorld._ids)}"
        self.pad_bytes = config.signal_pad_bytes() if pad_bytes is None else pad_bytes
        self._blocks: list[list[SymmAllocation]] = []     # one list of ws allocations per symmetric tensor
        self._handles: dict[int, list[SymmHandle]] = {}
        self._by_kind: dict[tuple, list[int]] = {}
        self._requests: dict[tuple, int] = {}
        self._ws_pools: dict[str, list[SymmHandle]] = {}
        self._keep = []

    def _make_block(self, nbytes: int) -> int:
        allocs = [SymmAllocation(nbytes, self.device, self.pad_bytes) for _ in range(self.world_size)]
        self._blocks.append(allocs)
        bufs = [a.local_ptr for a in allocs]
        pads = [a.local_ptr + a.data_bytes for a in allocs]
        bufs_dev = torch.tensor(bufs, dtype=torch.int64, device=self.device)
        pads_dev = torch.tensor(pads, dtype=torch.int64, device=self.device)
        self._keep += [bufs_dev, pads_dev]
        idx = len(self._blocks) - 1
        self._handles[idx] = [
            SymmHandle(allocs[r], GroupInfo(r, self.world_size, self.name, None, self), buffer_ptrs=bufs,
                       signal_pad_ptrs=pads, buffer_ptrs_dev=bufs_dev.data_ptr(), signal_pad_ptrs_dev=pads_dev.data_ptr(),
                       multicast_ptr=0, buffer_size=allocs[r].data_bytes, signal_pad_size=self.pad_bytes,
                       device=self.device)
            for r in range(self.world_size)
        ]
        return idx

    def empty(self, rank: int, shape, dtype) -> torch.Tensor:
        """Rank `rank`'s view of a symmetric tensor. The k-th request of a rank for a given
        (shape, dtype) maps to the k-th block of that kind, so ranks that allocate in the same
        order (as real ranks do) end up sharing blocks."""
        n = 1
        for s in shape:
            n *= int(s)
        key = (tuple(int(s) for s in shape), dtype)
        blocks = self._by_kind.setdefault(key, [])
        k = self._requests.get((key, rank), 0)
        self._requests[(key, rank)] = k + 1
        if k >= len(blocks):
            blocks.append(self._make_block(n * torch.empty((), dtype=dtype).element_size()))
        return self._blocks[blocks[k]][rank].tensor(shape, dtype)

    def symmetric(self, shape, dtype) -> list[torch.Tensor]:
        """All ranks' views of one new symmetric tensor."""
        n = 1
        for s in shape:
            n *= int(s)
        idx = self._make_block(n * torch.empty((), dtype=dtype).element_size())
        return [a.tensor(shape, dtype) for a in self._blocks[idx]]

    def owns(self, t: torch.Tensor) -> bool:
        return any(a.contains(t.data_ptr()) for blk in self._blocks for a in blk)

    def handle_for(self, t: torch.Tensor, rank: int) -> SymmHandle:
        ptr = t.data_ptr()
        for idx, blk in enumerate(self._blocks):
            if blk[rank].contains(ptr):
                return self._handles[idx][rank]
        raise ValueError("tensor is not rank %d's view of an emulated symmetric tensor" % rank)

    def workspace(self, rank: int, min_size: int, kind: str = "shared") -> SymmHandle:
        pools = self._ws_pools
        handles = pools.get(kind)
        if handles is None or handles[0].buffer_size < min_size:
            size = max(int(min_size), 1 << 20)
            idx = self._make_block(size)
            handles = pools[kind] = self._handles[idx]
        return handles[rank]

    @contextlib.contextmanager
    def rank(self, r: int):
        prev = _emu_ctx()
        _tls.emu = (self, r)
        try:
            yield
        finally:
            _tls.emu = prev

    @contextlib.contextmanager
    def launch(self):
        """Records the per-rank launches made inside the block and runs them as ONE cooperative
        kernel on exit. Exactly one kernel launch per rank may happen inside."""
        L = _lib.lib()
        _lib.check(L.kr_emu_begin(self.world_size))
        try:
            yield
        except BaseException:
            L.kr_emu_abort()
            raise
        _lib.check(L.kr_emu_end(_lib.current_stream_ptr()))

    def run(self, fn):
        """Calls fn(rank) for every virtual rank inside one emulated launch; returns the results."""
        outs = []
        with self.launch():
            for r in range(self.world_size):
                with self.rank(r):
                    outs.append(fn(r))
        return outs


def capturing() -> bool:
    """True while the current stream is being captured into a CUDA graph. Ops that alternate two
    buffer halves / flag banks from call to call (so that they need no barrier) must not do so
    under capture: a replayed graph repeats the SAME half every time, so they switch to their
    barrier-protected variants instead."""
    try:
        return bool(torch.cuda.is_current_stream_capturing())
    except Exception:
        return False


_CALL_COUNTERS = ("_push_calls", "_gemm_ar_calls", "_gemm_rs_calls", "_ag_calls")


def reset_signal_pads(handle: SymmHandle) -> None:
    """Recovery after a reported timeout. A wait that gave up can leave tokens behind in the signal
    pads, and a rank that made a call its peers did not make is one call ahead in the per-workspace
    call counters (which pick buffer halves, flag banks and tags). Collective over the handle's
    group, host side: between two process-group barriers every rank zeroes its own pad of the handle
    and of every library workspace of that group, and the call counters are set to one common value
    above every rank's (so no tag is ever reused), after which all protocols start clean again."""
    pg = handle.group.pg
    torch.cuda.synchronize()
    if pg is not None:
        dist.barrier(group=pg)
    handle.get_signal_pad(handle.rank).zero_()
    dev_index = handle.get_signal_pad(handle.rank).device.index
    spaces = [h for (name, dev, _kind), h in sorted(_workspaces.items(), key=lambda kv: kv[0][2])
              if name == handle.group.name and dev == dev_index]
    for h in spaces:
        h.get_signal_pad(h.rank).zero_()
    counts = [int(getattr(h, attr, 0)) for h in spaces for attr in _CALL_COUNTERS]
    if counts:
        top = max(counts)
        if pg is not None:
            on_gpu = dist.get_backend(pg) == "nccl"
            t = torch.tensor([top], dtype=torch.int64, device=handle.get_signal_pad(handle.rank).device if on_gpu else "cpu")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=pg)
            top = int(t.item())
        for h in spaces:
            for attr in _CALL_COUNTERS:
                if hasattr(h, attr):
                    setattr(h, attr, top + 2)
    torch.cuda.synchronize()
    if pg is not None:
        dist.barrier(group=pg)
