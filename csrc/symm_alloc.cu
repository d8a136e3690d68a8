// Symmetric-memory allocator over the CUDA virtual-memory API, plus the unix-socket channel that
// passes allocation handles (file descriptors) between the ranks of one node.
//
// One allocation = one physical cuMemCreate block laid out as [ data | signal pad ], exported as a
// POSIX fd, imported and mapped by every peer, and optionally bound to an NVLS multicast object.
// It provides what the reference takes from torch.distributed._symmetric_memory
// (empty/rendezvous, buffer_ptrs_dev, signal_pad_ptrs_dev, multicast_ptr; used e.g. at
// kraken/comm/one_shot_all_reduce.py:89-97 and kraken/comm/two_shot_all_reduce.py:124-141).
// Ranks order the steps (export -> exchange -> import -> finalize) with their process group;
// this file holds no cross-process protocol beyond "send one fd" / "receive one fd".
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <sys/socket.h>
#include <sys/un.h>
#include <poll.h>
#include <unistd.h>
#include "kraken/driver_api.h"

namespace kraken {

static std::mutex g_drv_mu;
static std::map<std::string, void*> g_drv;

void* driver_entry(const char* raw_name) {
  // cuda.h renames some entry points with macros (cuStreamWriteValue32 -> cuStreamWriteValue32_v2);
  // the runtime's lookup wants the base name and picks the version itself.
  std::string base(raw_name);
  for (const char* suffix : {"_v2", "_v3", "_ptsz"}) {
    const size_t n = strlen(suffix);
    if (base.size() > n && base.compare(base.size() - n, n, suffix) == 0) base.resize(base.size() - n);
  }
  const char* name = base.c_str();
  std::lock_guard<std::mutex> lk(g_drv_mu);
  auto it = g_drv.find(base);
  if (it != g_drv.end()) return it->second;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess) {
    fn = nullptr;
    (void)cudaGetLastError();
  }
  g_drv[base] = fn;
  return fn;
}

std::string cu_error_string(CUresult r) {
  auto fn = KR_DRV_FN(cuGetErrorString);
  const char* s = nullptr;
  if (fn && fn(r, &s) == CUDA_SUCCESS && s) return std::string(s) + " (" + std::to_string((int)r) + ")";
  return "CUresult " + std::to_string((int)r);
}

struct SymmAlloc {
  int device = 0;
  int rank = -1, ws = 0;
  size_t data_bytes = 0;    // offset of the signal pad
  size_t pad_bytes = 0;
  size_t total = 0;         // mapped size (granularity multiple)
  CUmemGenericAllocationHandle local_handle = 0;
  CUdeviceptr local_ptr = 0;
  std::vector<CUmemGenericAllocationHandle> peer_handles;   // imported (0 for self)
  std::vector<CUdeviceptr> ptrs;                            // per-rank mapped base
  void** bufs_dev = nullptr;       // device array [ws]
  uint32_t** pads_dev = nullptr;   // device array [ws]
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_ptr = 0;
  bool mc_bound = false;
};

static size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int mem_prop(CUmemAllocationProp* prop, int device) {
  memset(prop, 0, sizeof(*prop));
  prop->type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop->location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop->location.id = device;
  prop->requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return 0;
}

static int map_rw(CUdeviceptr* out, CUmemGenericAllocationHandle h, size_t total, size_t gran, int device) {
  CUdeviceptr va = 0;
  KR_CU(cuMemAddressReserve, &va, total, gran, 0, 0);
  KR_CU(cuMemMap, va, total, 0, h, 0);
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  KR_CU(cuMemSetAccess, va, total, &acc, 1);
  *out = va;
  return KR_SUCCESS;
}

static int multicast_supported(int device) {
  int v = 0;
  auto fn = KR_DRV_FN(cuDeviceGetAttribute);
  if (!fn) return 0;
  if (fn(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != CUDA_SUCCESS) return 0;
  return v;
}

}  // namespace kraken

using namespace kraken;

// ---- allocation -------------------------------------------------------------------------------

// Answered once per device and cached: ops ask on every call, also while a stream is being captured,
// when nothing that touches the context (cudaFree) may run.
KR_API int kr_symm_multicast_supported() {
  static std::mutex mu;
  static int cached[64];
  static bool init = false;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  std::lock_guard<std::mutex> lk(mu);
  if (!init) {
    for (int& c : cached) c = -1;
    init = true;
  }
  if (dev < 0 || dev >= 64) return 0;
  if (cached[dev] < 0) {
    (void)cudaFree(0);   // make sure the primary context exists
    cached[dev] = multicast_supported(dev) ? 1 : 0;
  }
  return cached[dev];
}

// Creates this rank's block: `bytes` of data followed by `pad_bytes` of signal pad, all zeroed. The
// block is usable locally at once; kr_symm_set_group + import + finalize make it symmetric.
KR_API int kr_symm_alloc(unsigned long long bytes, unsigned long long pad_bytes, void** out) {
  KR_REQUIRE(pad_bytes % 16 == 0, "signal pad size must be a multiple of 16");
  KR_CUDA(cudaFree(0));   // make sure the primary context exists
  auto* a = new SymmAlloc();
  KR_CUDA(cudaGetDevice(&a->device));
  int ndev = 1;
  KR_CUDA(cudaGetDeviceCount(&ndev));
  const int ws = ndev > 1 ? ndev : 1;
  a->data_bytes = round_up(bytes ? bytes : 16, 4096);
  a->pad_bytes = pad_bytes;
  CUmemAllocationProp prop;
  mem_prop(&prop, a->device);
  size_t gran = 0;
  KR_CU(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  if (ws > 1 && multicast_supported(a->device)) {
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = ws;
    mp.size = round_up(a->data_bytes + a->pad_bytes, gran);
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t mgran = 0;
    auto fn = KR_DRV_FN(cuMulticastGetGranularity);
    if (fn && fn(&mgran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran > gran) gran = mgran;
  }
  a->total = round_up(a->data_bytes + a->pad_bytes, gran);
  KR_CU(cuMemCreate, &a->local_handle, a->total, &prop, 0);
  CUdeviceptr va = 0;
  int rc = map_rw(&va, a->local_handle, a->total, gran, a->device);
  if (rc) return rc;
  a->local_ptr = va;
  // The whole block starts out zero: the signal pad has to, and ops that tag their data (the decode
  // GEMM -> all-reduce's tagged push) rely on never meeting a stale tag in fresh memory. No peer can
  // have written yet: the block is not shared before the exchange that follows.
  KR_CUDA(cudaMemset((void*)va, 0, a->total));
  KR_CUDA(cudaDeviceSynchronize());
  *out = a;
  return KR_SUCCESS;
}

KR_API void* kr_symm_local_ptr(void* h) { return (void*)((SymmAlloc*)h)->local_ptr; }

// Declares which rank of which world size this block is; peers can be imported afterwards.
KR_API int kr_symm_set_group(void* h, int rank, int ws) {
  auto* a = (SymmAlloc*)h;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(a->ws == 0, "block already belongs to a group");
  a->rank = rank;
  a->ws = ws;
  a->peer_handles.assign(ws, 0);
  a->ptrs.assign(ws, 0);
  a->ptrs[rank] = a->local_ptr;
  return KR_SUCCESS;
}

KR_API unsigned long long kr_symm_total_bytes(void* h) { return ((SymmAlloc*)h)->total; }
KR_API unsigned long long kr_symm_data_bytes(void* h) { return ((SymmAlloc*)h)->data_bytes; }
KR_API unsigned long long kr_symm_pad_bytes(void* h) { return ((SymmAlloc*)h)->pad_bytes; }

// Exports the local block as a file descriptor the caller must close after sending it.
KR_API int kr_symm_export_fd(void* h, int* fd_out) {
  auto* a = (SymmAlloc*)h;
  int fd = -1;
  KR_CU(cuMemExportToShareableHandle, (void*)&fd, a->local_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  *fd_out = fd;
  return KR_SUCCESS;
}

// Maps the block of `peer` (received as `fd`; the fd is closed here).
KR_API int kr_symm_import_fd(void* h, int peer, int fd) {
  auto* a = (SymmAlloc*)h;
  KR_REQUIRE(peer >= 0 && peer < a->ws && peer != a->rank, "bad peer rank");
  KR_REQUIRE(a->ptrs[peer] == 0, "peer already imported");
  CUmemGenericAllocationHandle ph = 0;
  KR_CU(cuMemImportFromShareableHandle, &ph, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  CUmemAllocationProp prop;
  mem_prop(&prop, a->device);
  size_t gran = 0;
  KR_CU(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  CUdeviceptr va = 0;
  int rc = map_rw(&va, ph, a->total, gran, a->device);
  if (rc) return rc;
  a->peer_handles[peer] = ph;
  a->ptrs[peer] = va;
  return KR_SUCCESS;
}

// After every peer is imported: builds the device pointer tables.
KR_API int kr_symm_finalize(void* h) {
  auto* a = (SymmAlloc*)h;
  std::vector<void*> bufs(a->ws);
  std::vector<uint32_t*> pads(a->ws);
  for (int r = 0; r < a->ws; ++r) {
    KR_REQUIRE(a->ptrs[r] != 0, "finalize before all peers were imported");
    bufs[r] = (void*)a->ptrs[r];
    pads[r] = (uint32_t*)(a->ptrs[r] + a->data_bytes);
  }
  KR_CUDA(cudaMalloc(&a->bufs_dev, sizeof(void*) * a->ws));
  KR_CUDA(cudaMalloc(&a->pads_dev, sizeof(void*) * a->ws));
  KR_CUDA(cudaMemcpy(a->bufs_dev, bufs.data(), sizeof(void*) * a->ws, cudaMemcpyHostToDevice));
  KR_CUDA(cudaMemcpy(a->pads_dev, pads.data(), sizeof(void*) * a->ws, cudaMemcpyHostToDevice));
  return KR_SUCCESS;
}

KR_API void* kr_symm_ptr(void* h, int rank) {
  auto* a = (SymmAlloc*)h;
  return (rank >= 0 && rank < a->ws) ? (void*)a->ptrs[rank] : nullptr;
}
KR_API void* kr_symm_pad_ptr(void* h, int rank) {
  auto* a = (SymmAlloc*)h;
  return (rank >= 0 && rank < a->ws && a->ptrs[rank]) ? (void*)(a->ptrs[rank] + a->data_bytes) : nullptr;
}
KR_API void* kr_symm_bufs_dev(void* h) { return ((SymmAlloc*)h)->bufs_dev; }
KR_API void* kr_symm_pads_dev(void* h) { return ((SymmAlloc*)h)->pads_dev; }
KR_API void* kr_symm_mc_ptr(void* h) { return ((SymmAlloc*)h)->mc_bound ? (void*)((SymmAlloc*)h)->mc_ptr : nullptr; }

// ---- NVLS multicast: rank 0 creates + exports; all ranks attach (add device), then — after a
//      process-group barrier — bind their block and map the multicast address.
KR_API int kr_symm_mc_create(void* h, int* fd_out) {
  auto* a = (SymmAlloc*)h;
  KR_REQUIRE(multicast_supported(a->device), "multicast not supported on this device");
  CUmulticastObjectProp mp;
  memset(&mp, 0, sizeof(mp));
  mp.numDevices = a->ws;
  mp.size = a->total;
  mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  KR_CU(cuMulticastCreate, &a->mc_handle, &mp);
  int fd = -1;
  KR_CU(cuMemExportToShareableHandle, (void*)&fd, a->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  *fd_out = fd;
  return KR_SUCCESS;
}
KR_API int kr_symm_mc_import(void* h, int fd) {
  auto* a = (SymmAlloc*)h;
  KR_CU(cuMemImportFromShareableHandle, &a->mc_handle, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  close(fd);
  return KR_SUCCESS;
}
KR_API int kr_symm_mc_add_device(void* h) {
  auto* a = (SymmAlloc*)h;
  KR_REQUIRE(a->mc_handle != 0, "no multicast object");
  KR_CU(cuMulticastAddDevice, a->mc_handle, a->device);
  return KR_SUCCESS;
}
KR_API int kr_symm_mc_bind(void* h) {
  auto* a = (SymmAlloc*)h;
  KR_REQUIRE(a->mc_handle != 0, "no multicast object");
  KR_CU(cuMulticastBindMem, a->mc_handle, 0, a->local_handle, 0, a->total, 0);
  CUmemAllocationProp prop;
  mem_prop(&prop, a->device);
  size_t gran = 0;
  KR_CU(cuMemGetAllocationGranularity, &gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
  CUdeviceptr va = 0;
  int rc = map_rw(&va, a->mc_handle, a->total, gran, a->device);
  if (rc) return rc;
  a->mc_ptr = va;
  a->mc_bound = true;
  return KR_SUCCESS;
}

// Unmaps and releases everything. Every rank must have stopped using the block (host barrier).
KR_API int kr_symm_free(void* h) {
  auto* a = (SymmAlloc*)h;
  if (!a) return KR_SUCCESS;
  (void)cudaDeviceSynchronize();
  auto unmap = KR_DRV_FN(cuMemUnmap);
  auto rel = KR_DRV_FN(cuMemRelease);
  auto afree = KR_DRV_FN(cuMemAddressFree);
  auto unbind = KR_DRV_FN(cuMulticastUnbind);
  if (unmap && rel && afree) {
    if (a->mc_bound) {
      unmap(a->mc_ptr, a->total);
      afree(a->mc_ptr, a->total);
      if (unbind) unbind(a->mc_handle, a->device, 0, a->total);
    }
    if (a->mc_handle) rel(a->mc_handle);
    for (int r = 0; r < a->ws; ++r) {
      if (!a->ptrs[r] || r == a->rank) continue;
      unmap(a->ptrs[r], a->total);
      afree(a->ptrs[r], a->total);
      if (a->peer_handles[r]) rel(a->peer_handles[r]);
    }
    unmap(a->local_ptr, a->total);
    afree(a->local_ptr, a->total);
    rel(a->local_handle);
  }
  if (a->bufs_dev) cudaFree(a->bufs_dev);
  if (a->pads_dev) cudaFree(a->pads_dev);
  delete a;
  return KR_SUCCESS;
}

// ---- fd passing over unix datagram sockets ------------------------------------------------------

static int make_addr(const char* path, sockaddr_un* addr, socklen_t* len) {
  memset(addr, 0, sizeof(*addr));
  addr->sun_family = AF_UNIX;
  size_t n = strlen(path);
  if (n == 0 || n >= sizeof(addr->sun_path) - 1) return -1;
  // abstract namespace (leading NUL): no file to clean up, private to the network namespace
  memcpy(addr->sun_path + 1, path, n);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
  return 0;
}

KR_API int kr_ipc_open(const char* name, int* sock_out) {
  int s = socket(AF_UNIX, SOCK_DGRAM, 0);
  if (s < 0) return fail(KR_FAIL_STATE, std::string("socket: ") + strerror(errno));
  sockaddr_un addr;
  socklen_t len;
  if (make_addr(name, &addr, &len)) {
    close(s);
    return fail(KR_FAIL_ARG, "bad socket name");
  }
  if (bind(s, (sockaddr*)&addr, len) != 0) {
    std::string m = std::string("bind: ") + strerror(errno);
    close(s);
    return fail(KR_FAIL_STATE, m);
  }
  *sock_out = s;
  return KR_SUCCESS;
}
KR_API int kr_ipc_close(int sock) {
  close(sock);
  return KR_SUCCESS;
}
// Sends `fd` with a 4-byte tag (the sender's rank) to the socket bound at `dst_name`.
KR_API int kr_ipc_send_fd(int sock, const char* dst_name, int fd, int tag) {
  sockaddr_un addr;
  socklen_t len;
  if (make_addr(dst_name, &addr, &len)) return fail(KR_FAIL_ARG, "bad socket name");
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  iovec iov;
  iov.iov_base = &tag;
  iov.iov_len = sizeof(tag);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_name = &addr;
  msg.msg_namelen = len;
  char cbuf[CMSG_SPACE(sizeof(int))];
  memset(cbuf, 0, sizeof(cbuf));
  msg.msg_control = cbuf;
  msg.msg_controllen = sizeof(cbuf);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (int attempt = 0; attempt < 200; ++attempt) {
    if (sendmsg(sock, &msg, 0) >= 0) return KR_SUCCESS;
    if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN) break;
    usleep(20000);   // receiver not bound yet
  }
  return fail(KR_FAIL_STATE, std::string("sendmsg: ") + strerror(errno));
}
// Receives one fd and its tag; gives up after timeout_ms.
KR_API int kr_ipc_recv_fd(int sock, int timeout_ms, int* fd_out, int* tag_out) {
  pollfd pfd;
  pfd.fd = sock;
  pfd.events = POLLIN;
  int pr = poll(&pfd, 1, timeout_ms);
  if (pr == 0) return fail(KR_FAIL_STATE, "timed out waiting for a peer's memory handle");
  if (pr < 0) return fail(KR_FAIL_STATE, std::string("poll: ") + strerror(errno));
  msghdr msg;
  memset(&msg, 0, sizeof(msg));
  int tag = -1;
  iovec iov;
  iov.iov_base = &tag;
  iov.iov_len = sizeof(tag);
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char cbuf[CMSG_SPACE(sizeof(int))];
  msg.msg_control = cbuf;
  msg.msg_controllen = sizeof(cbuf);
  if (recvmsg(sock, &msg, 0) < 0) return fail(KR_FAIL_STATE, std::string("recvmsg: ") + strerror(errno));
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS)
    return fail(KR_FAIL_STATE, "message carried no file descriptor");
  int fd = -1;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  *fd_out = fd;
  *tag_out = tag;
  return KR_SUCCESS;
}

// ---- stream memory operations and copy-engine collectives ---------------------------------------

KR_API int kr_stream_write_value32(cudaStream_t stream, void* addr, uint32_t value) {
  KR_CU(cuStreamWriteValue32, (CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WRITE_VALUE_DEFAULT);
  return KR_SUCCESS;
}
KR_API int kr_stream_wait_value32(cudaStream_t stream, void* addr, uint32_t value) {
  KR_CU(cuStreamWaitValue32, (CUstream)stream, (CUdeviceptr)addr, value, CU_STREAM_WAIT_VALUE_EQ);
  return KR_SUCCESS;
}

// Copy-engine all-gather with progress flags (reference: copy_engine_all_gather.py:40-54):
// on `stream`, for step, split: output chunk[src*S+split] <- peer shard slice, then
// progress[src*S+split] = 1 by a stream memory operation. src = (rank+step+1) % ws.
KR_API int kr_ce_all_gather(void* const* shard_ptrs_host, int rank, int ws, void* output, uint32_t* progress,
                            int splits, unsigned long long shard_bytes, cudaStream_t stream) {
  KR_REQUIRE(splits >= 1 && shard_bytes % (unsigned long long)splits == 0, "shard must divide into splits");
  const size_t chunk = shard_bytes / splits;
  for (int step = 0; step < ws; ++step) {
    const int src = (rank + step + 1) % ws;
    for (int sp = 0; sp < splits; ++sp) {
      const int idx = src * splits + sp;
      KR_CUDA(cudaMemcpyAsync((char*)output + (size_t)idx * chunk, (const char*)shard_ptrs_host[src] + (size_t)sp * chunk,
                              chunk, cudaMemcpyDeviceToDevice, stream));
      if (progress) KR_CU(cuStreamWriteValue32, (CUstream)stream, (CUdeviceptr)(progress + idx), 1u,
                          CU_STREAM_WRITE_VALUE_DEFAULT);
    }
  }
  return KR_SUCCESS;
}

// Copy-engine scatter of GEMM output slabs (reference: gemm_reduce_scatter_ce_persistent.py:137-175):
// for step: wait until signals[remote] == 1, then copy slab `remote` of gemm_out into the slot
// `rank` of remote's workspace.
KR_API int kr_ce_scatter_slabs(void* const* workspace_ptrs_host, int rank, int ws, const void* gemm_out,
                               uint32_t* signals, unsigned long long slab_bytes, cudaStream_t stream) {
  for (int step = 0; step < ws; ++step) {
    const int remote = (rank + step + 1) % ws;
    if (signals) KR_CU(cuStreamWaitValue32, (CUstream)stream, (CUdeviceptr)(signals + remote), 1u, CU_STREAM_WAIT_VALUE_EQ);
    KR_CUDA(cudaMemcpyAsync((char*)workspace_ptrs_host[remote] + (size_t)rank * slab_bytes,
                            (const char*)gemm_out + (size_t)remote * slab_bytes, slab_bytes,
                            cudaMemcpyDeviceToDevice, stream));
  }
  return KR_SUCCESS;
}
