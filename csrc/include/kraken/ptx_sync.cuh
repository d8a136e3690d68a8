// Device-side synchronisation primitives for symmetric-memory kernels (sm_100a).
//
// Covers the roles of the reference's kraken/_ptx_utils/symm_mem_barrier.py:54-158
// (send/wait signal, per-block cross-device barrier) and
// kraken/_ptx_utils/gmem_barrier_arrive_wait.py:6-69 (intra-GPU producer/consumer flag),
// re-designed so that no wait is unbounded: every spin carries a %globaltimer deadline.
// When a deadline passes the waiter records a code in a device status word and returns
// false; it never traps, so the CUDA context stays usable and the host can raise an error.
//
// Signal-pad slot layout is the reference's: pad[dst][block_id * world_size + src], uint32.
// The protocol differs: a slot is a counting semaphore. The sender adds 1 with a
// fire-and-forget `red.release.sys` (one NVLink crossing, no round trip); the receiver polls
// its OWN memory with `ld.acquire.sys` and then subtracts 1. Pads start zero-filled and are
// zero again after every completed barrier, so launches need no host-side epoch and replay
// under CUDA graphs. A CAS-style send (`send_signal_cas`) is kept for consumers that need a
// flag that is exactly 0/1 (stream memory operations on the host side).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

namespace kraken {

// Status codes written to SyncCtx::status[0] (first error wins).
enum : uint32_t {
  KR_OK = 0,
  KR_ERR_TIMEOUT_SIGNAL = 1,   // cross-device signal wait ran out
  KR_ERR_TIMEOUT_GMEM = 2,     // intra-GPU flag wait ran out
  KR_ERR_TIMEOUT_MBAR = 3,     // mbarrier (TMA / tcgen05 pipeline) wait ran out
  KR_ERR_BOUNDS = 4,           // debug bounds check failed
  KR_ERR_TIMEOUT_CAS = 5,      // CAS-style send could not find the slot free
};

// status word = code | site << 8 | peer << 16 | block << 24 (block truncated to 8 bits)
__host__ __device__ inline uint32_t make_status(uint32_t code, uint32_t site, uint32_t peer,
                                                uint32_t block) {
  return (code & 0xffu) | ((site & 0xffu) << 8) | ((peer & 0xffu) << 16) | ((block & 0xffu) << 24);
}

struct SyncCtx {
  uint32_t* status;      // device word(s) in THIS GPU's memory; status[0] sticky error
  uint64_t timeout_ns;   // deadline for every wait
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool status_ok(const SyncCtx& c) { return ld_volatile_u32(c.status) == 0; }

__device__ __forceinline__ void set_status(const SyncCtx& c, uint32_t word) {
  atomicCAS(c.status, 0u, word);
}

// ---- debug bounds checks -----------------------------------------------------------------------
// Compiled in with -DKRAKEN_DEBUG=1 (the library's debug build), compiled away otherwise. A failed
// check records KR_ERR_BOUNDS with its site in the status word and returns false; the caller then
// SKIPS the access, so a wrong index shows up as a host-side error, never as a memory fault.
#ifdef KRAKEN_DEBUG
__device__ __forceinline__ bool kr_in_bounds(bool ok, const SyncCtx& c, uint32_t site) {
  if (!ok) set_status(c, make_status(KR_ERR_BOUNDS, site, 0, blockIdx.x));
  return ok;
}
#else
__device__ __forceinline__ constexpr bool kr_in_bounds(bool, const SyncCtx&, uint32_t) { return true; }
#endif

// ---- raw memory-model operations -------------------------------------------------------------

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// 64-bit relaxed accesses at system scope: single-copy atomic, so a {value, tag} pair written with
// one store is seen whole by one load (the tagged push of the decode GEMM -> all-reduce).
__device__ __forceinline__ void st_relaxed_sys_u64(void* p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_u64(const void* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Two adjacent 64-bit words with one 16-byte request; each word by itself is read whole.
__device__ __forceinline__ void ld_relaxed_sys_u64x2(const void* p, unsigned long long& a, unsigned long long& b) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ void red_add_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_release_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.release.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_add_acqrel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_cas_release_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.release.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_cas_relaxed_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.relaxed.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_cas_acquire_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t atom_exch_release_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.release.gpu.global.exch.b32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// Orders generic-proxy accesses with async-proxy (TMA) accesses of the executing thread.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- bounded spinning ------------------------------------------------------------------------

// Polls `pred()` until it holds, the deadline passes, or another waiter already failed.
// Returns true when pred held. The clock is read every 32 polls.
template <class Pred>
__device__ __forceinline__ bool spin_until(Pred pred, const SyncCtx& c, uint32_t err_word) {
  if (pred()) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t n = 0;
  while (true) {
    if (pred()) return true;
    if ((++n & 31u) == 0u) {
      if (!status_ok(c)) return false;
      if (globaltimer_ns() - t0 > c.timeout_ns) {
        set_status(c, err_word);
        return false;
      }
    }
  }
}

// ---- cross-device signals (K1/K2 of the reference, semaphore form) ----------------------------

template <bool RELEASE>
__device__ __forceinline__ void send_signal(uint32_t* remote_slot) {
  if (RELEASE) red_add_release_sys(remote_slot, 1u);
  else red_add_relaxed_sys(remote_slot, 1u);
}

template <bool ACQUIRE>
__device__ __forceinline__ bool wait_signal(uint32_t* local_slot, const SyncCtx& c, uint32_t site,
                                            uint32_t peer, uint32_t block) {
  bool ok = spin_until(
      [&] { return (ACQUIRE ? ld_acquire_sys(local_slot) : ld_relaxed_sys(local_slot)) != 0u; }, c,
      make_status(KR_ERR_TIMEOUT_SIGNAL, site, peer, block));
  if (ok) red_add_relaxed_sys(local_slot, 0xffffffffu);   // consume one token
  return ok;
}

// CAS-style send: waits (bounded) for the slot to be 0, then sets it to 1. The reference's
// `send_signal(addrs, sem)` (symm_mem_barrier.py:54-72); used where the consumer is a
// stream memory operation that compares for equality with 1.
template <bool RELEASE>
__device__ __forceinline__ bool send_signal_cas(uint32_t* slot, const SyncCtx& c, uint32_t site,
                                                uint32_t peer) {
  return spin_until(
      [&] { return (RELEASE ? atom_cas_release_sys(slot, 0u, 1u) : atom_cas_relaxed_sys(slot, 0u, 1u)) == 0u; },
      c, make_status(KR_ERR_TIMEOUT_CAS, site, peer, 0));
}
// CAS-style wait: spins (bounded) until the slot is 1 and resets it to 0
// (symm_mem_barrier.py:76-94).
template <bool ACQUIRE>
__device__ __forceinline__ bool wait_signal_cas(uint32_t* slot, const SyncCtx& c, uint32_t site,
                                                uint32_t peer) {
  return spin_until(
      [&] { return (ACQUIRE ? atom_cas_acquire_sys(slot, 1u, 0u) : atom_cas_relaxed_sys(slot, 1u, 0u)) == 1u; },
      c, make_status(KR_ERR_TIMEOUT_SIGNAL, site, peer, 0));
}

// Per-block cross-device barrier (K3, symm_mem_barrier.py:98-158): blocks with the same
// `block_id` on all `ws` ranks meet. PREV: this block wrote symmetric memory that peers will
// read after the barrier (bar.sync + release). SUBSEQ: this block will read symmetric memory
// peers wrote before the barrier (acquire + bar.sync).
// Must be called by ALL threads of the block. Returns false (uniformly across the block when
// SUBSEQ) if any wait failed or the status word was already set.
template <bool PREV, bool SUBSEQ>
__device__ __forceinline__ bool symm_mem_sync(uint32_t* const* signal_pads, uint32_t block_id, int rank,
                                              int ws, const SyncCtx& c, uint32_t site = 0) {
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  if (PREV) __syncthreads();
  bool ok = true;
  if (tid < ws) {
    uint32_t* remote = signal_pads[tid] + (size_t)block_id * ws + rank;
    uint32_t* local = signal_pads[rank] + (size_t)block_id * ws + tid;
    send_signal<PREV>(remote);
    ok = wait_signal<SUBSEQ>(local, c, site, (uint32_t)tid, block_id);
  }
  if (SUBSEQ) {
    __syncthreads();
    return status_ok(c);
  }
  return ok;
}

// ---- intra-GPU producer/consumer flags (K4/K5) -----------------------------------------------

// All threads call; thread 0 publishes after the block's prior writes (bar.sync + release).
__device__ __forceinline__ void arrive_gmem_barrier(uint32_t* addr, uint32_t update = 1u,
                                                    bool skip_sync = false) {
  if (!skip_sync) __syncthreads();
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  if (tid == 0) atom_exch_release_gpu(addr, update);
}
// All threads call; thread 0 spins (bounded) until *addr == expect, then bar.sync.
template <bool SYS_SCOPE = false>
__device__ __forceinline__ bool wait_gmem_barrier(const uint32_t* addr, uint32_t expect, const SyncCtx& c,
                                                  uint32_t site = 0, bool skip_sync = false) {
  const int tid = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  if (tid == 0) {
    spin_until([&] { return (SYS_SCOPE ? ld_acquire_sys(addr) : ld_acquire_gpu(addr)) == expect; }, c,
               make_status(KR_ERR_TIMEOUT_GMEM, site, 0, blockIdx.x));
  }
  if (!skip_sync) __syncthreads();
  return status_ok(c);
}
// Single-thread form for warp-specialised kernels (the caller handles intra-CTA ordering).
__device__ __forceinline__ bool wait_flag_acquire_gpu(const uint32_t* addr, uint32_t at_least,
                                                      const SyncCtx& c, uint32_t site) {
  return spin_until([&] { return ld_acquire_gpu(addr) >= at_least; }, c,
                    make_status(KR_ERR_TIMEOUT_GMEM, site, 0, blockIdx.x));
}
__device__ __forceinline__ bool wait_flag_acquire_sys(const uint32_t* addr, uint32_t at_least,
                                                      const SyncCtx& c, uint32_t site) {
  return spin_until([&] { return ld_acquire_sys(addr) >= at_least; }, c,
                    make_status(KR_ERR_TIMEOUT_SIGNAL, site, 0, blockIdx.x));
}

}  // namespace kraken
