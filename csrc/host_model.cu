// Host model of the signal-pad barrier protocol: the same slot layout and the same semaphore rules
// as symm_mem_sync in kraken/ptx_sync.cuh, executed by CPU processes on a region of shared memory
// (std::atomic on mmap'd words instead of .sys-scope PTX atomics on NVLink-mapped memory). It lets
// the protocol — including its failure behaviour: a rank that never arrives, a duplicated signal, a
// stale token — be exercised with ordinary processes and no GPU. The reference has no counterpart:
// its barrier (kraken/_ptx_utils/symm_mem_barrier.py:98-158) spins without bound.
//
// Layout: `base` points at ws pads of `pad_words` uint32 each; pad r belongs to rank r;
// slot(dst, block, src) = base[dst * pad_words + block * ws + src].
#include <atomic>
#include <chrono>
#include <thread>
#include "kraken/host.h"

namespace {
inline std::atomic<uint32_t>* slot(uint32_t* base, unsigned long long pad_words, int dst, int block, int ws, int src) {
  return reinterpret_cast<std::atomic<uint32_t>*>(base + (size_t)dst * pad_words + (size_t)block * ws + src);
}
}  // namespace

// One barrier of `rank` with all other ranks on barrier id `block`. Returns 0 when every peer's
// token arrived, else make_status(KR_ERR_TIMEOUT_SIGNAL, site 90, peer, block) for the first peer
// whose token did not arrive within timeout_ms (the tokens already received stay consumed, as on
// the device). skip_send: fault injection — wait without signalling (models a rank whose signal is
// lost); extra_sends: fault injection — signal that many additional times.
KR_API unsigned int kr_host_barrier(uint32_t* base, unsigned long long pad_words, int block, int rank, int ws,
                                    double timeout_ms, int skip_send, int extra_sends) {
  using clock = std::chrono::steady_clock;
  for (int rep = 0; rep < 1 + extra_sends; ++rep)
    if (!skip_send || rep > 0)
      for (int dst = 0; dst < ws; ++dst) slot(base, pad_words, dst, block, ws, rank)->fetch_add(1u, std::memory_order_release);
  const auto deadline = clock::now() + std::chrono::duration<double, std::milli>(timeout_ms);
  for (int src = 0; src < ws; ++src) {
    std::atomic<uint32_t>* s = slot(base, pad_words, rank, block, ws, src);
    unsigned spins = 0;
    while (s->load(std::memory_order_acquire) == 0u) {
      if ((++spins & 255u) == 0u) {
        if (clock::now() > deadline) return kraken::make_status(kraken::KR_ERR_TIMEOUT_SIGNAL, 90, (uint32_t)src, (uint32_t)block);
        std::this_thread::yield();
      }
    }
    s->fetch_sub(1u, std::memory_order_relaxed);   // consume one token
  }
  return 0u;
}

// Number of non-zero words in rank's pad (0 after any number of completed barriers).
KR_API unsigned long long kr_host_pad_nonzero(uint32_t* base, unsigned long long pad_words, int rank) {
  unsigned long long n = 0;
  for (unsigned long long i = 0; i < pad_words; ++i)
    if (reinterpret_cast<std::atomic<uint32_t>*>(base + (size_t)rank * pad_words + i)->load(std::memory_order_relaxed) != 0u) ++n;
  return n;
}
