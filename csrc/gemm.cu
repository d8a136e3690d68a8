// tcgen05 GEMM kernels: the plain GEMM, the fused all-gather -> GEMM and the producer GEMM of the
// copy-engine reduce-scatter, plus the host-side pieces every GEMM translation unit shares (tensor-map
// cache, operand set-up, tile-order defaults). The reduce-scatter GEMMs live in gemm_rs.cu, the
// decode GEMM -> all-reduce in gemm_ar.cu, the tf32 kernels in gemm_tf32.cu.
//
//  * all-gather -> GEMM (reference: kraken/fused/all_gather_matmul.py:222-325): comm CTAs of the
//    same launch move the shards (push: the own shard into every peer's gathered buffer with posted
//    bulk stores; pull: the peers' shards into the local one) and raise per-chunk flags; the MMA
//    CTAs start on the local shard (rank pivot) and consume remote chunks as their flags appear.
//    One launch, no copy engine, no second stream. A copy-engine feed is available as well.
//  * copy-engine reduce-scatter producer (reference: gemm_reduce_scatter_ce_persistent.py:46-134).
#include <deque>
#include <map>
#include <mutex>
#include <tuple>
#include "kraken/gemm_host.h"
#include "kraken/gemm_hooks.cuh"

namespace kraken {

// ---------------------------------------------------------------------------------------------
// hooks
// ---------------------------------------------------------------------------------------------
struct AgHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  // Row tile tr covers gathered rows [tr*128, +128). Rows of the own shard come from the own
  // shard's tensor map at once; other rows wait until every chunk they touch has landed.
  __device__ __forceinline__ bool before_load(const GemmParams& p, int tr, const CUtensorMap*& rmap, int& row0) {
    const int lo = tr * kBM;
    if (lo >= p.rows_r) return true;           // padding tile of a CTA pair: nothing to wait for
    const int hi = min(lo + kBM, p.rows_r) - 1;
    const int own_lo = p.rank * p.shard_rows;
    if (lo >= own_lo && hi < own_lo + p.shard_rows) {
      rmap = &p.tmap_r_local;
      row0 = lo - own_lo;
      return true;
    }
    const int c_lo = lo / p.chunk_rows, c_hi = hi / p.chunk_rows;
    for (int c = c_lo; c <= c_hi; ++c) {
      // push: the chunk's owner raises a flag in this rank's signal pad; else a local engine sets progress
      const bool ok = p.ag_push ? wait_flag_acquire_sys(p.pads[p.rank] + p.flag_base + c, 1u, p.sync, 50)
                                : wait_flag_acquire_gpu(p.progress + c, 1u, p.sync, 50);
      if (!ok) return false;
    }
    fence_proxy_async();   // chunk was written through another proxy / by other CTAs or another GPU
    return true;
  }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols, p.use_tma_store ? &p.tmap_out[0] : nullptr};
  }
  __device__ __forceinline__ bool after_store(const GemmParams&, int, int, int, int) { return true; }
};

// Producer GEMM of the copy-engine reduce-scatter variant
// (reference: gemm_reduce_scatter_ce_persistent.py:46-134): tiles go to the local gemm_out; a
// per-destination counter tracks finished tiles and the tile that completes a slab raises that
// slab's signal word to 1 with system-scope release, which a stream wait on the host side consumes.
struct CeHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols, p.use_tma_store ? &p.tmap_out[0] : nullptr};
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    epi_bar_sync();
    if (q == 0 && lane == 0) {
      const int dst = (tr * kBM) / p.slab_rows;
      const uint32_t per_slab = (uint32_t)(p.slab_rows / kBM) * (uint32_t)p.tiles_c;
      const uint32_t old = atom_add_acqrel_gpu(p.counters + dst, 1u);
      if (old == per_slab - 1) {
        p.counters[dst] = 0;
        st_release_sys(p.progress + dst, 1u);
      }
    }
    return true;
  }
};

// ---------------------------------------------------------------------------------------------
// AG comm CTAs: one elected thread moves chunks peer -> shared -> local with bulk async copies.
// ---------------------------------------------------------------------------------------------
constexpr int kAgPiece = 16384;   // bytes per bulk copy
constexpr int kAgSlots = 12;      // ring depth (192 KB of shared memory in flight)

__device__ __forceinline__ void ag_comm_cta(const GemmParams& p, unsigned comm_id, unsigned n_comm,
                                            unsigned char* smem_raw) {
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kAgSlots * kAgPiece;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgSlots; ++s) mbar_init(bars + 8u * s, 1);
    mbar_fence_init();
  }
  // peers' shards must be complete (written by earlier kernels on their streams)
  if (!symm_mem_sync<false, true>(p.pads, p.pad_base / p.ws + comm_id, p.rank, p.ws, p.sync, 52)) return;
  if (threadIdx.x == 0) {
    const size_t row_bytes = (size_t)p.K * 2;
    const size_t chunk_bytes = (size_t)p.chunk_rows * row_bytes;
    const size_t pieces = (chunk_bytes + kAgPiece - 1) / kAgPiece;
    uint32_t issued = 0, stored = 0;   // global piece counters over the ring
    bool ok = true;
    for (int step = 0; step < p.ws && ok; ++step) {
      const int src = (p.rank + step + 1) % p.ws;
      for (int sp = 0; sp < p.splits && ok; ++sp) {
        const int idx = src * p.splits + sp;
        const char* from = (const char*)p.bufs[src] + (size_t)sp * chunk_bytes;
        char* to = (char*)p.a_out + (size_t)idx * chunk_bytes;
        // my pieces of this chunk: comm_id, comm_id + n_comm, ...
        size_t next_load = comm_id, next_store = comm_id;
        while (next_store < pieces && ok) {
          // keep the ring full
          // at most kAgSlots-2 loads are ahead of the stores, so the store that last read this
          // slot has at least two younger bulk groups behind it
          while (next_load < pieces && issued - stored < (uint32_t)(kAgSlots - 2)) {
            const uint32_t slot = issued % kAgSlots;
            if (issued >= (uint32_t)kAgSlots) bulk_wait_group_read<2>();
            const size_t off = next_load * kAgPiece;
            const uint32_t bytes = (uint32_t)min((size_t)kAgPiece, chunk_bytes - off);
            mbar_expect_tx(bars + 8u * slot, bytes);
            bulk_load_1d(base + slot * kAgPiece, from + off, bytes, bars + 8u * slot);
            ++issued;
            next_load += n_comm;
          }
          const uint32_t slot = stored % kAgSlots;
          ok = mbar_wait(bars + 8u * slot, (stored / kAgSlots) & 1u, p.sync, 53);
          if (!ok) break;
          const size_t off = next_store * kAgPiece;
          const uint32_t bytes = (uint32_t)min((size_t)kAgPiece, chunk_bytes - off);
          fence_proxy_async();
          bulk_store_1d(to + off, base + slot * kAgPiece, bytes);
          bulk_commit_group();
          ++stored;
          next_store += n_comm;
        }
        // chunk boundary: my stores must be complete and visible before I count myself in
        bulk_wait_group<0>();
        fence_proxy_async();
        const uint32_t old = atom_add_acqrel_gpu(p.counters + idx, 1u);
        if (old == n_comm - 1) {
          p.counters[idx] = 0;
          st_release_gpu(p.progress + idx, 1u);
        }
      }
    }
    bulk_wait_group<0>();
  }
  // peers may overwrite their shards only after every rank finished pulling
  symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + comm_id, p.rank, p.ws, p.sync, 54);
}

// ---------------------------------------------------------------------------------------------
// AG push engine: every rank writes its OWN shard into every peer's gathered buffer (local bulk
// load -> shared memory -> bulk store to the peer: posted NVLink writes, no remote round trip) and
// then raises the chunk's flag in that peer's signal pad. Destinations are served in the order
// rank-1, rank-2, ...: a destination computes on the shards of rank+1, rank+2, ... in that order,
// so each shard travels at full link rate exactly when it is needed next. The own copy goes last.
// Flags live in two banks used alternately call by call and are put back to zero by the last CTA
// of the launch; with the library's double-buffered gathered buffer no barrier is needed at all.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ag_push_cta(const GemmParams& p, unsigned comm_id, unsigned n_comm,
                                            unsigned char* smem_raw) {
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + kAgSlots * kAgPiece;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgSlots; ++s) mbar_init(bars + 8u * s, 1);
    mbar_fence_init();
  }
  // A caller-owned gathered buffer may still be read by a slower peer's previous consumer.
  if (p.ag_entry_barrier && !symm_mem_sync<true, true>(p.pads, p.pad_base / p.ws + comm_id, p.rank, p.ws, p.sync, 52)) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    const size_t row_bytes = (size_t)p.K * 2;
    const size_t chunk_bytes = (size_t)p.chunk_rows * row_bytes;
    const size_t pieces = (chunk_bytes + kAgPiece - 1) / kAgPiece;
    const char* shard = (const char*)p.ag_shard;
    uint32_t issued = 0, stored = 0;   // piece counters over the ring
    bool ok = true;
    for (int step = 0; step < p.ws && ok; ++step) {
      int dst = p.rank - 1 - step;
      while (dst < 0) dst += p.ws;                       // ..., rank itself last
      for (int sp = 0; sp < p.splits && ok; ++sp) {
        const int idx = p.rank * p.splits + sp;
        const char* from = shard + (size_t)sp * chunk_bytes;
        char* to = (char*)p.bufs[dst] + p.ag_out_off + (size_t)idx * chunk_bytes;
        size_t next_load = comm_id, next_store = comm_id;
        while (next_store < pieces && ok) {
          while (next_load < pieces && issued - stored < (uint32_t)(kAgSlots - 2)) {
            const uint32_t slot = issued % kAgSlots;
            if (issued >= (uint32_t)kAgSlots) bulk_wait_group_read<2>();
            const size_t off = next_load * kAgPiece;
            const uint32_t bytes = (uint32_t)min((size_t)kAgPiece, chunk_bytes - off);
            mbar_expect_tx(bars + 8u * slot, bytes);
            bulk_load_1d(base + slot * kAgPiece, from + off, bytes, bars + 8u * slot);
            ++issued;
            next_load += n_comm;
          }
          const uint32_t slot = stored % kAgSlots;
          ok = mbar_wait(bars + 8u * slot, (stored / kAgSlots) & 1u, p.sync, 53);
          if (!ok) break;
          const size_t off = next_store * kAgPiece;
          const uint32_t bytes = (uint32_t)min((size_t)kAgPiece, chunk_bytes - off);
          fence_proxy_async();
          if (kr_in_bounds(idx < p.ws * p.splits && off + bytes <= chunk_bytes && dst >= 0 && dst < p.ws, p.sync, 72))
            bulk_store_1d(to + off, base + slot * kAgPiece, bytes);
          bulk_commit_group();
          ++stored;
          next_store += n_comm;
        }
        if (!ok) break;
        // my pieces of this chunk are at the destination before I count myself in; the comm CTA
        // that completes the chunk tells the destination
        bulk_wait_group<0>();
        fence_proxy_async();
        uint32_t* cnt = p.counters + (size_t)dst * p.splits + sp;
        const uint32_t old = atom_add_acqrel_gpu(cnt, 1u);
        if (old == n_comm - 1) {
          *cnt = 0;
          red_add_release_sys(p.pads[dst] + p.flag_base + idx, 1u);
        }
      }
    }
    bulk_wait_group<0>();
    // the caller's progress words: in the order the chunks arrive here
    if (comm_id == 0 && p.progress != nullptr) {
      for (int step = 1; step <= p.ws && ok; ++step) {
        const int src = (p.rank + step) % p.ws;
        for (int sp = 0; sp < p.splits && ok; ++sp) {
          const int idx = src * p.splits + sp;
          ok = wait_flag_acquire_sys(p.pads[p.rank] + p.flag_base + idx, 1u, p.sync, 54);
          if (ok) st_release_gpu(p.progress + idx, 1u);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// AG multicast push engine: every rank writes its own shard ONCE, to the multicast address of the
// gathered buffer; the NVSwitch delivers it to all ranks (this one included). One elected thread
// streams the shard local memory -> shared memory with bulk loads; all threads of the comm CTA
// forward each landed piece with multimem.st (posted, from registers, so shared memory only holds
// data on its way in). A finished chunk's flag is raised on every rank with one multimem.red.
// NVLink bytes out per rank: one shard instead of ws - 1 of them.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ag_mc_cta(const GemmParams& p, unsigned comm_id, unsigned n_comm,
                                          unsigned char* smem_raw) {
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kAgSlots * kAgPiece;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgSlots; ++s) mbar_init(bars + 8u * s, 1);
    mbar_fence_init();
  }
  if (p.ag_entry_barrier && !symm_mem_sync<true, true>(p.pads, p.pad_base / p.ws + comm_id, p.rank, p.ws, p.sync, 52)) return;
  __syncthreads();
  const size_t row_bytes = (size_t)p.K * 2;
  const size_t chunk_bytes = (size_t)p.chunk_rows * row_bytes;
  const size_t pieces = (chunk_bytes + kAgPiece - 1) / kAgPiece;            // per chunk
  const size_t mine_per_chunk = pieces > comm_id ? (pieces - comm_id + n_comm - 1) / n_comm : 0;
  const size_t total_mine = mine_per_chunk * (size_t)p.splits;
  const char* shard = (const char*)p.ag_shard;
  char* mc_out = (char*)p.ag_mc_out + (size_t)p.rank * p.splits * chunk_bytes;   // this rank's rows in every gathered buffer
  // j-th piece of this CTA: chunk j / mine_per_chunk, piece comm_id + (j % mine_per_chunk) * n_comm
  auto piece_off = [&](size_t j, uint32_t& bytes) -> size_t {
    const size_t sp = j / mine_per_chunk, pc = comm_id + (j - sp * mine_per_chunk) * n_comm;
    const size_t off = pc * kAgPiece;
    bytes = (uint32_t)min((size_t)kAgPiece, chunk_bytes - off);
    return sp * chunk_bytes + off;
  };
  if (threadIdx.x == 0) {
    for (size_t j = 0; j < total_mine && j < (size_t)kAgSlots; ++j) {
      uint32_t bytes;
      const size_t off = piece_off(j, bytes);
      mbar_expect_tx(bars + 8u * (uint32_t)j, bytes);
      bulk_load_1d(base + (uint32_t)j * kAgPiece, shard + off, bytes, bars + 8u * (uint32_t)j);
    }
  }
  bool ok = true;
  for (size_t j = 0; j < total_mine; ++j) {
    const uint32_t slot = (uint32_t)(j % kAgSlots);
    uint32_t bytes;
    const size_t off = piece_off(j, bytes);
    ok = mbar_wait(bars + 8u * slot, (uint32_t)(j / kAgSlots) & 1u, p.sync, 53);
    ok = __syncthreads_and(ok ? 1 : 0) != 0;
    if (!ok) break;
    const unsigned char* src = base_ptr + (size_t)slot * kAgPiece;
    if (p.ag_mc_weak) {
      for (uint32_t v = threadIdx.x; v < bytes / 16; v += blockDim.x)
        multimem_st16_weak(mc_out + off + (size_t)v * 16, *(const U4*)(src + (size_t)v * 16));
    } else {
      for (uint32_t v = threadIdx.x; v < bytes / 16; v += blockDim.x)
        multimem_st16(mc_out + off + (size_t)v * 16, *(const U4*)(src + (size_t)v * 16));
    }
    __syncthreads();                                   // every thread has read the slot and issued its stores
    if (threadIdx.x == 0) {
      const size_t jn = j + kAgSlots;
      if (jn < total_mine) {
        uint32_t nbytes;
        const size_t noff = piece_off(jn, nbytes);
        fence_proxy_async();                           // the slot's generic reads before the bulk copy overwrites it
        mbar_expect_tx(bars + 8u * slot, nbytes);
        bulk_load_1d(base + slot * kAgPiece, shard + noff, nbytes, bars + 8u * slot);
      }
      // last of my pieces of this chunk: count myself in; the comm CTA that completes the chunk
      // raises its flag on every rank
      if ((j + 1) % mine_per_chunk == 0) {
        const int sp = (int)(j / mine_per_chunk);
        uint32_t* cnt = p.counters + (size_t)p.rank * p.splits + sp;
        const uint32_t old = atom_add_acqrel_gpu(cnt, 1u);
        if (old == n_comm - 1) {
          *cnt = 0;
          multimem_red_add_release_u32(p.ag_mc_flags + p.rank * p.splits + sp, 1u);
        }
      }
    }
  }
  // the caller's progress words: in the order the chunks become usable here
  if (threadIdx.x == 0 && comm_id == 0 && p.progress != nullptr && ok) {
    for (int sp = 0; sp < p.splits && ok; ++sp)
      for (int step = 0; step < p.ws && ok; ++step) {
        const int idx = ((p.rank + step) % p.ws) * p.splits + sp;
        ok = wait_flag_acquire_sys(p.pads[p.rank] + p.flag_base + idx, 1u, p.sync, 54);
        if (ok) st_release_gpu(p.progress + idx, 1u);
      }
  }
}

// Push mode, every CTA on its way out: the last one puts this call's flag bank back to zero (all
// peers have signalled — every consumer has seen every flag — and the peers' next signals to this
// bank belong to the call after next).
__device__ __forceinline__ void ag_push_finish(const GemmParams& p, unsigned num_ctas) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* done = p.counters + (size_t)p.ws * p.splits;
    const uint32_t old = atom_add_acqrel_gpu(done, 1u);
    if (old == num_ctas - 1) {
      *done = 0;
      if (status_ok(p.sync))
        for (int i = 0; i < p.ws * p.splits; ++i) st_relaxed_sys(p.pads[p.rank] + p.flag_base + i, 0u);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// kernels
// ---------------------------------------------------------------------------------------------
template <int BN>
__device__ __forceinline__ void gemm_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned n_mma = (unsigned)p.num_mma_ctas;
  if (p.mode == GEMM_PLAIN) {
    PlainHooks h;
    h.bn = BN;
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
  } else if (p.mode == GEMM_AG) {
    if (bid >= n_mma) {
      if (p.ag_push && p.ag_mc_out != nullptr) ag_mc_cta(p, bid - n_mma, nb - n_mma, smem_raw);
      else if (p.ag_push) ag_push_cta(p, bid - n_mma, nb - n_mma, smem_raw);
      else ag_comm_cta(p, bid - n_mma, nb - n_mma, smem_raw);
    } else {
      AgHooks h;
      h.bn = BN;
      gemm_mainloop<BN>(p, bid, n_mma, h, smem_raw);
    }
    if (p.ag_push) ag_push_finish(p, nb);
  } else {
    CeHooks h;
    h.bn = BN;
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
  }
}

// CTA-pair kernel (256 x 256 tiles, tcgen05 cta_group::2); launched as clusters of two CTAs.
__device__ __forceinline__ void gemm_pair_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  const unsigned n_mma = (unsigned)p.num_mma_ctas;   // even
  if (p.mode == GEMM_PLAIN) {
    PlainHooks h;
    h.bn = 256;
    gemm_mainloop_pair(p, bid / 2, nb / 2, h, smem_raw);
  } else if (p.mode == GEMM_AG) {
    if (bid >= n_mma) {
      if (p.ag_push && p.ag_mc_out != nullptr) ag_mc_cta(p, bid - n_mma, nb - n_mma, smem_raw);
      else if (p.ag_push) ag_push_cta(p, bid - n_mma, nb - n_mma, smem_raw);
      else ag_comm_cta(p, bid - n_mma, nb - n_mma, smem_raw);
    } else {
      AgHooks h;
      h.bn = 256;
      gemm_mainloop_pair(p, bid / 2, n_mma / 2, h, smem_raw);
    }
    if (p.ag_push) ag_push_finish(p, nb);
  } else {
    CeHooks h;
    h.bn = 256;
    gemm_mainloop_pair(p, bid / 2, nb / 2, h, smem_raw);
  }
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_pair_kernel(const __grid_constant__ GemmParams p) {
  gemm_pair_body(p, blockIdx.x, gridDim.x);
}

#define KR_DEFINE_GEMM(BN)                                                                              \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm##BN##_kernel(const __grid_constant__ GemmParams p) { \
    gemm_body<BN>(p, blockIdx.x, gridDim.x);                                                            \
  }                                                                                                     \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm##BN##_emu_kernel(const GemmParams* ps) {       \
    gemm_body<BN>(ps[blockIdx.y], blockIdx.x, gridDim.x);                                               \
  }
KR_DEFINE_GEMM(256)
KR_DEFINE_GEMM(128)
KR_DEFINE_GEMM(64)
KR_DEFINE_GEMM(32)
KR_DEFINE_GEMM(16)

// ---------------------------------------------------------------------------------------------
// host: tensor-map cache
// ---------------------------------------------------------------------------------------------
struct TmapKey {
  const void* ptr;
  unsigned long long rows, cols, ld;
  unsigned box_rows;
  int elt;
  bool operator<(const TmapKey& o) const {
    return std::tie(ptr, rows, cols, ld, box_rows, elt) < std::tie(o.ptr, o.rows, o.cols, o.ld, o.box_rows, o.elt);
  }
};
static std::mutex g_tmap_mu;
static std::map<TmapKey, CUtensorMap> g_tmap_cache;
static std::deque<TmapKey> g_tmap_order;             // insertion order, for eviction
constexpr size_t kTmapCacheEntries = 4096;
static unsigned long long g_tmap_hits = 0, g_tmap_misses = 0;

// Tensor map of a row-major matrix [rows, cols] of bf16 (elt 2) or fp32 (elt 4) elements (cols
// contiguous, `ld` elements per row), box = 128 bytes of columns x box_rows rows, 128-byte swizzle,
// out-of-range elements read as zero.
int get_tmap(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                    unsigned box_rows, CUtensorMap* out, int elt) {
  TmapKey key{ptr, rows, cols, ld, box_rows, elt};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      ++g_tmap_hits;
      return KR_SUCCESS;
    }
  }
  KR_REQUIRE(((uintptr_t)ptr & 15) == 0, "GEMM operand must be 16-byte aligned");
  KR_REQUIRE(elt == 2 || elt == 4, "GEMM operands are bf16 or fp32");
  KR_REQUIRE((ld * elt) % 16 == 0, "GEMM operand row stride must be a multiple of 16 bytes");
  KR_REQUIRE(box_rows >= 1 && box_rows <= 256, "bad TMA box");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * (unsigned long long)elt};
  cuuint32_t box[2] = {(cuuint32_t)(128 / elt), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  KR_CU(cuTensorMapEncodeTiled, &m, elt == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
        const_cast<void*>(ptr), gdim, gstride, box,
        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    // bounded: the oldest descriptors go first, so a loop over a few operands keeps hitting
    while (g_tmap_cache.size() >= kTmapCacheEntries && !g_tmap_order.empty()) {
      g_tmap_cache.erase(g_tmap_order.front());
      g_tmap_order.pop_front();
    }
    if (g_tmap_cache.emplace(key, m).second) g_tmap_order.push_back(key);
    ++g_tmap_misses;
  }
  *out = m;
  return KR_SUCCESS;
}

// Row tiles (of 128 rows) that share one sweep over the column tiles. Larger groups re-read the
// column operand from DRAM fewer times; the group's rows (group * 128 * K * 2 bytes) should stay
// well inside the 126 MB L2. KRAKEN_GEMM_GROUP overrides for tuning.
int default_group_r() {
  static int v = 0;
  if (v == 0) {
    const char* e = getenv("KRAKEN_GEMM_GROUP");
    v = e ? atoi(e) : 16;
    if (v < 1) v = 16;
  }
  return v;
}

static bool tma_store_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("KRAKEN_TMA_STORE");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Tensor map for storing bf16 tiles into a row-major matrix [rows, cols] (row stride ld elements).
// Returns false (and leaves `m` alone) when the matrix cannot be described to TMA.
bool store_tmap(const void* ptr, long long rows, long long cols, long long ld, CUtensorMap* m) {
  if (!tma_store_enabled() || !ptr || ((uintptr_t)ptr & 15) || (ld * 2) % 16 || cols < 1 || rows < 1) return false;
  return get_tmap(ptr, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, 32, m) == KR_SUCCESS;
}

int pick_bn(int rows_c) {
  if (rows_c > 128) return 256;
  if (rows_c > 64) return 128;
  if (rows_c > 32) return 64;
  if (rows_c > 16) return 32;
  return 16;
}

// The tf32 kernels exist for three column-tile widths.
int tf32_bn(int rows_c) { return rows_c <= 16 ? 16 : (rows_c <= 64 ? 64 : 256); }

constexpr size_t kAgSmem = (size_t)kAgSlots * kAgPiece + 1024 + 128;
static_assert(kAgSmem <= (size_t)kSmemLimit, "comm ring exceeds shared memory");

bool pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("KRAKEN_GEMM_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Whether this problem can run on the CTA-pair kernel: 256-column tiles, at least one full pair of
// row tiles, a mode the pair kernel implements, slabs aligned to 256 rows where tiles belong to
// ranks, and no rank emulation (the emulated launch is cooperative, not clustered).
static bool pair_eligible(int bn, const GemmParams& p) {
  if (!pair_enabled() || emu_recorder().active) return false;
  if (bn != 256 || p.transposed || p.rows_r < 256 || p.in_fp32) return false;
  if (p.mode == GEMM_AR) return false;
  if (p.mode == GEMM_CE && (p.slab_rows % 256) != 0) return false;
  return true;
}

// Re-expresses the tiling in 256-row pair tiles and launches clusters of two CTAs.
// nb_single = CTAs the single-CTA kernel would have used (already capped); n_comm = comm CTAs (AG).
static int launch_pair(GemmParams p, unsigned cap, unsigned n_comm, cudaStream_t stream) {
  const int tiles128 = p.tiles_r;
  p.tiles_r = (p.rows_r + 255) / 256;
  p.pivot_r = p.tiles_r > 0 ? (p.pivot_r / 2) % p.tiles_r : 0;
  p.group_r = p.group_r >= 2 ? p.group_r / 2 : 1;
  if (p.mode == GEMM_CE) {
    const int per_slab = p.slab_rows / 256;
    if (p.group_r > per_slab) p.group_r = per_slab;
    while (per_slab % p.group_r) --p.group_r;
  }
  (void)tiles128;
  // each CTA of a pair loads its own 128 rows of the column operand: box of 128 rows, not 256
  int rc0 = get_tmap(p.host_c_ptr, p.rows_c, p.K, p.host_ldc, 128, &p.tmap_c);
  if (rc0) return rc0;
  n_comm = (n_comm + 1) & ~1u;
  cap &= ~1u;
  unsigned n_mma = 2u * (unsigned)(p.tiles_r * p.tiles_c);
  if (n_mma > cap - n_comm) n_mma = (cap - n_comm) & ~1u;
  if (n_mma < 2) return fail(KR_FAIL_ARG, "not enough CTAs for the pair kernel");
  p.num_mma_ctas = (int)n_mma;
  size_t smem = PairCfg::SMEM;
  if (p.mode == GEMM_AG && smem < kAgSmem) smem = kAgSmem;
  int rc = ensure_dynamic_smem((const void*)gemm_pair_kernel, smem);
  if (rc) return rc;
  void* args[] = {(void*)&p};
  KR_CUDA(cudaLaunchKernel((const void*)gemm_pair_kernel, dim3(n_mma + n_comm), dim3(kGemmThreads), args, smem, stream));
  return KR_SUCCESS;
}

int launch_gemm(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream) {
  if (p.in_fp32) return launch_gemm_tf32(bn, p, nb, stream);
  if (p.mode == GEMM_AR) return launch_gemm_ar(bn, p, nb, stream);
  const size_t floor_smem = p.mode == GEMM_AG ? kAgSmem : 0;   // comm CTAs reuse the block's shared memory
  auto sm = [&](size_t s) { return s > floor_smem ? s : floor_smem; };
  switch (bn) {
    case 256: return launch_ranked(gemm256_kernel, gemm256_emu_kernel, p, nb, kGemmThreads, sm(GemmCfg<256>::SMEM), stream);
    case 128: return launch_ranked(gemm128_kernel, gemm128_emu_kernel, p, nb, kGemmThreads, sm(GemmCfg<128>::SMEM), stream);
    case 64: return launch_ranked(gemm64_kernel, gemm64_emu_kernel, p, nb, kGemmThreads, sm(GemmCfg<64>::SMEM), stream);
    case 32: return launch_ranked(gemm32_kernel, gemm32_emu_kernel, p, nb, kGemmThreads, sm(GemmCfg<32>::SMEM), stream);
    default: return launch_ranked(gemm16_kernel, gemm16_emu_kernel, p, nb, kGemmThreads, sm(GemmCfg<16>::SMEM), stream);
  }
}

unsigned grid_cap(const DeviceState* d) {
  unsigned cap = (unsigned)d->num_sms;
  if (emu_recorder().active) {
    cap /= (unsigned)emu_recorder().ws;
    if (cap < 1) cap = 1;
  }
  return cap;
}

// Fills the operand/tiling part of the parameter block for C[M,N] = A[M,K] * Bt[N,K]^T.
// swap: the weights (Bt) become the 128-row operand and the tile is stored transposed.
int setup_problem(GemmParams& p, const void* a, long long lda, const void* bt, long long ldb, int M, int N,
                         int K, bool swap, int bn_override, int* bn_out, int elt) {
  KR_REQUIRE(M >= 1 && N >= 1 && K >= 8 && (K * elt) % 16 == 0, "GEMM needs K rows of whole 16-byte units and positive sizes");
  p.in_fp32 = elt == 4 ? 1 : 0;
  const void* r = swap ? bt : a;
  const void* c = swap ? a : bt;
  long long ldr = swap ? ldb : lda, ldc = swap ? lda : ldb;
  p.rows_r = swap ? N : M;
  p.rows_c = swap ? M : N;
  p.K = K;
  int bn = bn_override > 0 ? bn_override : pick_bn(p.rows_c);
  *bn_out = bn;
  p.tiles_r = (p.rows_r + kBM - 1) / kBM;
  p.tiles_c = (p.rows_c + bn - 1) / bn;
  p.group_r = default_group_r();
  p.pivot_r = 0;
  p.transposed = swap ? 1 : 0;
  int rc = get_tmap(r, p.rows_r, K, ldr, kBM, &p.tmap_r, elt);
  if (rc) return rc;
  rc = get_tmap(c, p.rows_c, K, ldc, bn, &p.tmap_c, elt);
  if (rc) return rc;
  p.host_c_ptr = c;
  p.host_ldc = ldc;
  p.tmap_r_local = p.tmap_r;
  return KR_SUCCESS;
}

}  // namespace kraken

using namespace kraken;

KR_API int kr_tmap_cache_stats(unsigned long long* hits, unsigned long long* misses) {
  std::lock_guard<std::mutex> lk(g_tmap_mu);
  *hits = g_tmap_hits;
  *misses = g_tmap_misses;
  return KR_SUCCESS;
}

// out[M,N] (bf16 or fp32, row stride ldo) = a[M,K] (row stride lda) * bt[N,K]^T (row stride ldb).
// swap_ab: -1 auto (weights on the 128-row side when M <= 64), 0/1 forced.
// use_pair: 0 forces the single-CTA kernel, anything else lets eligible shapes use CTA pairs.
// in_fp32: a and bt hold fp32 and are multiplied as tf32 (single-CTA kernels; strides in elements).
KR_API int kr_gemm_bf16(const void* a, long long lda, const void* bt, long long ldb, void* out, long long ldo, int M,
                        int N, int K, int out_fp32, int swap_ab, int bn_override, int max_ctas, int use_pair,
                        int in_fp32, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const bool swap = swap_ab < 0 ? (M <= 64 && N >= 128) : swap_ab != 0;
  int bn = 0;
  if (in_fp32 && bn_override <= 0) bn_override = tf32_bn(swap ? M : N);
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, swap, bn_override, &bn, in_fp32 ? 4 : 2);
  if (rc) return rc;
  if (in_fp32) KR_REQUIRE(bn == 16 || bn == 64 || bn == 256, "tf32 GEMM supports column tiles of 16, 64 and 256");
  p.mode = GEMM_PLAIN;
  p.out = out;
  p.ldo = ldo;
  p.out_rows = M;
  p.out_cols = N;
  p.out_fp32 = out_fp32;
  p.ws = 1;
  p.sync = sync_ctx(d);
  if (!swap && !out_fp32 && bn >= 64) p.use_tma_store = store_tmap(out, M, N, ldo, &p.tmap_out[0]) ? 1 : 0;
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (max_ctas > 0 && (unsigned)max_ctas < cap) cap = (unsigned)max_ctas;
  if (pair_eligible(bn, p) && cap >= 2 && use_pair != 0) return launch_pair(p, cap, 0, stream);
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

// Fused all-gather -> GEMM. a_out [ws*shard_rows, K] receives the gathered A; c[ws*shard_rows, N] =
// a_out * bt^T. progress [ws*splits] must be zero on entry; counters [ws*splits + 1] zero
// (self-resetting). Engines that fill a_out:
//   push == 0: bufs[r] = rank r's A shard (symmetric memory); num_comm_ctas > 0 comm CTAs pull the
//              shards, num_comm_ctas < 0: an external engine (copy engines) fills a_out and progress.
//   push == 1: bufs[r] = the symmetric buffer that holds rank r's gathered A at byte offset a_out_off
//              (a_out is this rank's address of it); num_comm_ctas comm CTAs push own_shard into every
//              rank's buffer and raise flags in the signal pads from word flag_base on (zero on entry,
//              zero again after the call; the caller alternates two banks). entry_barrier: wait for
//              all ranks before the first remote write (needed unless the caller alternates buffers).
//              mc_out / mc_flags: multicast addresses of the gathered buffer (at a_out_off) and of the
//              flag word flag_base — then the shard is written once, through the NVSwitch, and the
//              tile order after the own shard goes chunk by chunk over all peers; nullptr: one
//              unicast copy per peer, the peer that needs the shard first served first.
KR_API int kr_ag_gemm_bf16(void* const* bufs, uint32_t* const* pads, const void* own_shard, int rank, int ws,
                           void* a_out, const void* bt, long long ldb, void* c, long long ldc, int shard_rows, int N,
                           int K, int splits, uint32_t* progress, uint32_t* counters, int num_comm_ctas,
                           uint32_t pad_base, int push, unsigned long long a_out_off, uint32_t flag_base,
                           unsigned long long pad_words, int entry_barrier, void* mc_out, uint32_t* mc_flags,
                           cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(splits >= 1 && shard_rows % splits == 0, "shard rows must divide into splits");
  KR_REQUIRE(((size_t)(shard_rows / splits) * K * 2) % 16 == 0, "chunk size must be a multiple of 16 bytes");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  const int M = ws * shard_rows;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int bn = 0;
  int rc = setup_problem(p, a_out, K, bt, ldb, M, N, K, false, 0, &bn);
  if (rc) return rc;
  // own shard: read straight from the symmetric shard (address known on the host for self only)
  rc = get_tmap(own_shard, shard_rows, K, K, kBM, &p.tmap_r_local);
  if (rc) return rc;
  p.mode = GEMM_AG;
  p.out = c;
  p.ldo = ldc;
  p.out_rows = M;
  p.out_cols = N;
  if (bn >= 64) p.use_tma_store = store_tmap(c, M, N, ldc, &p.tmap_out[0]) ? 1 : 0;
  p.rank = rank;
  p.ws = ws;
  p.bufs = bufs;
  p.pads = pads;
  p.pad_base = pad_base;
  p.a_out = a_out;
  p.progress = progress;
  p.counters = counters;
  p.splits = splits;
  p.shard_rows = shard_rows;
  p.chunk_rows = shard_rows / splits;
  p.ag_push = push ? 1 : 0;
  p.ag_shard = own_shard;
  p.ag_out_off = a_out_off;
  p.ag_entry_barrier = entry_barrier ? 1 : 0;
  if (push) {
    KR_REQUIRE(num_comm_ctas > 0, "the push engine needs comm CTAs");
    KR_REQUIRE((unsigned long long)flag_base + (unsigned long long)ws * splits <= pad_words, "signal pad too small for the chunk flags");
    KR_REQUIRE(!entry_barrier || (unsigned long long)pad_base + (unsigned long long)d->num_sms * ws <= flag_base,
               "barrier slots overlap chunk flags");
    p.flag_base = flag_base;
    if (mc_out != nullptr) {
      KR_REQUIRE(mc_flags != nullptr, "multicast push needs the multicast address of the flags");
      p.ag_mc_out = mc_out;
      p.ag_mc_flags = mc_flags;
      static const int weak = [] { const char* e = getenv("KRAKEN_AG_MC_WEAK"); return (e && e[0] == '1') ? 1 : 0; }();
      p.ag_mc_weak = weak;
    }
  }
  p.pivot_r = (rank * shard_rows) / kBM;   // start on (or next to) the local shard
  if (p.tiles_r > 0) p.pivot_r %= p.tiles_r;
  // group must not mix chunks of different arrival times more than necessary
  int tiles_per_chunk = p.chunk_rows / kBM;
  p.group_r = tiles_per_chunk >= default_group_r() ? default_group_r() : (tiles_per_chunk >= 1 ? tiles_per_chunk : 1);
  p.sync = sync_ctx(d);
  unsigned cap = grid_cap(d);
  // num_comm_ctas < 0: no comm CTAs — an external engine (copy engine + stream memory operations)
  // fills a_out and sets the progress flags.
  unsigned n_comm = num_comm_ctas > 0 ? (unsigned)num_comm_ctas : (num_comm_ctas < 0 ? 0u : 8u);
  if (n_comm >= cap) n_comm = cap > 1 ? cap / 2 : 1;
  KR_REQUIRE(cap >= 2, "all-gather GEMM needs at least two CTAs");
  const bool pair = pair_eligible(bn, p) && cap >= 4;
  if (p.ag_mc_out != nullptr && ws > 1) {
    // chunk-major order needs chunks made of whole row tiles of the kernel that runs
    const int tile_rows = pair ? 256 : kBM;
    if (p.chunk_rows % tile_rows == 0) {
      p.ag_chunk_major = p.chunk_rows / tile_rows;
      p.ag_tiles_per_shard = shard_rows / tile_rows;
      p.pivot_r = 0;
      p.group_r = p.ag_chunk_major * (pair ? 2 : 1);       // launch_pair halves it again
    }
  }
  if (pair) return launch_pair(p, cap, n_comm, stream);
  unsigned n_mma = (unsigned)(p.tiles_r * p.tiles_c);
  if (n_mma > cap - n_comm) n_mma = cap - n_comm;
  p.num_mma_ctas = (int)n_mma;
  return launch_gemm(bn, p, n_mma + n_comm, stream);
}

// Producer GEMM of the copy-engine reduce-scatter variant: gemm_out[M, N] = a * bt^T on this GPU;
// signals[dst] becomes 1 when slab dst (rows [dst*M/ws, +M/ws)) is complete. signals must be zero
// on entry; counters [ws] zero (self-resetting). Slab of rank+1 is produced first.
KR_API int kr_gemm_ce_producer_bf16(const void* a, long long lda, const void* bt, long long ldb, void* gemm_out,
                                    long long ldo, int M, int N, int K, int rank, int ws, uint32_t* signals,
                                    uint32_t* counters, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(M % ws == 0 && (M / ws) % kBM == 0, "copy-engine GEMM reduce-scatter needs (M / world_size) % 128 == 0");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int bn = 0;
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, false, N >= 256 ? 256 : 0, &bn);
  if (rc) return rc;
  p.mode = GEMM_CE;
  p.out = gemm_out;
  p.ldo = ldo;
  p.out_rows = M;
  p.out_cols = N;
  if (bn >= 64) p.use_tma_store = store_tmap(gemm_out, M, N, ldo, &p.tmap_out[0]) ? 1 : 0;
  p.rank = rank;
  p.ws = ws;
  p.progress = signals;
  p.counters = counters;
  p.slab_rows = M / ws;
  const int tiles_per_slab = p.slab_rows / kBM;
  p.pivot_r = (((rank + 1) % ws) * tiles_per_slab) % p.tiles_r;
  p.group_r = tiles_per_slab >= default_group_r() ? default_group_r() : tiles_per_slab;
  while (tiles_per_slab % p.group_r) --p.group_r;
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (pair_eligible(bn, p) && cap >= 2) return launch_pair(p, cap, 0, stream);
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

// Host evaluation of the persistent tile order (the same function the kernels run): writes
// (row tile, column tile) of linear tile t to out[2t], out[2t+1]. For tests of the index math.
KR_API int kr_tile_order(int tiles_r, int tiles_c, int group_r, int pivot_r, int interleave_r, int* out) {
  KR_REQUIRE(tiles_r >= 1 && tiles_c >= 1 && group_r >= 1 && pivot_r >= 0 && pivot_r < tiles_r, "bad tiling");
  KR_REQUIRE(interleave_r <= 1 || tiles_r % interleave_r == 0, "interleave must divide the row tiles");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.tiles_r = tiles_r;
  p.tiles_c = tiles_c;
  p.group_r = group_r;
  p.pivot_r = pivot_r;
  p.interleave_r = interleave_r;
  for (int t = 0; t < tiles_r * tiles_c; ++t) tile_coords(p, t, out[2 * t], out[2 * t + 1]);
  return KR_SUCCESS;
}

// The same for the chunk-major order of the all-gather GEMM fed by a multicast push: `tiles_per_shard`
// row tiles per rank, `chunk_tiles` of them per chunk.
KR_API int kr_tile_order_ag(int tiles_c, int group_r, int rank, int ws, int tiles_per_shard, int chunk_tiles, int* out) {
  KR_REQUIRE(tiles_c >= 1 && group_r >= 1 && ws >= 1 && rank >= 0 && rank < ws, "bad tiling");
  KR_REQUIRE(chunk_tiles >= 1 && tiles_per_shard % chunk_tiles == 0, "chunks must be whole row tiles");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.tiles_r = ws * tiles_per_shard;
  p.tiles_c = tiles_c;
  p.group_r = group_r;
  p.rank = rank;
  p.ws = ws;
  p.ag_chunk_major = chunk_tiles;
  p.ag_tiles_per_shard = tiles_per_shard;
  for (int t = 0; t < p.tiles_r * tiles_c; ++t) tile_coords(p, t, out[2 * t], out[2 * t + 1]);
  return KR_SUCCESS;
}
