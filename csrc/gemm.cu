// tcgen05 GEMM kernels: plain GEMM and the three fused GEMM + collective kernels.
//
//  * all-gather -> GEMM (reference: kraken/fused/all_gather_matmul.py:222-325): a few comm CTAs
//    pull the peers' A shards into the local gathered buffer with 1-D bulk async copies and
//    publish per-chunk progress flags; the MMA CTAs start on the local shard (rank pivot) and
//    consume remote chunks as their flags appear. One launch, no copy engine, no second stream.
//  * GEMM -> reduce-scatter (reference: kraken/fused/gemm_reduce_scatter_fused.py:152-235 and
//    gemm_reduce_scatter_ce_persistent.py:326-375): the epilogue pushes each finished tile straight
//    into the OWNER rank's staging slab over NVLink and bumps a per-tile flag there; after its last
//    GEMM tile every CTA turns reducer for tiles of its own slab, summing the ws slabs in fixed
//    rank order (bitwise reproducible).
//  * GEMM -> all-reduce for decode (reference: kraken/fused/gemm_one_shot_all_reduce_fused.py:106-178):
//    fp32 partial tile to the own staging buffer, per-tile flags to all peers, then each rank sums
//    the tile from all ranks in rank order into its fp32 output.
#include <map>
#include <mutex>
#include <tuple>
#include "kraken/driver_api.h"
#include "kraken/gemm_core.cuh"

namespace kraken {

// ---------------------------------------------------------------------------------------------
// hooks
// ---------------------------------------------------------------------------------------------
struct PlainHooks {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols};
  }
  __device__ __forceinline__ bool after_store(const GemmParams&, int, int, int, int) { return true; }
};

struct AgHooks {
  int bn;
  // Row tile tr covers gathered rows [tr*128, +128). Rows of the own shard come from the own
  // shard's tensor map at once; other rows wait until every chunk they touch has landed.
  __device__ __forceinline__ bool before_load(const GemmParams& p, int tr, const CUtensorMap*& rmap, int& row0) {
    const int lo = tr * kBM;
    const int hi = min(lo + kBM, p.rows_r) - 1;
    const int own_lo = p.rank * p.shard_rows;
    if (lo >= own_lo && hi < own_lo + p.shard_rows) {
      rmap = &p.tmap_r_local;
      row0 = lo - own_lo;
      return true;
    }
    const int c_lo = lo / p.chunk_rows, c_hi = hi / p.chunk_rows;
    for (int c = c_lo; c <= c_hi; ++c)
      if (!wait_flag_acquire_gpu(p.progress + c, 1u, p.sync, 50)) return false;
    fence_proxy_async();   // chunk was written through another proxy / by other CTAs
    return true;
  }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols};
  }
  __device__ __forceinline__ bool after_store(const GemmParams&, int, int, int, int) { return true; }
};

struct RsHooks {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  // Tile (tr, tc) of the full [M, N] product belongs to rank owner = row / slab_rows; it goes to
  // slot `rank` of the owner's staging [ws][slab_rows][N].
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    const int owner = (tr * kBM) / p.slab_rows;
    char* base = (char*)p.bufs[owner] + (size_t)p.rank * p.slab_rows * p.rows_c * 2;
    return TileDest{base, (long long)p.rows_c, tr * kBM - owner * p.slab_rows, tc * bn, p.slab_rows, p.rows_c};
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    epi_bar_sync();   // all four epilogue warps have issued their stores of this tile
    if (q == 0 && lane == 0) {
      const int owner = (tr * kBM) / p.slab_rows;
      const int tiles_per_slab = p.slab_rows / kBM;
      const int local_tile = (tr - owner * tiles_per_slab) * p.tiles_c + tc;
      red_add_release_sys(p.pads[owner] + p.flag_base + local_tile, 1u);
    }
    return true;
  }
};

struct ArHooks {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  // partial tile -> own fp32 staging [out_rows][out_cols]
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.bufs[p.rank], (long long)p.out_cols, tr * kBM, tc * bn, p.out_rows, p.out_cols};
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    const int tile = tr * p.tiles_c + tc;
    const int tid = q * 32 + lane;   // 0..127 over the epilogue warps (q is a permutation of 0..3)
    epi_bar_sync();
    if (tid < p.ws && tid != p.rank) red_add_release_sys(p.pads[tid] + p.flag_base + tile, 1u);
    if (tid == 0 && p.ws > 1) {
      uint32_t* f = p.pads[p.rank] + p.flag_base + tile;
      const uint32_t need = (uint32_t)(p.ws - 1);
      if (spin_until([&] { return ld_acquire_sys(f) >= need; }, p.sync,
                     make_status(KR_ERR_TIMEOUT_SIGNAL, 51, 0, blockIdx.x)))
        red_add_relaxed_sys(f, 0u - need);
    }
    epi_bar_sync();
    if (!status_ok(p.sync)) return false;
    // sum the tile from every rank in rank order; the region in `out` orientation:
    int r_lo, r_n, c_lo, c_n;
    if (p.transposed) { r_lo = tc * bn; r_n = bn; c_lo = tr * kBM; c_n = kBM; }
    else { r_lo = tr * kBM; r_n = kBM; c_lo = tc * bn; c_n = bn; }
    const int upr = c_n / 4;   // 16-byte units per row
    for (int i = tid; i < r_n * upr; i += 128) {
      const int rr = r_lo + i / upr, cc = c_lo + (i % upr) * 4;
      if (rr >= p.out_rows || cc >= p.out_cols) continue;
      const size_t off = ((size_t)rr * p.out_cols + cc) * 4;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cc + 4 <= p.out_cols && (p.out_cols % 4) == 0 && (p.ldo % 4) == 0) {
        for (int s = 0; s < p.ws; ++s) {
          U4 v = ld16((const char*)p.bufs[s] + off);
          a.x += __uint_as_float(v.x); a.y += __uint_as_float(v.y);
          a.z += __uint_as_float(v.z); a.w += __uint_as_float(v.w);
        }
        *(float4*)((float*)p.out + (size_t)rr * p.ldo + cc) = a;
      } else {
        for (int e = 0; e < 4 && cc + e < p.out_cols; ++e) {
          float acc = 0.f;
          for (int s = 0; s < p.ws; ++s) acc += ((const volatile float*)((const char*)p.bufs[s] + off))[e];
          ((float*)p.out)[(size_t)rr * p.ldo + cc + e] = acc;
        }
      }
    }
    return true;
  }
};

// Producer GEMM of the copy-engine reduce-scatter variant
// (reference: gemm_reduce_scatter_ce_persistent.py:46-134): tiles go to the local gemm_out; a
// per-destination counter tracks finished tiles and the tile that completes a slab raises that
// slab's signal word to 1 with system-scope release, which a stream wait on the host side consumes.
struct CeHooks {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols};
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
// RS reducer: after the GEMM loop, sum the ws staged slabs of my own slab tile by tile.
// ---------------------------------------------------------------------------------------------
template <int BN>
__device__ __forceinline__ void rs_reduce_phase(const GemmParams& p, unsigned bid, unsigned nb) {
  const int tiles_per_slab = p.slab_rows / kBM;
  const int slab_tiles = tiles_per_slab * p.tiles_c;
  const char* stage = (const char*)p.bufs[p.rank];
  const size_t slab_bytes = (size_t)p.slab_rows * p.rows_c * 2;
  // visit tiles in the order peers finish them: each peer computes my slab at a different time,
  // but all of them sweep it row tile by row tile
  for (int t = bid; t < slab_tiles; t += nb) {
    uint32_t* f = p.pads[p.rank] + p.flag_base + t;
    if (threadIdx.x == 0) {
      const uint32_t need = (uint32_t)p.ws;
      if (spin_until([&] { return ld_acquire_sys(f) >= need; }, p.sync,
                     make_status(KR_ERR_TIMEOUT_SIGNAL, 55, 0, bid)))
        red_add_relaxed_sys(f, 0u - need);
    }
    __syncthreads();
    if (!status_ok(p.sync)) return;
    const int tr = t / p.tiles_c, tc = t % p.tiles_c;
    const int upr = BN / 8;   // 16-byte units per tile row
    for (int i = threadIdx.x; i < kBM * upr; i += blockDim.x) {
      const int rr = tr * kBM + i / upr;
      const int cc = tc * BN + (i % upr) * 8;
      if (rr >= p.slab_rows || cc >= p.rows_c) continue;
      const size_t off = ((size_t)rr * p.rows_c + cc) * 2;
      float f8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      U4 x[8];
      for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s0 + s < p.ws) x[s] = ld16(stage + (size_t)(s0 + s) * slab_bytes + off);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s0 + s < p.ws) acc8(x[s], f8);
      }
      st16((char*)p.out + ((size_t)rr * p.ldo + cc) * 2, pack8(f8));
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
    PlainHooks h{BN};
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
  } else if (p.mode == GEMM_AG) {
    if (bid >= n_mma) {
      ag_comm_cta(p, bid - n_mma, nb - n_mma, smem_raw);
    } else {
      AgHooks h{BN};
      gemm_mainloop<BN>(p, bid, n_mma, h, smem_raw);
    }
  } else if (p.mode == GEMM_RS) {
    RsHooks h{BN};
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
    __syncthreads();
    rs_reduce_phase<BN>(p, bid, nb);
    // staging slabs and flags may be reused by the next launch only after every rank is done
    symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 56);
  } else if (p.mode == GEMM_CE) {
    CeHooks h{BN};
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
  } else {
    ArHooks h{BN};
    gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
    symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 57);
  }
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
  bool operator<(const TmapKey& o) const {
    return std::tie(ptr, rows, cols, ld, box_rows) < std::tie(o.ptr, o.rows, o.cols, o.ld, o.box_rows);
  }
};
static std::mutex g_tmap_mu;
static std::map<TmapKey, CUtensorMap> g_tmap_cache;
static unsigned long long g_tmap_hits = 0, g_tmap_misses = 0;

// Tensor map of a row-major bf16 matrix [rows, cols] (cols contiguous, `ld` elements per row),
// box = 64 columns x box_rows rows, 128-byte swizzle, out-of-range elements read as zero.
static int get_tmap(const void* ptr, unsigned long long rows, unsigned long long cols, unsigned long long ld,
                    unsigned box_rows, CUtensorMap* out) {
  TmapKey key{ptr, rows, cols, ld, box_rows};
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
  KR_REQUIRE((ld * 2) % 16 == 0, "GEMM operand row stride must be a multiple of 8 elements");
  KR_REQUIRE(box_rows >= 1 && box_rows <= 256, "bad TMA box");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  KR_CU(cuTensorMapEncodeTiled, &m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box,
        estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  {
    std::lock_guard<std::mutex> lk(g_tmap_mu);
    if (g_tmap_cache.size() > 4096) g_tmap_cache.clear();
    g_tmap_cache[key] = m;
    ++g_tmap_misses;
  }
  *out = m;
  return KR_SUCCESS;
}

static int pick_bn(int rows_c) {
  if (rows_c > 128) return 256;
  if (rows_c > 64) return 128;
  if (rows_c > 32) return 64;
  if (rows_c > 16) return 32;
  return 16;
}

constexpr size_t kAgSmem = (size_t)kAgSlots * kAgPiece + 1024 + 128;
static_assert(kAgSmem <= (size_t)kSmemLimit, "comm ring exceeds shared memory");

static int launch_gemm(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream) {
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

static unsigned grid_cap(const DeviceState* d) {
  unsigned cap = (unsigned)d->num_sms;
  if (emu_recorder().active) {
    cap /= (unsigned)emu_recorder().ws;
    if (cap < 1) cap = 1;
  }
  return cap;
}

// Fills the operand/tiling part of the parameter block for C[M,N] = A[M,K] * Bt[N,K]^T.
// swap: the weights (Bt) become the 128-row operand and the tile is stored transposed.
static int setup_problem(GemmParams& p, const void* a, long long lda, const void* bt, long long ldb, int M, int N,
                         int K, bool swap, int bn_override, int* bn_out) {
  KR_REQUIRE(M >= 1 && N >= 1 && K >= 8 && K % 8 == 0, "GEMM needs K % 8 == 0 and positive sizes");
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
  p.group_r = 8;
  p.pivot_r = 0;
  p.transposed = swap ? 1 : 0;
  int rc = get_tmap(r, p.rows_r, K, ldr, kBM, &p.tmap_r);
  if (rc) return rc;
  rc = get_tmap(c, p.rows_c, K, ldc, bn, &p.tmap_c);
  if (rc) return rc;
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
KR_API int kr_gemm_bf16(const void* a, long long lda, const void* bt, long long ldb, void* out, long long ldo, int M,
                        int N, int K, int out_fp32, int swap_ab, int bn_override, int max_ctas, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const bool swap = swap_ab < 0 ? (M <= 64 && N >= 128) : swap_ab != 0;
  int bn = 0;
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, swap, bn_override, &bn);
  if (rc) return rc;
  p.mode = GEMM_PLAIN;
  p.out = out;
  p.ldo = ldo;
  p.out_rows = M;
  p.out_cols = N;
  p.out_fp32 = out_fp32;
  p.ws = 1;
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (max_ctas > 0 && (unsigned)max_ctas < cap) cap = (unsigned)max_ctas;
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

// Fused all-gather -> GEMM. bufs[r] = rank r's A shard [shard_rows, K] (symmetric memory);
// a_out [ws*shard_rows, K] receives the gathered A; c[ws*shard_rows, N] = a_out * bt^T.
// progress [ws*splits] must be zero on entry; counters [ws*splits] zero (self-resetting).
KR_API int kr_ag_gemm_bf16(void* const* bufs, uint32_t* const* pads, const void* own_shard, int rank, int ws,
                           void* a_out, const void* bt, long long ldb, void* c, long long ldc, int shard_rows, int N,
                           int K, int splits, uint32_t* progress, uint32_t* counters, int num_comm_ctas,
                           uint32_t pad_base, cudaStream_t stream) {
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
  p.pivot_r = (rank * shard_rows) / kBM;   // start on (or next to) the local shard
  if (p.tiles_r > 0) p.pivot_r %= p.tiles_r;
  // group must not mix chunks of different arrival times more than necessary
  int tiles_per_chunk = p.chunk_rows / kBM;
  p.group_r = tiles_per_chunk >= 8 ? 8 : (tiles_per_chunk >= 1 ? tiles_per_chunk : 1);
  p.sync = sync_ctx(d);
  unsigned cap = grid_cap(d);
  // num_comm_ctas < 0: no comm CTAs — an external engine (copy engine + stream memory operations)
  // fills a_out and sets the progress flags.
  unsigned n_comm = num_comm_ctas > 0 ? (unsigned)num_comm_ctas : (num_comm_ctas < 0 ? 0u : 8u);
  if (n_comm >= cap) n_comm = cap > 1 ? cap / 2 : 1;
  KR_REQUIRE(cap >= 2, "all-gather GEMM needs at least two CTAs");
  unsigned n_mma = (unsigned)(p.tiles_r * p.tiles_c);
  if (n_mma > cap - n_comm) n_mma = cap - n_comm;
  p.num_mma_ctas = (int)n_mma;
  return launch_gemm(bn, p, n_mma + n_comm, stream);
}

// Fused GEMM -> reduce-scatter. a[M, K_local], bt[N, K_local]; bufs[r] = rank r's staging
// workspace of at least M*N*2 bytes; out[M/ws, N] bf16. Tile flags live in the signal pads at
// word offset flag_base (zero on entry, zero again on exit).
KR_API int kr_gemm_rs_bf16(void* const* bufs, uint32_t* const* pads, int rank, int ws, const void* a, long long lda,
                           const void* bt, long long ldb, void* out, long long ldo, int M, int N, int K,
                           uint32_t pad_base, uint32_t flag_base, unsigned long long pad_words, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(M % ws == 0 && (M / ws) % kBM == 0, "fused GEMM reduce-scatter needs (M / world_size) % 128 == 0");
  KR_REQUIRE(N % 8 == 0, "fused GEMM reduce-scatter needs N % 8 == 0");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int bn = 0;
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, false, N >= 256 ? 256 : 0, &bn);
  if (rc) return rc;
  p.mode = GEMM_RS;
  p.out = out;
  p.ldo = ldo;
  p.out_rows = M / ws;
  p.out_cols = N;
  p.rank = rank;
  p.ws = ws;
  p.bufs = bufs;
  p.pads = pads;
  p.pad_base = pad_base;
  p.flag_base = flag_base;
  p.slab_rows = M / ws;
  const int tiles_per_slab = p.slab_rows / kBM;
  KR_REQUIRE((unsigned long long)flag_base + (unsigned long long)tiles_per_slab * p.tiles_c <= pad_words,
             "signal pad too small for the tile flags");
  p.pivot_r = (((rank + 1) % ws) * tiles_per_slab) % p.tiles_r;   // next rank's slab first, own slab last
  p.group_r = tiles_per_slab >= 8 ? 8 : tiles_per_slab;
  while (tiles_per_slab % p.group_r) --p.group_r;                 // groups never straddle two slabs
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (nb > cap) nb = cap;
  KR_REQUIRE((unsigned long long)pad_base + (unsigned long long)nb * ws <= flag_base, "barrier slots overlap tile flags");
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

// Fused GEMM -> one-shot all-reduce (decode). bufs[r] = fp32 staging [M, N] of rank r;
// out[M, N] fp32 = sum_r a_r[M, K_local] * bt_r[N, K_local]^T.
KR_API int kr_gemm_ar_bf16(void* const* bufs, uint32_t* const* pads, int rank, int ws, const void* a, long long lda,
                           const void* bt, long long ldb, void* out, long long ldo, int M, int N, int K, int swap_ab,
                           uint32_t pad_base, uint32_t flag_base, unsigned long long pad_words, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const bool swap = swap_ab < 0 ? (M <= 64 && N >= 128) : swap_ab != 0;
  int bn = 0;
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, swap, 0, &bn);
  if (rc) return rc;
  p.mode = GEMM_AR;
  p.out = out;
  p.ldo = ldo;
  p.out_rows = M;
  p.out_cols = N;
  p.out_fp32 = 1;
  p.rank = rank;
  p.ws = ws;
  p.bufs = bufs;
  p.pads = pads;
  p.pad_base = pad_base;
  p.flag_base = flag_base;
  KR_REQUIRE((unsigned long long)flag_base + (unsigned long long)p.tiles_r * p.tiles_c <= pad_words,
             "signal pad too small for the tile flags");
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (nb > cap) nb = cap;
  KR_REQUIRE((unsigned long long)pad_base + (unsigned long long)nb * ws <= flag_base, "barrier slots overlap tile flags");
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
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
  p.rank = rank;
  p.ws = ws;
  p.progress = signals;
  p.counters = counters;
  p.slab_rows = M / ws;
  const int tiles_per_slab = p.slab_rows / kBM;
  p.pivot_r = (((rank + 1) % ws) * tiles_per_slab) % p.tiles_r;
  p.group_r = tiles_per_slab >= 8 ? 8 : tiles_per_slab;
  while (tiles_per_slab % p.group_r) --p.group_r;
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(p.tiles_r * p.tiles_c);
  unsigned cap = grid_cap(d);
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}
