// Fused GEMM -> reduce-scatter on the tcgen05 main loop (reference:
// kraken/fused/gemm_reduce_scatter_fused.py:152-235, gemm_reduce_scatter_ce_persistent.py:326-375).
// C[M, N] = A[M, K_local] * Bt[N, K_local]^T is a partial sum on every rank; rank r ends up with
// rows [r*M/ws, (r+1)*M/ws) of the sum over ranks. Two exchange algorithms share the main loop:
//
//  * pull: every rank TMA-stores ALL its partial tiles into its OWN symmetric staging matrix
//    [M][N] (local traffic only, the epilogue never touches NVLink) and bumps a per-tile arrival
//    counter in the tile owner's signal pad. Six extra "reducer" warps per CTA serve the tiles this
//    rank owns, in work items of 16 rows dealt round-robin to all CTAs: wait until all ws ranks have
//    stored the tile, then sum it across ranks with ws peer loads in rank order (or in the NVSwitch
//    with multimem.ld_reduce when asked to) and write the final rows.
//  * scatter: as pull, but the epilogue TMA-stores each tile into slot [rank] of the OWNER's
//    staging [ws][M/ws][N] over NVLink (posted writes), so the reducer warps sum ws slots out of
//    local memory.
//    In both, all ranks walk the tiles in the same order with the owners interleaved, so every
//    owner's tiles complete at an even rate and the reduction of one tile overlaps the MMAs of the
//    following ones. Staging halves and counter banks alternate call by call (a rank can only be
//    one call ahead of a peer: finishing a call takes a signal from every peer sent in that same
//    call), so there is no grid-wide or cross-rank barrier at all.
//  * push: the epilogue TMA-stores each remote tile into the owner's staging slab [src][M/ws][N]
//    over NVLink and bumps the owner's counter; own-slab tiles are computed last, their epilogue
//    waits for the ws-1 peers, adds the staged partial sums to the accumulator fragment in rank
//    order and writes the final rows. A per-block exit barrier protects the staging slabs.
#include "kraken/gemm_host.h"

namespace kraken {

constexpr int kRsReducerThreads = 192;   // six warps: with 12 warps per CTA the register budget per thread is the same as with 10
constexpr int kRsPullThreads = kGemmThreads + kRsReducerThreads;

// Named barriers of the two groups of 192 threads that reduce work items: 2 for the reducer warps,
// 3 for the pipeline warps once they help.
__device__ __forceinline__ void group_bar_sync(int group) {
  if (group == 0) asm volatile("bar.sync 2, 192;" ::: "memory");
  else asm volatile("bar.sync 3, 192;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// push: remote tiles go to the owner's staging slab, own tiles reduce in the epilogue
// ---------------------------------------------------------------------------------------------
struct RsPushHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ int owner_of(const GemmParams& p, int tr) const { return (tr * kBM) / p.slab_rows; }
  __device__ __forceinline__ int local_tile(const GemmParams& p, int tr, int tc) const {
    return (tr - owner_of(p, tr) * (p.slab_rows / kBM)) * p.tiles_c + tc;
  }
  // begin_tile of an own-slab tile blocks until the peers have pushed their partial tiles
  __device__ __forceinline__ bool may_wait(const GemmParams& p, int tr) const { return p.ws > 1 && owner_of(p, tr) == p.rank; }
  __device__ __forceinline__ bool begin_tile(const GemmParams& p, int tr, int tc, int q, int lane) {
    if (owner_of(p, tr) != p.rank || p.ws == 1) return true;
    uint32_t* f = p.pads[p.rank] + p.flag_base + local_tile(p, tr, tc);
    const uint32_t need = (uint32_t)(p.ws - 1);
    if (lane == 0)
      spin_until([&] { return ld_acquire_sys(f) >= need; }, p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 55, 0, blockIdx.x));
    __syncwarp();
    epi_bar_sync();                       // every epilogue warp has seen the flag
    if (q == 0 && lane == 0) red_add_relaxed_sys(f, 0u - need);
    return status_ok(p.sync);
  }
  // Remote tiles go to slot `rank` of the owner's staging [ws][slab_rows][N]; own tiles go to `out`.
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    const int owner = owner_of(p, tr);
    const int row0 = tr * kBM - owner * p.slab_rows;
    if (owner == p.rank) return TileDest{(char*)p.out, p.ldo, row0, tc * bn, p.slab_rows, p.rows_c, p.use_tma_store ? &p.tmap_out[p.ws] : nullptr};
    char* base = (char*)p.bufs[owner] + (size_t)p.rank * p.slab_rows * p.rows_c * 2;
    return TileDest{base, (long long)p.rows_c, row0, tc * bn, p.slab_rows, p.rows_c, p.use_tma_store ? &p.tmap_out[owner] : nullptr};
  }
  // Own tiles: add the peers' staged partial sums (bf16) to the fp32 fragment, in rank order.
  __device__ __forceinline__ void add_to_chunk(const GemmParams& p, int tr, int tc, int row_in_tile, int col_in_tile,
                                               uint32_t (&r)[32], int n) {
    if (owner_of(p, tr) != p.rank || p.ws == 1) return;
    const int row = tr * kBM - p.rank * p.slab_rows + row_in_tile;
    const int col = tc * bn + col_in_tile;
    if (row >= p.slab_rows) return;
    const char* stage = (const char*)p.bufs[p.rank];
    const size_t slab_bytes = (size_t)p.slab_rows * p.rows_c * 2;
    const size_t off = ((size_t)row * p.rows_c + col) * 2;
    // Peers in batches of four: the 16 loads of a batch are issued before the first add, so a chunk
    // costs ceil((ws-1)/4) memory round trips instead of ws-1. The order of the adds stays rank order.
    for (int s0 = 0; s0 < p.ws; s0 += 4) {
      U4 x[4][4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int s = s0 + k;
        if (s < p.ws && s != p.rank) {
          const char* src = stage + (size_t)s * slab_bytes + off;
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (u * 8 < n && col + u * 8 < p.rows_c) x[k][u] = ld16(src + u * 16);   // N % 8 == 0: units are all-in or all-out
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int s = s0 + k;
        if (s < p.ws && s != p.rank) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (u * 8 < n && col + u * 8 < p.rows_c) {
              const uint32_t w[4] = {x[k][u].x, x[k][u].y, x[k][u].z, x[k][u].w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                r[u * 8 + 2 * e] = __float_as_uint(__uint_as_float(r[u * 8 + 2 * e]) + bf16lo(w[e]));
                r[u * 8 + 2 * e + 1] = __float_as_uint(__uint_as_float(r[u * 8 + 2 * e + 1]) + bf16hi(w[e]));
              }
            }
          }
        }
      }
    }
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    const int owner = owner_of(p, tr);
    if (owner == p.rank) return true;
    epi_bar_sync();   // all four epilogue warps have issued their stores of this tile
    if (q == 0 && lane == 0) red_add_release_sys(p.pads[owner] + p.flag_base + local_tile(p, tr, tc), 1u);
    return true;
  }
};

// ---------------------------------------------------------------------------------------------
// pull / scatter: the epilogue only stores and signals; reducer warps sum the tiles this rank owns
// ---------------------------------------------------------------------------------------------
// A reduce work item is p.rs_sub_rows rows (16 ... 128, a power of two) of a 128-row tile: chosen
// on the host so that an item always moves about 64 KB (rows x 512 bytes x ws sources) and the last
// wave of tiles leaves about one item per CTA.

struct RsPullHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  __device__ __forceinline__ size_t slab_bytes(const GemmParams& p) const { return (size_t)p.slab_rows * p.rows_c * 2; }
  // pull: the own staging matrix [M][N]. scatter: slot [rank] of the owner's staging [ws][M/ws][N].
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    if (p.rs_algo == 2) {
      const int owner = (tr * kBM) / p.slab_rows;
      char* base = (char*)p.peer_buf[owner] + p.stage_off + (size_t)p.rank * slab_bytes(p);
      return TileDest{base, (long long)p.rows_c, tr * kBM - owner * p.slab_rows, tc * bn, p.slab_rows, p.rows_c,
                      p.use_tma_store ? &p.tmap_out[owner] : nullptr};
    }
    char* base = (char*)p.peer_buf[p.rank] + p.stage_off;
    return TileDest{base, (long long)p.rows_c, tr * kBM, tc * bn, p.rows_r, p.rows_c, p.use_tma_store ? &p.tmap_out[0] : nullptr};
  }
  // arrival counter of 128-row tile `tr`, column tile `tc` in its owner's signal pad
  __device__ __forceinline__ uint32_t* counter(const GemmParams& p, int owner, int tr, int tc) const {
    return p.peer_pad[owner] + p.flag_base + (size_t)(tr - owner * (p.slab_rows / kBM)) * p.tiles_c + tc;
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    if (tr * kBM >= p.rows_r) return true;
    epi_bar_sync();   // all four epilogue warps' stores of this tile are complete
    if (q == 0 && lane == 0) {
      const int owner = (tr * kBM) / p.slab_rows;
      const long long unit = (long long)(tr - owner * (p.slab_rows / kBM)) * p.tiles_c + tc;
      if (kr_in_bounds(owner >= 0 && owner < p.ws && unit >= 0 && unit < (long long)p.rs_done_off, p.sync, 70))
        red_add_release_sys(counter(p, owner, tr, tc), 1u);
    }
    return true;
  }
  // Where rank s's partial sums of this rank's slab start.
  __device__ __forceinline__ const char* source_slab(const GemmParams& p, int s) const {
    if (p.rs_algo == 2) return (const char*)p.peer_buf[p.rank] + p.stage_off + (size_t)s * slab_bytes(p);
    return (const char*)p.peer_buf[s] + p.stage_off + (size_t)p.rank * slab_bytes(p);
  }

  // Sum with plain loads: B vectors per thread, all W >= ws ranks' loads of all of them in flight
  // together (B * W = 8 requests per thread: sixteen made the register allocator spill the loaded
  // values, which turns every load into a synchronous one); adds in rank order (every call gives
  // the same bits).
  template <int B, int W>
  __device__ __forceinline__ void reduce_loads(const GemmParams& p, int tid, int total, int vpr, int lrow0, int col0) {
    const char* src[W];
#pragma unroll
    for (int s = 0; s < W; ++s) src[s] = s < p.ws ? source_slab(p, s) : nullptr;
    for (int i0 = tid; i0 < total; i0 += kRsReducerThreads * B) {
      U4 x[B][W];
#pragma unroll
      for (int k = 0; k < B; ++k) {
        const int i = i0 + k * kRsReducerThreads;
        if (i < total) {
          const int r = i / vpr, v = i - r * vpr;
          const size_t off = ((size_t)(lrow0 + r) * p.rows_c + col0 + v * 8) * 2;
#pragma unroll
          for (int s = 0; s < W; ++s)
            if (s < p.ws) x[k][s] = ld16(src[s] + off);
        }
      }
#pragma unroll
      for (int k = 0; k < B; ++k) {
        const int i = i0 + k * kRsReducerThreads;
        if (i < total) {
          float f8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int s = 0; s < W; ++s)
            if (s < p.ws) acc8(x[k][s], f8);
          const int r = i / vpr, v = i - r * vpr;
          st16((char*)p.out + ((size_t)(lrow0 + r) * p.ldo + col0 + v * 8) * 2, pack8(f8));
        }
      }
    }
  }

  // One work item: rows [sub*rs_sub_rows, +rs_sub_rows) of 128-row tile (tr, tc) of the own slab, summed over all
  // ranks into `out`. Thread tid of 192 handles 16-byte vectors tid, tid + 192, ...: a warp covers
  // one 512-byte row segment per instruction. The item that finishes a tile last puts the tile's
  // counters back to zero. Not inlined: the reducer warps get their own register allocation
  // instead of sharing the epilogue's.
  __device__ __noinline__ bool reduce_item(const GemmParams& p, int tr, int tc, int sub, int tid, int slot, int group) {
    uint32_t* f = counter(p, p.rank, tr, tc);
    uint32_t* done = f + p.rs_done_off;
    const uint32_t need = (uint32_t)p.ws;
    if (tid == 0) {
      if (group == 0) trace_put(p, 2, slot, 0);
      spin_until([&] { return ld_acquire_sys(f) >= need; }, p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 57, 0, blockIdx.x));
      if (group == 0) trace_put(p, 2, slot, 1);
    }
    group_bar_sync(group);
    if (!status_ok(p.sync)) return false;
    const int N = p.rows_c;
    const int col0 = tc * bn;
    const int vpr = min(bn, N - col0) / 8;                       // N % 8 == 0
    const int lrow0 = tr * kBM - p.rank * p.slab_rows + sub * p.rs_sub_rows;
    const int rows = min(p.rs_sub_rows, p.slab_rows - lrow0);
    const int total = rows * vpr;
    if (!kr_in_bounds(lrow0 >= 0 && rows > 0 && lrow0 + rows <= p.slab_rows && col0 >= 0 && col0 + vpr * 8 <= N &&
                          (f - (p.peer_pad[p.rank] + p.flag_base)) < (long long)p.rs_done_off, p.sync, 71))
      return false;
    if (p.mc_ptr != nullptr) {
      // in-switch sum (pull only)
      const char* src = (const char*)p.mc_ptr + p.stage_off + (size_t)p.rank * slab_bytes(p) + ((size_t)lrow0 * N + col0) * 2;
      constexpr int B = 4;
      for (int i0 = tid; i0 < total; i0 += kRsReducerThreads * B) {
        U4 x[B];
#pragma unroll
        for (int k = 0; k < B; ++k) {
          const int i = i0 + k * kRsReducerThreads;
          if (i < total) {
            const int r = i / vpr, v = i - r * vpr;
            x[k] = multimem_ld_reduce_bf16x8(src + ((size_t)r * N + v * 8) * 2);
          }
        }
#pragma unroll
        for (int k = 0; k < B; ++k) {
          const int i = i0 + k * kRsReducerThreads;
          if (i < total) {
            const int r = i / vpr, v = i - r * vpr;
            st16((char*)p.out + ((size_t)(lrow0 + r) * p.ldo + col0 + v * 8) * 2, x[k]);
          }
        }
      }
    } else if (p.ws <= 2) {
      reduce_loads<4, 2>(p, tid, total, vpr, lrow0, col0);
    } else if (p.ws <= 4) {
      reduce_loads<2, 4>(p, tid, total, vpr, lrow0, col0);
    } else {
      reduce_loads<1, 8>(p, tid, total, vpr, lrow0, col0);
    }
    group_bar_sync(group);                        // every thread's loads of this item have returned
    if (tid == 0) {
      if (atomicAdd(done, 1u) == (uint32_t)(kBM / p.rs_sub_rows - 1)) {
        *done = 0u;
        red_add_relaxed_sys(f, 0u - need);     // zero again for the call after next (the next uses the other bank)
      }
      if (group == 0) trace_put(p, 2, slot, 2);
    }
    return true;
  }

  // Work items. The items of the own slab are numbered in the order their tiles are computed
  // (tile_coords with pivot 0: row groups; inside a group column by column; inside a column the
  // group's rows; virtual row v belongs to rank v % ws and is row tile rank*per_slab + v/ws; a pair
  // tile: upper half first) and this CTA serves items me, me + num_ctas, ... . Item number -> tile
  // costs one division: earlier versions that walked the tile order tile by tile (a serial integer
  // chain on one warp) spent longer finding the next item than reducing it. Two groups of 192
  // threads take this CTA's items off one shared counter: the reducer warps from the start of the
  // kernel, the six pipeline warps once their last tile is stored — so the items of the last wave,
  // which nothing can overlap, are split between both groups.
  __device__ __forceinline__ unsigned* claim_words() {
    __shared__ unsigned words[4];      // [0] next item of this CTA; [1], [2] item just claimed by group 0 / 1
    return words;
  }
  __device__ __forceinline__ void setup(const GemmParams&) { claim_words()[0] = 0u; }

  __device__ __forceinline__ void serve_items(const GemmParams& p, unsigned worker, unsigned num_workers, int half, int tid,
                                              int group) {
    const unsigned halves = half < 0 ? 1u : 2u;
    const unsigned me = half < 0 ? worker : 2u * worker + (unsigned)half;
    const unsigned num_ctas = num_workers * halves;
    const unsigned subs = (unsigned)(kBM / p.rs_sub_rows);           // 1, 2, 4 or 8
    const unsigned per_tile = halves * subs;                          // a power of two
    const unsigned tile_shift = (unsigned)__ffs((int)per_tile) - 1u;
    const unsigned sub_shift = (unsigned)__ffs((int)subs) - 1u;
    const int per_slab = p.tiles_r / p.ws;                            // row tiles (of this kernel's tile height) per slab
    const unsigned total_items = ((unsigned)per_slab * (unsigned)p.tiles_c) << tile_shift;
    const unsigned my_items = me < total_items ? (total_items - me + num_ctas - 1u) / num_ctas : 0u;
    unsigned* words = claim_words();
    int served = 0;
    while (true) {
      if (tid == 0) words[1 + group] = atomicAdd(&words[0], 1u);
      group_bar_sync(group);
      const unsigned i = words[1 + group];
      if (i >= my_items) break;
      const unsigned id = me + i * num_ctas;
      const unsigned o = id >> tile_shift, k = id & (per_tile - 1u);
      // the row group that holds own tile o: [first, gend), its own rows v0, v0 + ws, ... (n_g of them)
      int first = 0, gend = min(p.group_r, p.tiles_r);
      int v0 = p.rank % p.ws;
      int n_g = v0 < gend ? (gend - 1 - v0) / p.ws + 1 : 0;
      unsigned o_base = 0;
      while (o >= o_base + (unsigned)(n_g * p.tiles_c)) {
        o_base += (unsigned)(n_g * p.tiles_c);
        first += p.group_r;
        gend = min(first + p.group_r, p.tiles_r);
        v0 = first + (p.rank - first % p.ws + p.ws) % p.ws;
        n_g = v0 < gend ? (gend - 1 - v0) / p.ws + 1 : 0;
      }
      const int idx = (int)(o - o_base);
      const int tc = idx / n_g, j = idx - tc * n_g;
      const int trv = p.rank * per_slab + v0 / p.ws + j;              // (v0 + j*ws) / ws
      const int tr = half < 0 ? trv : 2 * trv + (int)(k >> sub_shift);
      if (tr * kBM < p.rows_r && !reduce_item(p, tr, tc, (int)(k & (subs - 1u)), tid, served++, group)) return;
    }
  }
  __device__ __forceinline__ void side_role(const GemmParams& p, unsigned worker, unsigned num_workers, int half, int tid) {
    serve_items(p, worker, num_workers, half, tid, 0);
  }
  __device__ __forceinline__ void helper_role(const GemmParams& p, unsigned worker, unsigned num_workers, int half, int tid) {
    if (blockDim.x > (unsigned)kGemmThreads) serve_items(p, worker, num_workers, half, tid, 1);
  }
};

// ---------------------------------------------------------------------------------------------
// kernels: ALGO 0 push (192 threads), 1 pull / scatter (192 + 192 reducer threads)
// ---------------------------------------------------------------------------------------------
template <int ALGO>
__device__ __forceinline__ void rs_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  if (ALGO == 0) {
    RsPushHooks h;
    h.bn = 256;
    gemm_mainloop<256>(p, bid, nb, h, smem_raw);
    // staging slabs and flags may be reused by the next launch only after every rank is done
    symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 56);
  } else {
    RsPullHooks h;
    h.bn = 256;
    gemm_mainloop<256>(p, bid, nb, h, smem_raw);
  }
}
template <int ALGO>
__device__ __forceinline__ void rs_pair_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  if (ALGO == 0) {
    RsPushHooks h;
    h.bn = 256;
    gemm_mainloop_pair(p, bid / 2, nb / 2, h, smem_raw);
    symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 56);
  } else {
    RsPullHooks h;
    h.bn = 256;
    gemm_mainloop_pair(p, bid / 2, nb / 2, h, smem_raw);
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1) gemm_rs_push_kernel(const __grid_constant__ GemmParams p) {
  rs_body<0>(p, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_rs_push_emu_kernel(const GemmParams* ps) {
  rs_body<0>(ps[blockIdx.y], blockIdx.x, gridDim.x);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_rs_push_pair_kernel(const __grid_constant__ GemmParams p) {
  rs_pair_body<0>(p, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(kRsPullThreads, 1) gemm_rs_pull_kernel(const __grid_constant__ GemmParams p) {
  rs_body<1>(p, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(kRsPullThreads, 1) gemm_rs_pull_emu_kernel(const GemmParams* ps) {
  rs_body<1>(ps[blockIdx.y], blockIdx.x, gridDim.x);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kRsPullThreads, 1)
    gemm_rs_pull_pair_kernel(const __grid_constant__ GemmParams p) {
  rs_pair_body<1>(p, blockIdx.x, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------------------------
struct RsPlan {
  int pair;            // 1: CTA-pair kernel with 256 x 256 tiles, 0: single-CTA kernel with 128 x 256 tiles
  int tiles_r, tiles_c;
  int group_r, pivot_r, interleave_r;
  int workers;         // CTA pairs (pair) or CTAs that walk the tile order
  int grid;            // CTAs launched
  int sub_rows;        // pull / scatter: rows of a reduce work item
};

// Tiling and tile order of the fused reduce-scatter GEMM; one function for the launcher and for
// the host-side model of the flag protocol used by the tests.
static int rs_plan(int M, int N, int ws, int rank, int algo, unsigned cap, bool allow_pair, RsPlan* pl) {
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(M % ws == 0 && (M / ws) % kBM == 0, "fused GEMM reduce-scatter needs (M / world_size) % 128 == 0");
  KR_REQUIRE(N >= 256 && N % 8 == 0, "fused GEMM reduce-scatter needs N >= 256 and N % 8 == 0");
  KR_REQUIRE(cap >= 1, "no CTAs");
  const int slab_rows = M / ws;
  pl->pair = allow_pair && cap >= 2 && (slab_rows % 256) == 0 ? 1 : 0;
  const int rows_per_tile = pl->pair ? 256 : kBM;
  const int per_slab = slab_rows / rows_per_tile;
  pl->tiles_r = M / rows_per_tile;
  pl->tiles_c = (N + 255) / 256;
  int g = default_group_r();                    // counted in 128-row tiles
  if (pl->pair) g = g >= 2 ? g / 2 : 1;
  if (algo == 0) {
    // next rank's slab first, own slab last; groups never straddle two slabs
    pl->pivot_r = (((rank + 1) % ws) * per_slab) % pl->tiles_r;
    pl->interleave_r = 0;
    if (g > per_slab) g = per_slab;
    while (per_slab % g) --g;
  } else {
    // the same order on every rank, owners interleaved
    pl->pivot_r = 0;
    pl->interleave_r = ws;
    if (g > pl->tiles_r) g = pl->tiles_r;
  }
  pl->group_r = g;
  pl->sub_rows = kBM;
  while (pl->sub_rows > 16 && pl->sub_rows * ws > kBM) pl->sub_rows /= 2;   // about 128 / ws, at least 16
  const unsigned tiles = (unsigned)pl->tiles_r * (unsigned)pl->tiles_c;
  if (pl->pair) {
    unsigned pairs = tiles < cap / 2 ? tiles : cap / 2;
    pl->workers = (int)pairs;
    pl->grid = (int)(2 * pairs);
  } else {
    unsigned n = tiles < cap ? tiles : cap;
    pl->workers = (int)n;
    pl->grid = (int)n;
  }
  return KR_SUCCESS;
}

static unsigned long long* g_rs_trace = nullptr;
static unsigned long long g_rs_trace_words = 0;

}  // namespace kraken

using namespace kraken;

// Per-tile timeline of the next reduce-scatter GEMM launches on this process: `buf` is device memory
// of `words` 64-bit words (at least CTAs * 3 * 64 * 4), or nullptr to switch the timeline off.
KR_API int kr_gemm_rs_set_trace(unsigned long long* buf, unsigned long long words) {
  g_rs_trace = buf;
  g_rs_trace_words = words;
  return KR_SUCCESS;
}

// out[0..8] = {pair, tiles_r, tiles_c, group_r, pivot_r, interleave_r, workers, grid, sub_rows} for the
// given problem on a device with `num_ctas` CTAs available. For tests of the flag protocol.
KR_API int kr_rs_plan(int M, int N, int ws, int rank, int algo, int num_ctas, int allow_pair, int* out) {
  RsPlan pl;
  int rc = rs_plan(M, N, ws, rank, algo, (unsigned)num_ctas, allow_pair != 0, &pl);
  if (rc) return rc;
  out[0] = pl.pair; out[1] = pl.tiles_r; out[2] = pl.tiles_c; out[3] = pl.group_r;
  out[4] = pl.pivot_r; out[5] = pl.interleave_r; out[6] = pl.workers; out[7] = pl.grid;
  out[8] = pl.sub_rows;
  return KR_SUCCESS;
}

// Fused GEMM -> reduce-scatter. a[M, K_local], bt[N, K_local]; out[M/ws, N] bf16.
// bufs[r] = rank r's staging workspace (bufs: device table; bufs_host: the same addresses in host
// memory, used to describe staging to TMA, or nullptr; pads_host likewise for the signal pads): push needs M*N*2 bytes, pull and scatter
// 2*M*N*2 (two halves, alternating with call_parity) and DEDICATED to this op. mc_ptr: multicast
// address of the staging workspace (pull then sums in the NVSwitch) or nullptr (peer loads).
// algo: 0 push, 1 pull, 2 scatter. Tile counters live in the signal pads from word flag_base on
// (zero on entry, zero again after the call); pull and scatter use the bank selected by call_parity.
KR_API int kr_gemm_rs_bf16(void* const* bufs, void* const* bufs_host, uint32_t* const* pads,
                           uint32_t* const* pads_host, void* mc_ptr, int rank,
                           int ws, const void* a, long long lda, const void* bt, long long ldb, void* out,
                           long long ldo, int M, int N, int K, int algo, int call_parity, uint32_t pad_base,
                           uint32_t flag_base, unsigned long long pad_words, unsigned long long staging_bytes,
                           cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(algo >= 0 && algo <= 2, "algo must be 0 (push), 1 (pull) or 2 (scatter)");
  KR_REQUIRE(pad_base % (ws > 0 ? ws : 1) == 0, "pad_base must be a multiple of the world size");
  KR_REQUIRE(ldo % 8 == 0 && ((uintptr_t)out & 15) == 0, "output rows must be 16-byte aligned");
  const unsigned cap = grid_cap(d);
  RsPlan pl;
  int rc = rs_plan(M, N, ws, rank, algo == 0 ? 0 : 1, cap, pair_enabled() && !emu_recorder().active, &pl);
  if (rc) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  int bn = 0;
  rc = setup_problem(p, a, lda, bt, ldb, M, N, K, false, 256, &bn);
  if (rc) return rc;
  p.mode = GEMM_RS;
  p.rs_algo = algo;
  p.out = out;
  p.ldo = ldo;
  p.out_rows = M / ws;
  p.out_cols = N;
  p.rank = rank;
  p.ws = ws;
  p.bufs = bufs;
  p.pads = pads;
  p.pad_base = pad_base;
  p.slab_rows = M / ws;
  p.sync = sync_ctx(d);
  const unsigned long long mn2 = (unsigned long long)M * N * 2;
  const unsigned long long units = (unsigned long long)(p.slab_rows / kBM) * pl.tiles_c;
  if (algo == 0) {
    KR_REQUIRE(staging_bytes >= mn2, "staging workspace too small");
    KR_REQUIRE((unsigned long long)flag_base + units <= pad_words, "signal pad too small for the tile flags");
    KR_REQUIRE((unsigned long long)pad_base + (unsigned long long)cap * ws <= flag_base, "barrier slots overlap tile flags");
    p.flag_base = flag_base;
    // TMA-store destinations: rank o's staging slot [rank] for every o, and the local output.
    if (bufs_host != nullptr && ws <= 8) {
      bool ok = store_tmap(out, p.slab_rows, N, ldo, &p.tmap_out[ws]);
      for (int o = 0; o < ws && ok; ++o)
        ok = store_tmap((const char*)bufs_host[o] + (size_t)rank * p.slab_rows * N * 2, p.slab_rows, N, N, &p.tmap_out[o]);
      p.use_tma_store = ok ? 1 : 0;
    }
  } else {
    KR_REQUIRE(bufs_host != nullptr && pads_host != nullptr && ws <= 8,
               "pull and scatter need the peers' addresses on the host and world sizes up to 8");
    for (int r = 0; r < ws; ++r) {
      p.peer_buf[r] = bufs_host[r];
      p.peer_pad[r] = pads_host[r];
    }
    const unsigned long long half = staging_bytes / 2 / 1024 * 1024;
    KR_REQUIRE(half >= mn2, "staging workspace too small (pull and scatter need 2 * M * N * 2 bytes)");
    KR_REQUIRE(pad_words > flag_base, "signal pad too small for the tile counters");
    const unsigned long long bank = (pad_words - flag_base) / 2;
    KR_REQUIRE(2 * units <= bank, "signal pad too small for the tile counters");
    p.stage_off = (call_parity & 1) ? half : 0;
    p.flag_base = flag_base + ((call_parity & 1) ? (uint32_t)bank : 0u);
    p.rs_done_off = (uint32_t)units;           // per tile: [arrivals][work items done]
    p.rs_sub_rows = pl.sub_rows;
    p.mc_ptr = algo == 1 ? mc_ptr : nullptr;
    if (bufs_host != nullptr && algo == 1) {
      p.use_tma_store = store_tmap((const char*)bufs_host[rank] + p.stage_off, M, N, N, &p.tmap_out[0]) ? 1 : 0;
    } else if (bufs_host != nullptr && ws <= 8) {
      bool ok = true;
      for (int o = 0; o < ws && ok; ++o)
        ok = store_tmap((const char*)bufs_host[o] + p.stage_off + (size_t)rank * p.slab_rows * N * 2, p.slab_rows, N, N,
                        &p.tmap_out[o]);
      p.use_tma_store = ok ? 1 : 0;
    }
  }
  p.tiles_r = pl.tiles_r;
  p.tiles_c = pl.tiles_c;
  p.group_r = pl.group_r;
  p.pivot_r = pl.pivot_r;
  p.interleave_r = pl.interleave_r;
  p.num_mma_ctas = pl.grid;
  if (g_rs_trace != nullptr && !emu_recorder().active) {
    KR_REQUIRE(g_rs_trace_words >= (unsigned long long)pl.grid * kTraceRoles * kTraceTiles * kTraceFields,
               "trace buffer too small for this launch");
    p.trace = g_rs_trace;
  }
  const unsigned threads = algo == 0 ? kGemmThreads : kRsPullThreads;
  if (pl.pair) {
    // each CTA of a pair loads its own 128 rows of the column operand: box of 128 rows, not 256
    rc = get_tmap(p.host_c_ptr, p.rows_c, p.K, p.host_ldc, 128, &p.tmap_c);
    if (rc) return rc;
    const void* fn = algo == 0 ? (const void*)gemm_rs_push_pair_kernel : (const void*)gemm_rs_pull_pair_kernel;   // pull kernel also runs scatter
    rc = ensure_dynamic_smem(fn, PairCfg::SMEM);
    if (rc) return rc;
    void* args[] = {(void*)&p};
    KR_CUDA(cudaLaunchKernel(fn, dim3((unsigned)pl.grid), dim3(threads), args, PairCfg::SMEM, stream));
    return KR_SUCCESS;
  }
  if (algo == 0)
    return launch_ranked(gemm_rs_push_kernel, gemm_rs_push_emu_kernel, p, (unsigned)pl.grid, threads, GemmCfg<256>::SMEM, stream);
  return launch_ranked(gemm_rs_pull_kernel, gemm_rs_pull_emu_kernel, p, (unsigned)pl.grid, threads, GemmCfg<256>::SMEM, stream);
}
