// Persistent, warp-specialised tcgen05 GEMM core shared by the plain GEMM and by the fused
// all-gather->GEMM, GEMM->reduce-scatter and GEMM->all-reduce kernels.
//
//   D[128 x BN] tile = R[128 rows, K] * C[BN rows, K]^T      (both operands K-major, bf16)
//
// R ("row operand") and C ("column operand") are any two K-major matrices described by TMA
// tensor maps; the host decides which of the user's A / B^T plays which role (for decode-sized
// M the weights are the row operand and the epilogue stores the tile transposed).
//
// Warp roles in a 192-thread CTA (one CTA per SM):
//   warp 0     TMA producer: fills a ring of shared-memory stages (128-byte swizzle)
//   warp 1     allocates TMEM, one elected lane issues tcgen05.mma into one of two accumulators
//   warps 2-5  epilogue: tcgen05.ld the finished accumulator, convert, stage through shared
//              memory and write coalesced rows to local or PEER memory, while warp 1 already
//              runs the next tile's main loop into the other accumulator.
//   warps 6+   (only in kernels launched with more than 192 threads) a side role supplied by the
//              hooks, e.g. the reducer warps of the GEMM -> reduce-scatter kernel
// The reference's main loops are tl.dot recipes (kraken/fused/all_gather_matmul.py:25-123,
// kraken/fused/gemm_reduce_scatter_ce_persistent.py:46-134,
// kraken/fused/gemm_one_shot_all_reduce_fused.py:10-103); nothing of their structure is reused.
#pragma once
#include "kraken/tcgen05.cuh"
#include "kraken/vec.cuh"

namespace kraken {

constexpr int kGemmThreads = 192;
constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kEpiWarpBytes = 8192;             // per-epilogue-warp staging: 32 rows x 256 B
constexpr int kSmemLimit = 232448;              // 227 KB

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = kBM * kBK * 2;
  static constexpr int B_BYTES = BN * kBK * 2;
  static constexpr int B_BYTES_AL = (B_BYTES + 1023) / 1024 * 1024;
  static constexpr int STAGE = A_BYTES + B_BYTES_AL;
  static constexpr int EPI = 4 * kEpiWarpBytes;
  static constexpr int RAW_STAGES = (kSmemLimit - 1024 /*align*/ - EPI - 512 /*barriers*/) / STAGE;
  static constexpr int STAGES = RAW_STAGES > 8 ? 8 : RAW_STAGES;
  static constexpr int TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  static constexpr int SMEM = 1024 + STAGES * STAGE + EPI + 512;
};

enum GemmMode : int { GEMM_PLAIN = 0, GEMM_AG = 1, GEMM_RS = 2, GEMM_AR = 3, GEMM_CE = 4 };

struct alignas(64) GemmParams {
  CUtensorMap tmap_r;        // row operand, dims {K, rows_r}, box {64, 128}
  CUtensorMap tmap_c;        // column operand, dims {K, rows_c}, box {64, BN}
  CUtensorMap tmap_r_local;  // AG: this rank's own shard (read without waiting)
  // problem
  int rows_r, rows_c, K;
  int tiles_r, tiles_c;      // tile counts
  int group_r;               // consecutive row-tiles sharing column sweeps (L2 reuse)
  int pivot_r;               // row-tile rotation (rank pivot)
  int interleave_r;          // > 1: row tiles are dealt round-robin over this many equal slabs
  int mode;
  int transposed;            // 1: D tile is C^T (store element (i,j) at out[j][i])
  int out_fp32;              // 1: fp32 output, 0: bf16
  int in_fp32;               // 1: fp32 operands multiplied as tf32 (single-CTA kernels), 0: bf16
  int num_mma_ctas;          // CTAs [0, num_mma_ctas) run the GEMM; the rest are comm CTAs (AG)
  // output (PLAIN / AG / final result of RS and AR)
  // TMA-store destinations (bf16 row-major): [0] = `out`; GEMM->RS: [o] = rank o's staging slot for
  // this rank's tiles, [ws] = `out`. Valid when use_tma_store != 0.
  CUtensorMap tmap_out[9];
  int use_tma_store;
  void* out;
  long long ldo;             // elements between consecutive output rows
  int out_rows, out_cols;    // bounds of `out` in the orientation it is stored
  // collectives
  int rank, ws;
  void* const* bufs;         // [ws] symmetric workspaces (RS/AR staging, AG shards)
  uint32_t* const* pads;     // [ws] signal pads
  // The same addresses by value (world sizes up to 8, filled by launchers that know them on the
  // host): read from the kernel's parameter space instead of through two dependent global loads.
  void* peer_buf[8];
  uint32_t* peer_pad[8];
  uint32_t pad_base;         // first barrier slot
  uint32_t flag_base;        // first tile-flag word in the signal pad (RS / AR)
  // AG
  void* a_out;               // gathered A [ws * shard_rows, K]
  uint32_t* progress;        // [ws * splits] chunk flags
  uint32_t* counters;        // [ws * splits] arrival counters (zeroed, self-resetting)
  int splits, shard_rows, chunk_rows;
  const void* ag_shard;      // push: this rank's own shard [shard_rows, K]
  int ag_chunk_major;        // > 0: row tiles after the own shard go chunk by chunk over all peers (tiles per chunk)
  int ag_tiles_per_shard;    // row tiles (of this kernel's tile height) per shard, for ag_chunk_major
  void* ag_mc_out;           // multicast address of the gathered buffer (multicast push) or nullptr
  uint32_t* ag_mc_flags;     // multicast address of this call's chunk flags (multicast push)
  int ag_mc_weak;            // 1: the shard goes out with weak multimem stores (ordered by the flag's release)
  int ag_push;               // 1: every rank pushes its shard into the peers' gathered buffers (comm CTAs)
  int ag_entry_barrier;      // push into a caller-owned symmetric a_out: wait until every rank has entered
  unsigned long long ag_out_off;   // push: byte offset of the gathered buffer inside bufs[r]
  // AR (decode): byte offsets inside every rank's staging buffer and the second flag bank
  int ar_algo;               // 0: one-shot pull, 1: two-shot (tile owner reduces and publishes)
  unsigned long long stage_off;   // one-shot: this call's staging (alternates between two halves)
  unsigned long long part_off;    // two-shot: per-source partial tiles [ws][M][N] fp32
  unsigned long long res_off;     // two-shot: reduced result [M][N] fp32
  uint32_t flag2_base;            // two-shot: "result published" flags
  void* mc_ptr;                   // multicast address of the staging buffer (NVLS) or nullptr
  // Split-K (single-CTA kernels): with k_splits > 1 the persistent index runs over
  // k_splits * tiles work items, item = split * tiles + tile, and an item multiplies only the K
  // blocks of its split; the hooks see the split as Hooks::k_split and combine the partial sums.
  int k_splits;
  // AR, tagged push: this call's tag (never 0) and the byte offset of its slot array
  // [ws * k_splits][M][N] of {fp32 value, tag} pairs inside every rank's staging buffer
  uint32_t ll_tag;
  unsigned long long ll_off;
  // AR, tagged two-shot: pairs per partial slot at a tile's owner (tiles of one owner, packed), and
  // the byte offset of the [M][N] array of tagged results inside every rank's staging buffer
  unsigned long long ll_slot_pairs;
  unsigned long long ll_res_off;
  unsigned long long ll_end;        // byte offset one past this call's tagged region (bounds checks of the debug build)
  // RS
  int slab_rows;             // M / ws
  int rs_algo;               // 0: push, owner reduces in its epilogue; 1: pull; 2: scatter (push + reducer warps)
  int rs_sub_rows;           // pull / scatter: rows of one reduce work item (power of two, 16 ... 128)
  uint32_t rs_done_off;      // pull / scatter: words from a tile's arrival counter to its "items done" counter
  SyncCtx sync;
  // optional per-tile timeline (nullptr: off): [CTA][role][tile slot][field] %globaltimer stamps
  unsigned long long* trace;
  // host-side bookkeeping (not read on the device): the column operand as given, so that a
  // launcher can re-encode its tensor map with another box height
  const void* host_c_ptr;
  long long host_ldc;
};

// Linear persistent tile index -> (row tile, column tile): row tiles advance in groups of
// `group_r` so that concurrently running CTAs share operand tiles in L2, then the row index is
// rotated by `pivot_r` (rank pivot of the fused kernels).
__host__ __device__ __forceinline__ void tile_coords(const GemmParams& p, int t, int& tr, int& tc) {
  const int per_group = p.group_r * p.tiles_c;
  const int g = t / per_group;
  const int first = g * p.group_r;
  const int gsz = (p.tiles_r - first) < p.group_r ? (p.tiles_r - first) : p.group_r;
  const int in = t - g * per_group;
  tr = first + in % gsz;
  tc = in / gsz;
  tr += p.pivot_r;
  if (tr >= p.tiles_r) tr -= p.tiles_r;
  // Interleaved slabs: consecutive row tiles of the order belong to consecutive slabs (owners), so
  // every owner's tiles finish at an even rate instead of slab after slab.
  if (p.interleave_r > 1) tr = (tr % p.interleave_r) * (p.tiles_r / p.interleave_r) + tr / p.interleave_r;
  // All-gather GEMM fed by a multicast push: every peer's shard arrives chunk by chunk at the same
  // time, so after the own shard the order is chunk 0 of every peer, chunk 1 of every peer, ...
  // (`tr` counts positions from the start of the own shard; pivot_r is not used in this mode).
  if (p.ag_chunk_major > 0) {
    const int T = p.ag_tiles_per_shard, C = p.ag_chunk_major;
    if (tr < T) {
      tr += p.rank * T;
    } else {
      const int j = tr - T, round = (p.ws - 1) * C;
      const int c = j / round, r = j - c * round;
      const int s = r / C + 1, t = r - (s - 1) * C;
      int src = p.rank + s;
      if (src >= p.ws) src -= p.ws;
      tr = src * T + c * C + t;
    }
  }
}

// Per-tile timeline for performance work: when GemmParams::trace is set, one thread per role
// stamps %globaltimer at fixed points of every tile it handles (first kTraceTiles tiles per CTA).
//   role 0 (MMA issuer):  0 accumulator free, 1 first operand stage landed, 2 last MMA issued
//   role 1 (epilogue):    0 accumulator complete, 1 tile stored (stores issued), 2 completion hook done
//   role 2 (side role):   0 wait begins, 1 wait over, 2 work item done
constexpr int kTraceTiles = 64;
constexpr int kTraceRoles = 3;
constexpr int kTraceFields = 4;
__device__ __forceinline__ void trace_put(const GemmParams& p, int role, int slot, int field) {
  if (p.trace != nullptr && slot < kTraceTiles)
    p.trace[(((size_t)blockIdx.x * kTraceRoles + role) * kTraceTiles + slot) * kTraceFields + field] = globaltimer_ns();
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Hooks a fused kernel supplies to the main loop.
//   Producer hook: called by the producer lane before loading row tile `tr`; returns the tensor
//   map to read it from and may rewrite the row coordinate; false aborts.
//   Epilogue hooks: begin_tile (may wait for peers' data), tile_dest (where tile (tr, tc) is
//   stored), add_to_chunk (adds other ranks' partial sums to a row fragment still in registers;
//   row-major path only), after_store (what happens once the tile is stored), may_wait (whether
//   begin_tile of that row tile can block on another rank: the main loop then first runs any
//   completion hook it still holds back, so that no rank waits while it withholds a signal),
//   side_role (work of the warps beyond the six pipeline warps, if the launch has any),
//   helper_role (what the six pipeline warps do after their last tile, before the teardown).
struct HookDefaults {
  int k_split = 0;           // which K split the tile in hand belongs to (set by the main loop)
  __device__ __forceinline__ bool may_wait(const GemmParams&, int) const { return false; }
  // worker / num_workers: this CTA (or CTA pair) among those of the launch; half: -1 for a single
  // CTA, else the CTA's rank inside its pair; tid: thread index among the side-role warps.
  __device__ __forceinline__ void side_role(const GemmParams&, unsigned, unsigned, int, int) {}
  // setup: thread 0, before the block's first barrier. helper_role: the six pipeline warps once
  // their own roles are over (all tiles of this CTA computed and stored), tid in [0, 192).
  __device__ __forceinline__ void setup(const GemmParams&) {}
  __device__ __forceinline__ void helper_role(const GemmParams&, unsigned, unsigned, int, int) {}
};

struct TileDest {
  char* base;        // address of element (0,0) of the destination matrix
  long long ld;      // elements per destination row
  int row0, col0;    // where the tile's (0,0) lands in the destination
  int rows, cols;    // destination bounds
  const CUtensorMap* tmap;   // bf16 destination as a tensor map (box 64 columns x 32 rows, 128-byte
                             // swizzle) for TMA stores, or nullptr: plain vector stores
  // Tagged push (transposed fp32 tiles only): when ll_tag != 0 every element goes, as an 8-byte
  // {value, tag} pair, to byte offset ll_off + 8 * (row * ld + column) of EVERY rank's staging
  // buffer (GemmParams::peer_buf) instead of to `base`.
  uint32_t ll_tag = 0;
  unsigned long long ll_off = 0;
  // The pair of element (row, column) sits at ll_off + 8 * ((row - ll_row0) * ll_ld + (column - ll_col0));
  // ll_ld == 0 means the destination's own `ld`. ll_dst >= 0: only that rank receives it.
  int ll_row0 = 0, ll_col0 = 0;
  long long ll_ld = 0;
  int ll_dst = -1;
};

// Epilogue of one tile, run by the four epilogue warps: TMEM -> registers -> (hook: add peers'
// partial sums) -> convert -> swizzled staging in shared memory -> coalesced global stores.
// `tempty_addr` is the mbarrier that returns the accumulator to the MMA issuer: a local barrier,
// or (PAIR) the shared::cluster address of the barrier in the pair's leader CTA.
template <int BN, bool PAIR, class Hooks>
__device__ __forceinline__ bool gemm_epilogue_tile(const GemmParams& p, Hooks& hooks, int tr, int tc, int acc,
                                                   uint32_t tmem_base, int q, int lane, unsigned char* stg,
                                                   uint32_t tempty_addr, bool defer) {
  if (!hooks.begin_tile(p, tr, tc, q, lane)) return false;
  TileDest dst = hooks.tile_dest(p, tr, tc);
  const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
  if (p.transposed) {
    // D(i, j) -> dst[col0 + j][row0 + i]: lanes = consecutive destination columns.
    const int dcol = dst.row0 + q * 32 + lane;     // destination column index (tile row i)
    constexpr int CH = BN < 32 ? BN : 32;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += CH) {
      uint32_t r[32];
      if (CH == 32) tmem_ld32(t_addr + c0, r);
      else tmem_ld16(t_addr + c0, r);
      tmem_ld_wait();
      if (c0 + CH >= BN) {
        // all TMEM reads of this accumulator are done: hand it back before the global stores
        tc_fence_before();
        __syncwarp();
        if (lane == 0) { if (PAIR) mbar_arrive_cluster(tempty_addr); else mbar_arrive(tempty_addr); }
      }
      if (dcol < dst.cols) {
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int drow = dst.col0 + c0 + j;
          if (drow < dst.rows) {
            if (dst.ll_tag != 0) {
              const unsigned long long o =
                  dst.ll_off + 8ull * ((unsigned long long)(drow - dst.ll_row0) * (dst.ll_ld ? dst.ll_ld : dst.ld) +
                                       (unsigned long long)(dcol - dst.ll_col0));
              const unsigned long long v = ((unsigned long long)dst.ll_tag << 32) | r[j];
              if (!kr_in_bounds(o >= p.ll_off && o + 8 <= p.ll_end, p.sync, 76)) continue;
              if (dst.ll_dst >= 0) {
                st_relaxed_sys_u64((char*)p.peer_buf[dst.ll_dst] + o, v);
              } else {
                for (int d = 0; d < p.ws; ++d) st_relaxed_sys_u64((char*)p.peer_buf[d] + o, v);
              }
            } else if (p.out_fp32) ((float*)dst.base)[(long long)drow * dst.ld + dcol] = __uint_as_float(r[j]);
            else ((__nv_bfloat16*)dst.base)[(long long)drow * dst.ld + dcol] = __float2bfloat16(__uint_as_float(r[j]));
          }
        }
      }
    }
  } else if (BN >= 64 && !p.out_fp32 && dst.tmap != nullptr) {
    // bf16 row-major tile through TMA stores. The warp's 32 rows are staged as panels of 64 columns
    // (32 rows x 128 bytes, 16-byte chunks XOR-swizzled by row: the layout a 128-byte-swizzle
    // tensor map expects, and conflict-free for the row-per-lane writes); one elected lane stores
    // each panel with a single bulk tensor copy, to local or PEER memory. Two panel slots alternate.
    // The TMA engine keeps far more bytes in flight towards a peer than the SM's store path does.
    constexpr int PANELS = BN / 64;
#pragma unroll 1
    for (int pn = 0; pn < PANELS; ++pn) {
      unsigned char* slot = stg + (pn & 1) * 4096;
      // The store that last read this slot (two panels ago, possibly in the previous tile) must be
      // done with it; only the most recent group (the other slot) may still be reading.
      if (lane == 0) {
        if (PANELS == 1) bulk_wait_group_read<0>();
        else bulk_wait_group_read<1>();
      }
      __syncwarp();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        const int col = pn * 64 + c * 32;
        tmem_ld32(t_addr + col, r);
        tmem_ld_wait();
        if (pn == PANELS - 1 && c == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (PAIR) mbar_arrive_cluster(tempty_addr); else mbar_arrive(tempty_addr); }
        }
        hooks.add_to_chunk(p, tr, tc, q * 32 + lane, col, r, 32);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int chunk = c * 4 + u;
          const int phys = chunk ^ (lane & 7);
          U4 v;
          v.x = pack_bf16x2(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
          v.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
          v.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
          v.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
          *(U4*)(slot + lane * 128 + phys * 16) = v;
        }
      }
      fence_proxy_async_smem();       // staged bytes visible to the TMA engine
      __syncwarp();
      const int gx = dst.col0 + pn * 64, gy = dst.row0 + q * 32;
      if (lane == 0) {
        if (gx < dst.cols && gy < dst.rows) tma_store_2d(dst.tmap, smem_u32(slot), gx, gy);
        bulk_commit_group();           // one group per panel, empty or not, so groups can be counted
      }
    }
    // A tile's stores must be complete before the hook may tell anyone about them. Waiting for this
    // tile's own stores would put a peer round trip on every tile's epilogue; in deferred mode the
    // wait covers the PREVIOUS tile's groups (this tile's PANELS groups stay in flight) and the
    // caller runs the previous tile's hook.
    if (lane == 0) {
      if (defer) bulk_wait_group<PANELS>();
      else bulk_wait_group<0>();
      fence_proxy_async();
    }
    __syncwarp();
  } else {
    // Row-major store through per-warp staging: 32 rows x 256 bytes, 16-byte units XOR-swizzled
    // by row so that both the row-per-lane writes and the row-contiguous reads are conflict-free.
    const int elt = p.out_fp32 ? 4 : 2;
    const int cols_per_pass = 256 / elt;               // 128 bf16 or 64 fp32 columns
    const int passes = (BN + cols_per_pass - 1) / cols_per_pass;
    const int pass_cols = BN < cols_per_pass ? BN : cols_per_pass;
    const int units_per_row = pass_cols * elt / 16;    // 16-byte units actually used per row
    const bool vec_ok = ((dst.ld * elt) % 16 == 0) && ((((uintptr_t)dst.base) & 15) == 0) && ((dst.col0 * elt) % 16 == 0);
    for (int ps = 0; ps < passes; ++ps) {
      constexpr int CH = BN < 32 ? BN : 32;
      const int nch = pass_cols / CH;
      for (int c = 0; c < nch; ++c) {
        uint32_t r[32];
        const int col = ps * cols_per_pass + c * CH;
        if (CH == 32) tmem_ld32(t_addr + col, r);
        else tmem_ld16(t_addr + col, r);
        tmem_ld_wait();
        if (ps == passes - 1 && c == nch - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) { if (PAIR) mbar_arrive_cluster(tempty_addr); else mbar_arrive(tempty_addr); }
        }
        hooks.add_to_chunk(p, tr, tc, q * 32 + lane, col, r, CH);
        if (p.out_fp32) {
#pragma unroll
          for (int u = 0; u < CH / 4; ++u) {
            const int unit = c * (CH / 4) + u;
            const int phys = (unit & 8) | ((unit ^ lane) & 7);
            *(U4*)(stg + lane * 256 + phys * 16) = U4{r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]};
          }
        } else {
#pragma unroll
          for (int u = 0; u < CH / 8; ++u) {
            const int unit = c * (CH / 8) + u;
            const int phys = (unit & 8) | ((unit ^ lane) & 7);
            U4 v;
            v.x = pack_bf16x2(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
            v.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
            v.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
            v.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
            *(U4*)(stg + lane * 256 + phys * 16) = v;
          }
        }
      }
      __syncwarp();
      // coalesced write-out: `rpi` rows per warp instruction
      const int rpi = 32 / units_per_row > 0 ? 32 / units_per_row : 1;
      const int unit = lane % units_per_row;
      const int rsub = lane / units_per_row;
      const int per_unit = 16 / elt;
      const int gcol = dst.col0 + ps * cols_per_pass + unit * per_unit;
      if (rsub < rpi) {
        for (int r0 = 0; r0 < 32; r0 += rpi) {
          const int rr = r0 + rsub;
          const int grow = dst.row0 + q * 32 + rr;
          const int phys = (unit & 8) | ((unit ^ rr) & 7);
          const U4 v = *(const U4*)(stg + rr * 256 + phys * 16);
          if (grow < dst.rows) {
            char* gp = dst.base + ((long long)grow * dst.ld + gcol) * elt;
            if (vec_ok && gcol + per_unit <= dst.cols) {
              st16(gp, v);
            } else {
              const uint32_t w[4] = {v.x, v.y, v.z, v.w};
              for (int e = 0; e < per_unit; ++e)
                if (gcol + e < dst.cols) {
                  if (p.out_fp32) ((uint32_t*)gp)[e] = w[e];
                  else ((uint16_t*)gp)[e] = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
                }
            }
          }
        }
      }
      __syncwarp();
    }
  }
  return true;
}

// ELT = bytes per operand element: 2 (bf16, kind::f16) or 4 (fp32 read as tf32, kind::tf32). A stage
// always holds 128-byte rows (64 bf16 or 32 fp32 along K) and feeds four MMAs of 32 bytes of K each.
template <int BN, class Hooks, int ELT = 2>
__device__ __forceinline__ void gemm_mainloop(const GemmParams& p, unsigned bid, unsigned nb, Hooks& hooks,
                                              unsigned char* smem_raw) {
  using Cfg = GemmCfg<BN>;
  constexpr int kStageK = 128 / ELT;            // operand elements along K per stage
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // ---- shared memory carve-up (1024-byte aligned for the 128-byte swizzle)
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t stage0 = smem_base;
  unsigned char* epi_ptr = smem_al + Cfg::STAGES * Cfg::STAGE;
  const uint32_t bars = smem_base + Cfg::STAGES * Cfg::STAGE + Cfg::EPI;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + 2 + a); };
  uint32_t* tmem_slot = (uint32_t*)(smem_al + Cfg::STAGES * Cfg::STAGE + Cfg::EPI + 8 * (2 * Cfg::STAGES + 4));

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_fence_init();
    hooks.setup(p);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_rc = p.tiles_r * p.tiles_c;
  const int ksp = p.k_splits > 1 ? p.k_splits : 1;
  const int total_tiles = tiles_rc * ksp;
  const int num_kb = (p.K + kStageK - 1) / kStageK;
  // work item t -> (tile, K-block range): split-major, so one wave of CTAs covers every tile once
  auto item_of = [&](int t, int& tile, int& split, int& kb_lo, int& kb_hi) {
    split = ksp > 1 ? t / tiles_rc : 0;
    tile = t - split * tiles_rc;
    kb_lo = (int)((long long)num_kb * split / ksp);
    kb_hi = (int)((long long)num_kb * (split + 1) / ksp);
  };

  if (warp == 0) {
    // ================= TMA producer =================
    if (elect_one()) {
      tma_prefetch_desc(&p.tmap_r);
      tma_prefetch_desc(&p.tmap_c);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = bid; t < total_tiles && ok; t += nb) {
        int tr, tc, tile, split, kb_lo, kb_hi;
        item_of(t, tile, split, kb_lo, kb_hi);
        tile_coords(p, tile, tr, tc);
        const CUtensorMap* rmap = &p.tmap_r;
        int row0 = tr * kBM;
        ok = hooks.before_load(p, tr, rmap, row0);
        for (int kb = kb_lo; kb < kb_hi && ok; ++kb) {
          ok = mbar_wait(empty_bar(s), ph ^ 1u, p.sync, 40);
          if (!ok) break;
          mbar_expect_tx(full_bar(s), Cfg::A_BYTES + Cfg::B_BYTES);
          const uint32_t sa = stage0 + s * Cfg::STAGE;
          tma_load_2d(sa, rmap, full_bar(s), kb * kStageK, row0);
          tma_load_2d(sa + Cfg::A_BYTES, &p.tmap_c, full_bar(s), kb * kStageK, tc * BN);
          if (++s == Cfg::STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (elect_one()) {
      constexpr uint32_t idesc = ELT == 2 ? make_idesc_bf16(kBM, BN) : make_idesc_tf32(kBM, BN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = bid; t < total_tiles && ok; t += nb, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
        ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, p.sync, 41);
        if (!ok) break;
        tc_fence_after();
        trace_put(p, 0, it, 0);
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        int tile, split, kb_lo, kb_hi;
        item_of(t, tile, split, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          ok = mbar_wait(full_bar(s), ph, p.sync, 42);
          if (!ok) break;
          tc_fence_after();
          if (kb == kb_lo) trace_put(p, 0, it, 1);
          const uint32_t sa = stage0 + s * Cfg::STAGE;
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if (ELT == 2) umma_bf16(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > kb_lo || k != 0) ? 1u : 0u);
            else umma_tf32(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb > kb_lo || k != 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));   // frees the stage once these MMAs have read it
          if (++s == Cfg::STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));   // accumulator complete
        trace_put(p, 0, it, 2);
      }
    }
  } else if (warp >= 6) {
    hooks.side_role(p, bid, nb, -1, (int)threadIdx.x - kGemmThreads);
  } else {
    // ================= epilogue warps =================
    const int q = warp & 3;                                  // TMEM lane quarter this warp may read
    unsigned char* stg = epi_ptr + (warp - 2) * kEpiWarpBytes;
    // tiles leave through TMA stores: run each tile's completion hook one tile late (see the epilogue)
    const bool defer = BN >= 64 && !p.out_fp32 && !p.transposed && p.use_tma_store != 0;
    int prev_tr = -1, prev_tc = -1;
    int it = 0;
    bool ok = true;
    for (int t = bid; t < total_tiles && ok; t += nb, ++it) {
      int tr, tc, tile, split, kb_lo, kb_hi;
      item_of(t, tile, split, kb_lo, kb_hi);
      tile_coords(p, tile, tr, tc);
      hooks.k_split = split;
      const int acc = it & 1;
      const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
      ok = mbar_wait(tfull_bar(acc), acc_ph, p.sync, 43);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (q == 0 && lane == 0) trace_put(p, 1, it, 0);
      if (defer && prev_tr >= 0 && hooks.may_wait(p, tr)) {
        // never block on a peer while a finished tile's signal is still held back
        if (lane == 0) {
          bulk_wait_group<0>();
          fence_proxy_async();
        }
        __syncwarp();
        ok = hooks.after_store(p, prev_tr, prev_tc, q, lane);
        prev_tr = -1;
        if (!ok) break;
      }
      ok = gemm_epilogue_tile<BN, false>(p, hooks, tr, tc, acc, tmem_base, q, lane, stg, tempty_bar(acc), defer);
      if (!ok) break;
      if (q == 0 && lane == 0) trace_put(p, 1, it, 1);
      if (defer) {
        if (prev_tr >= 0) ok = hooks.after_store(p, prev_tr, prev_tc, q, lane);
        prev_tr = tr;
        prev_tc = tc;
      } else {
        ok = hooks.after_store(p, tr, tc, q, lane);
      }
      if (q == 0 && lane == 0) trace_put(p, 1, it, 2);
    }
    if (defer && prev_tr >= 0) {
      if (lane == 0) {
        bulk_wait_group<0>();
        fence_proxy_async();
      }
      __syncwarp();
      if (ok) hooks.after_store(p, prev_tr, prev_tc, q, lane);
    }
  }

  // The producer and MMA warps ran their roles on one elected lane: wait for it, so that the other
  // lanes do not start polling in the helper role while it still has tiles to feed.
  __syncwarp();
  if (warp < 6) hooks.helper_role(p, bid, nb, -1, (int)threadIdx.x);

  // ---- teardown: every role arrives here, on the normal path and after a failed wait
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}


// ---------------------------------------------------------------------------------------------
// CTA-pair variant: two CTAs of a 2-CTA cluster compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2. Each CTA TMA-loads (plain, non-multicast loads) its own 128 rows of the
// row operand and its own 128 rows of the column operand, so every stage moves 32 KB per CTA
// instead of 48 KB and six stages fit; the leader CTA (cluster rank 0) issues the MMAs, which
// read both CTAs' shared memory; each CTA keeps the accumulator rows of its own 128 rows in its
// own TMEM and runs the same epilogue as the single-CTA kernel on them.
//   full[s]    in the leader, 1 arrival (the leader's expect_tx for both CTAs' bytes) + the bytes
//   empty[s]   one per CTA, 1 arrival: the leader commits to its own and to the peer's barrier
//   tfull[a]   one per CTA, 1 arrival: same double commit
//   tempty[a]  in the leader, 8 arrivals: the four epilogue warps of each CTA
// ---------------------------------------------------------------------------------------------
struct PairCfg {
  static constexpr int BN = 256;                 // pair tile: 256 rows x 256 columns
  static constexpr int A_BYTES = kBM * kBK * 2;  // this CTA's 128 rows of the row operand
  static constexpr int B_BYTES = 128 * kBK * 2;  // this CTA's 128 rows of the column operand
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int EPI = 4 * kEpiWarpBytes;
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM = 1024 + STAGES * STAGE + EPI + 512;
};
static_assert(PairCfg::SMEM <= kSmemLimit, "pair kernel shared memory");

template <class Hooks>
__device__ __forceinline__ void gemm_mainloop_pair(const GemmParams& p, unsigned pair_id, unsigned num_pairs,
                                                   Hooks& hooks, unsigned char* smem_raw) {
  using Cfg = PairCfg;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();
  const bool leader = cta == 0;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t stage0 = smem_base;
  unsigned char* epi_ptr = smem_al + Cfg::STAGES * Cfg::STAGE;
  const uint32_t bars = smem_base + Cfg::STAGES * Cfg::STAGE + Cfg::EPI;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::STAGES + s); };
  auto tfull_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + a); };
  auto tempty_bar = [&](int a) { return bars + 8u * (2 * Cfg::STAGES + 2 + a); };
  uint32_t* tmem_slot = (uint32_t*)(smem_al + Cfg::STAGES * Cfg::STAGE + Cfg::EPI + 8 * (2 * Cfg::STAGES + 4));

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    mbar_fence_init();
    hooks.setup(p);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_r * p.tiles_c;      // tiles_r counts 256-row pair tiles here
  const int num_kb = (p.K + kBK - 1) / kBK;

  if (warp == 0) {
    // ================= TMA producer (both CTAs) =================
    if (elect_one()) {
      tma_prefetch_desc(&p.tmap_r);
      tma_prefetch_desc(&p.tmap_c);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int tr2, tc;
        tile_coords(p, t, tr2, tc);
        const int tr = 2 * tr2 + (int)cta;
        const CUtensorMap* rmap = &p.tmap_r;
        int row0 = tr * kBM;
        ok = hooks.before_load(p, tr, rmap, row0);
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          ok = mbar_wait(empty_bar(s), ph ^ 1u, p.sync, 44);
          if (!ok) break;
          const uint32_t lead_full = mapa_shared(full_bar(s), 0);
          // Only the leader arrives (with the byte count of BOTH CTAs); the peer's loads just
          // complete bytes on the leader's barrier. The peer cannot run a phase ahead: it waits for
          // its own empty barrier, which the leader signals after the MMAs that waited on full[s].
          if (leader) mbar_expect_tx(full_bar(s), 2 * (Cfg::A_BYTES + Cfg::B_BYTES));
          const uint32_t sa = stage0 + s * Cfg::STAGE;
          tma_load_2d_pair(sa, rmap, lead_full, kb * kBK, row0);
          tma_load_2d_pair(sa + Cfg::A_BYTES, &p.tmap_c, lead_full, kb * kBK, tc * Cfg::BN + (int)cta * 128);
          if (++s == Cfg::STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (leader CTA only) =================
    if (leader && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(256, Cfg::BN);
      uint32_t peer_empty[Cfg::STAGES], peer_tfull[2];
      for (int s = 0; s < Cfg::STAGES; ++s) peer_empty[s] = mapa_shared(empty_bar(s), 1);
      for (int a = 0; a < 2; ++a) peer_tfull[a] = mapa_shared(tfull_bar(a), 1);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
        ok = mbar_wait(tempty_bar(acc), acc_ph ^ 1u, p.sync, 45);
        if (!ok) break;
        tc_fence_after();
        trace_put(p, 0, it, 0);
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * Cfg::BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(full_bar(s), ph, p.sync, 46);
          if (!ok) break;
          tc_fence_after();
          if (kb == 0) trace_put(p, 0, it, 1);
          const uint32_t sa = stage0 + s * Cfg::STAGE;
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + Cfg::A_BYTES);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k)
            umma_bf16_pair(d_tmem, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit_pair(empty_bar(s));      // own stage free
          umma_commit_pair(peer_empty[s]);     // peer's stage free
          if (++s == Cfg::STAGES) { s = 0; ph ^= 1u; }
        }
        if (ok) {
          umma_commit_pair(tfull_bar(acc));
          umma_commit_pair(peer_tfull[acc]);
        }
        trace_put(p, 0, it, 2);
      }
    }
  } else if (warp >= 6) {
    hooks.side_role(p, pair_id, num_pairs, (int)cta, (int)threadIdx.x - kGemmThreads);
  } else {
    // ================= epilogue warps (both CTAs, own 128 rows) =================
    const int q = warp & 3;
    unsigned char* stg = epi_ptr + (warp - 2) * kEpiWarpBytes;
    const uint32_t lead_tempty[2] = {mapa_shared(tempty_bar(0), 0), mapa_shared(tempty_bar(1), 0)};
    const bool defer = !p.out_fp32 && !p.transposed && p.use_tma_store != 0;
    int prev_tr = -1, prev_tc = -1;
    int it = 0;
    bool ok = true;
    for (int t = pair_id; t < total_tiles && ok; t += num_pairs, ++it) {
      int tr2, tc;
      tile_coords(p, t, tr2, tc);
      const int tr = 2 * tr2 + (int)cta;
      const int acc = it & 1;
      const uint32_t acc_ph = (uint32_t)(it >> 1) & 1u;
      ok = mbar_wait(tfull_bar(acc), acc_ph, p.sync, 47);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      if (q == 0 && lane == 0) trace_put(p, 1, it, 0);
      if (defer && prev_tr >= 0 && hooks.may_wait(p, tr)) {
        if (lane == 0) {
          bulk_wait_group<0>();
          fence_proxy_async();
        }
        __syncwarp();
        ok = hooks.after_store(p, prev_tr, prev_tc, q, lane);
        prev_tr = -1;
        if (!ok) break;
      }
      ok = gemm_epilogue_tile<Cfg::BN, true>(p, hooks, tr, tc, acc, tmem_base, q, lane, stg, lead_tempty[acc], defer);
      if (!ok) break;
      if (q == 0 && lane == 0) trace_put(p, 1, it, 1);
      if (defer) {
        if (prev_tr >= 0) ok = hooks.after_store(p, prev_tr, prev_tc, q, lane);
        prev_tr = tr;
        prev_tc = tc;
      } else {
        ok = hooks.after_store(p, tr, tc, q, lane);
      }
      if (q == 0 && lane == 0) trace_put(p, 1, it, 2);
    }
    if (defer && prev_tr >= 0) {
      if (lane == 0) {
        bulk_wait_group<0>();
        fence_proxy_async();
      }
      __syncwarp();
      if (ok) hooks.after_store(p, prev_tr, prev_tc, q, lane);
    }
  }

  // The producer and MMA warps ran their roles on one elected lane: wait for it, so that the other
  // lanes do not start polling in the helper role while it still has tiles to feed.
  __syncwarp();
  if (warp < 6) hooks.helper_role(p, pair_id, num_pairs, (int)cta, (int)threadIdx.x);

  // ---- teardown: nobody leaves while the pair may still touch its shared memory or barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace kraken
