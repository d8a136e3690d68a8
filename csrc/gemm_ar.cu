// Fused GEMM -> all-reduce for decode shapes (reference:
// kraken/fused/gemm_one_shot_all_reduce_fused.py:106-178): the single-CTA tcgen05 main loop, with K
// optionally split over several CTAs per tile, and the exchange hooks of gemm_hooks.cuh. Four
// exchanges: fp32 partial tiles behind per-tile flags (one-shot: summed in the NVSwitch with
// multimem.ld_reduce or from ws peer loads; two-shot: by tile owner), or partial elements that carry
// a per-call tag in the same 8-byte store and need no flag at all (pushed to every rank, or to the
// tile owner with tagged results coming back). The launcher picks exchange and split count by a
// cost model. Kernels of their own, so that the exchange code does not share a register allocation
// with the other GEMM modes.
#include "kraken/gemm_host.h"
#include "kraken/gemm_hooks.cuh"

namespace kraken {

template <int BN>
__device__ __forceinline__ void gemm_ar_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  ArHooksT<(BN <= 64)> h;   // the tagged push only exists for decode rows (column tiles up to 64)
  h.bn = BN;
  gemm_mainloop<BN>(p, bid, nb, h, smem_raw);
}

#define KR_DEFINE_GEMM_AR(BN)                                                                                \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm_ar##BN##_kernel(const __grid_constant__ GemmParams p) { \
    gemm_ar_body<BN>(p, blockIdx.x, gridDim.x);                                                              \
  }                                                                                                          \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm_ar##BN##_emu_kernel(const GemmParams* ps) {          \
    gemm_ar_body<BN>(ps[blockIdx.y], blockIdx.x, gridDim.x);                                                 \
  }
KR_DEFINE_GEMM_AR(256)
KR_DEFINE_GEMM_AR(128)
KR_DEFINE_GEMM_AR(64)
KR_DEFINE_GEMM_AR(32)
KR_DEFINE_GEMM_AR(16)

int launch_gemm_ar(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream) {
  switch (bn) {
    case 256: return launch_ranked(gemm_ar256_kernel, gemm_ar256_emu_kernel, p, nb, kGemmThreads, GemmCfg<256>::SMEM, stream);
    case 128: return launch_ranked(gemm_ar128_kernel, gemm_ar128_emu_kernel, p, nb, kGemmThreads, GemmCfg<128>::SMEM, stream);
    case 64: return launch_ranked(gemm_ar64_kernel, gemm_ar64_emu_kernel, p, nb, kGemmThreads, GemmCfg<64>::SMEM, stream);
    case 32: return launch_ranked(gemm_ar32_kernel, gemm_ar32_emu_kernel, p, nb, kGemmThreads, GemmCfg<32>::SMEM, stream);
    default: return launch_ranked(gemm_ar16_kernel, gemm_ar16_emu_kernel, p, nb, kGemmThreads, GemmCfg<16>::SMEM, stream);
  }
}

// What one call does: which operand sits on the 128-row side, the column tile, the exchange
// algorithm (0 one-shot pull, 1 two-shot, 2 tagged push, 3 tagged two-shot) and the number of K splits, picked by a
// small cost model (seconds). Splitting K puts more CTAs on the weight stream but multiplies the
// partial sums that cross NVLink. algo / k_splits: -1 / 0 = choose; a given value is kept if valid.
struct ArPlan {
  bool swap;
  int bn, tiles, algo, ks;
};
static bool ar_plan(const DeviceState* d, int M, int N, int K, int ws, int swap_ab, int in_fp32, int algo, int k_splits,
                    unsigned long long S, bool host_ptrs, ArPlan& pl) {
  pl.swap = swap_ab < 0 ? (M <= 64 && N >= 128) : swap_ab != 0;
  // column tile: as many CTAs as the problem allows (up to one per SM), tiles no wider than needed
  const int rows_c = pl.swap ? M : N;
  const int tiles_r = ((pl.swap ? N : M) + kBM - 1) / kBM;
  int bn = pick_bn(rows_c);
  while (bn > 16 && tiles_r * ((rows_c + bn - 1) / bn) < d->num_sms / 2 && tiles_r * ((rows_c + bn / 2 - 1) / (bn / 2)) <= d->num_sms)
    bn /= 2;
  if (in_fp32) bn = bn <= 16 ? 16 : (bn <= 64 ? 64 : 256);
  pl.bn = bn;
  pl.tiles = tiles_r * ((rows_c + bn - 1) / bn);
  const unsigned cap = grid_cap(d);
  const unsigned long long mn = (unsigned long long)M * N, mn4 = mn * 4;
  const int elt = in_fp32 ? 4 : 2;
  const int num_kb = (K + 128 / elt - 1) / (128 / elt);
  const double cta_bytes = (double)(kBM + bn) * K * elt, all_bytes = cta_bytes * pl.tiles;
  auto ks_ok = [&](int ks) { return ks == 1 || ((unsigned)(pl.tiles * ks) <= cap && 2 * ks <= num_kb); };
  auto ll_ok = [&](int ks) { return pl.swap && host_ptrs && ws <= 8 && (unsigned long long)ws * ks * mn * 8 <= S / 8; };
  auto two_ok = [&](int ks) { return (unsigned long long)(ws * ks + 1) * mn4 <= S / 2; };
  // tagged two-shot: per slot the packed tiles of one owner, then the [M][N] tagged results
  const unsigned long long slot_pairs = (unsigned long long)((pl.tiles + ws - 1) / ws) * bn * kBM;
  auto tag2_ok = [&](int ks) {
    return pl.swap && host_ptrs && ws <= 8 && N % 4 == 0 && ((unsigned long long)ws * ks * slot_pairs + mn) * 8 <= S / 8;
  };
  auto t_main = [&](int ks) { const double a1 = cta_bytes / ks / 80e9, a2 = all_bytes / 6.5e12; return a1 > a2 ? a1 : a2; };
  auto t_xfer = [&](int al, int ks) {
    // Fixed costs as measured on top of the plain GEMM of the same shape at 2 and 8 ranks (they grow
    // with the number of peers: flag round trips for the one- and two-shot forms, polling for the
    // tagged ones), plus the bytes a rank receives at the rate each form was seen to reach.
    const double peers = (double)(ws - 1);
    if (al == 3) return (3.0 + 1.3 * peers) * 1e-6 + (double)(ks + 1) * peers / ws * mn * 8 / 400e9;
    if (al == 2) return (1.0 + 1.1 * peers) * 1e-6 + (double)ks * peers * mn * 8 / 400e9;
    if (al == 1) return (11.0 + 1.2 * peers) * 1e-6 + (double)(ks + 1) * peers / ws * mn4 / 600e9;
    return (9.0 + 0.15 * peers) * 1e-6 + peers * mn4 / 400e9;
  };
  pl.algo = -1;
  pl.ks = 1;
  while (k_splits > 1 && !ks_ok(k_splits)) --k_splits;   // a requested split count is an upper bound
  double best = 1e30;
  for (int al = 0; al <= 3; ++al) {
    if (algo >= 0 && al != algo) continue;
    // flag forms: above 2 ranks one-shot pull traffic grows with ws - 1, so large outputs go two-shot;
    // at 2 ranks both move the same bytes and one-shot has one flag hop less (measured faster at every M)
    if (algo < 0 && al == 0 && ws > 2 && (unsigned long long)(ws - 1) * mn4 > (1ull << 20)) continue;
    if (algo < 0 && al == 1 && ws == 2 && mn4 <= S / 8) continue;
    for (int ks = 1; ks <= 4; ++ks) {
      if (k_splits > 0 && ks != k_splits) continue;
      if (!ks_ok(ks)) continue;
      if (al == 0 && (ks != 1 || mn4 > S / 8)) continue;
      if (al == 1 && !two_ok(ks)) continue;
      if (al == 2 && !ll_ok(ks)) continue;
      if (al == 3 && !tag2_ok(ks)) continue;
      const double t = t_main(ks) + t_xfer(al, ks);
      if (t < best) { best = t; pl.algo = al; pl.ks = ks; }
    }
  }
  return pl.algo >= 0;
}

}  // namespace kraken

using namespace kraken;

// Fused GEMM -> all-reduce (decode). bufs[r] = rank r's staging buffer of staging_bytes (bufs: device
// table; bufs_host: the same addresses in host memory, or nullptr), DEDICATED to this op (nothing
// else may write it between calls, and it must have been all zero before its first use).
// out[M, N] fp32 = sum_r a_r[M, K_local] * bt_r[N, K_local]^T.
// algo: 0 one-shot pull, 1 two-shot, 2 tagged push, 3 tagged two-shot, -1 by size. k_splits: parts the K range is cut
// into (more CTAs streaming the weights), 0 = chosen here. call_seq: the number of calls made on
// this staging buffer so far; every rank passes the same value.
// Needs staging_bytes >= 8*M*N*4 (one-shot), >= 2*(ws*k_splits+1)*M*N*4 (two-shot); the tagged push
// is used only where its ws*k_splits*M*N*8 bytes fit into an eighth of the buffer.
KR_API int kr_gemm_ar_bf16(void* const* bufs, void* const* bufs_host, uint32_t* const* pads, void* mc_ptr, int rank,
                           int ws, const void* a, long long lda, const void* bt, long long ldb, void* out,
                           long long ldo, int M, int N, int K, int swap_ab, int algo, int k_splits,
                           unsigned call_seq, uint32_t flag_base, unsigned long long pad_words,
                           unsigned long long staging_bytes, int in_fp32, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(algo >= -1 && algo <= 3 && k_splits >= 0 && k_splits <= 8, "bad algorithm or split count");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  ArPlan pl;
  KR_REQUIRE(staging_bytes % 1024 == 0, "staging size must be a multiple of 1024 bytes");
  KR_REQUIRE(ar_plan(d, M, N, K, ws, swap_ab, in_fp32, algo, k_splits, staging_bytes, bufs_host != nullptr, pl),
             "staging buffer too small (or shape not eligible) for the requested GEMM all-reduce exchange");
  const bool swap = pl.swap;
  const int bn_pick = pl.bn;
  int bn = 0;
  int rc = setup_problem(p, a, lda, bt, ldb, M, N, K, swap, bn_pick, &bn, in_fp32 ? 4 : 2);
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
  p.mc_ptr = mc_ptr;
  if (bufs_host != nullptr && ws <= 8)
    for (int r = 0; r < ws; ++r) p.peer_buf[r] = bufs_host[r];
  const unsigned long long mn = (unsigned long long)M * N, mn4 = mn * 4;
  const int tiles = p.tiles_r * p.tiles_c;
  const unsigned cap = grid_cap(d);
  const unsigned long long S = staging_bytes;
  KR_REQUIRE(tiles <= 50000 && (unsigned long long)flag_base + 200000ull <= pad_words,
             "signal pad too small for the tile flags");
  KR_REQUIRE(bn == pl.bn && tiles == pl.tiles, "tile plan mismatch");
  algo = pl.algo;
  const int best_ks = pl.ks;
  p.ar_algo = algo;
  p.k_splits = best_ks;
  // Fixed layout of the dedicated staging buffer (S bytes) and of the flag words, independent of the
  // problem shape, so that consecutive calls of different shapes or algorithms never share a region
  // a slower rank may still be reading:
  //   [0, S/8) one-shot, even calls | [S/8, S/4) one-shot, odd | [S/4, 3S/8) tagged push, even |
  //   [3S/8, S/2) tagged push, odd | [S/2, S) two-shot partial slots + result
  //   flag words: one-shot even | +50000 one-shot odd | +100000 two-shot "partial stored" | +150000 "published"
  const unsigned odd = call_seq & 1u;
  if (algo == 0) {
    p.stage_off = odd ? S / 8 : 0;
    p.flag_base = flag_base + (odd ? 50000u : 0u);
  } else if (algo == 2 || algo == 3) {
    p.ll_off = S / 4 + (odd ? S / 8 : 0);
    p.ll_end = p.ll_off + S / 8;
    p.ll_tag = call_seq % 0x7fffffffu + 1u;      // never 0, and never the tag this region saw two calls ago
    if (algo == 3) {
      p.ll_slot_pairs = (unsigned long long)((tiles + ws - 1) / ws) * bn * kBM;
      p.ll_res_off = p.ll_off + (unsigned long long)ws * best_ks * p.ll_slot_pairs * 8;
    }
  } else {
    p.part_off = S / 2;
    p.res_off = S / 2 + (unsigned long long)ws * best_ks * mn4;
    p.flag_base = flag_base + 100000u;
    p.flag2_base = flag_base + 150000u;
  }
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)(tiles * best_ks);
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

// What kr_gemm_ar_bf16 picks for a shape: out[0] = algorithm (0 one-shot, 1 two-shot, 2 tagged push, 3 tagged two-shot),
// out[1] = K splits, out[2] = column tile, out[3] = CTAs, out[4] = 1 when the weights sit on the
// 128-row side. For logs and tests; no launch.
KR_API int kr_gemm_ar_plan(int M, int N, int K, int ws, int in_fp32, int algo, int k_splits,
                           unsigned long long staging_bytes, int host_ptrs, int* out) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  ArPlan pl;
  KR_REQUIRE(ar_plan(d, M, N, K, ws, -1, in_fp32, algo, k_splits, staging_bytes, host_ptrs != 0, pl),
             "no GEMM all-reduce plan for this shape and staging size");
  unsigned nb = (unsigned)(pl.tiles * pl.ks), cap = grid_cap(d);
  out[0] = pl.algo;
  out[1] = pl.ks;
  out[2] = pl.bn;
  out[3] = (int)(nb > cap ? cap : nb);
  out[4] = pl.swap ? 1 : 0;
  return KR_SUCCESS;
}
