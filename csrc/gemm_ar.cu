// Fused GEMM -> all-reduce for decode shapes (reference:
// kraken/fused/gemm_one_shot_all_reduce_fused.py:106-178): the single-CTA tcgen05 main loop with the
// exchange hooks of gemm_hooks.cuh — fp32 partial tile to a staging buffer, per-tile flags to the
// peers, then a one-shot sum (in the NVSwitch with multimem.ld_reduce, or ws peer loads) or a
// two-shot exchange by tile owner. Kernels of their own, so that the exchange code does not share a
// register allocation with the other GEMM modes.
#include "kraken/gemm_host.h"
#include "kraken/gemm_hooks.cuh"

namespace kraken {

template <int BN>
__device__ __forceinline__ void gemm_ar_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  ArHooks h;
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

}  // namespace kraken

using namespace kraken;

// Fused GEMM -> all-reduce (decode). bufs[r] = rank r's staging buffer of staging_bytes, DEDICATED
// to this op (nothing else may write it between calls); needs staging_bytes >= 2*(ws+1)*M*N*4.
// out[M, N] fp32 =
// sum_r a_r[M, K_local] * bt_r[N, K_local]^T. algo: 0 one-shot, 1 two-shot, -1 by size.
// call_parity: 0/1, alternating from call to call on the same staging buffer.
KR_API int kr_gemm_ar_bf16(void* const* bufs, uint32_t* const* pads, void* mc_ptr, int rank, int ws, const void* a,
                           long long lda, const void* bt, long long ldb, void* out, long long ldo, int M, int N, int K,
                           int swap_ab, int algo, int call_parity, uint32_t flag_base, unsigned long long pad_words,
                           unsigned long long staging_bytes, int in_fp32, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const bool swap = swap_ab < 0 ? (M <= 64 && N >= 128) : swap_ab != 0;
  // column tile: as many CTAs as the problem allows (up to one per SM), tiles no wider than needed
  const int rows_c = swap ? M : N;
  const int tiles_r = ((swap ? N : M) + kBM - 1) / kBM;
  int bn_pick = pick_bn(rows_c);
  while (bn_pick > 16 && tiles_r * ((rows_c + bn_pick - 1) / bn_pick) < d->num_sms / 2 &&
         tiles_r * ((rows_c + bn_pick / 2 - 1) / (bn_pick / 2)) <= d->num_sms)
    bn_pick /= 2;
  if (in_fp32) bn_pick = bn_pick <= 16 ? 16 : (bn_pick <= 64 ? 64 : 256);
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
  const unsigned long long mn4 = (unsigned long long)M * N * 4;
  const int tiles = p.tiles_r * p.tiles_c;
  if (algo < 0) algo = ((unsigned long long)(ws - 1) * mn4 > (1ull << 20)) ? 1 : 0;   // > 1 MiB of pull traffic
  p.ar_algo = algo;
  // Fixed layout of the dedicated staging buffer (S bytes) and of the flag words, independent of the
  // problem shape, so that consecutive calls of different shapes or algorithms never share a region
  // a slower rank may still be reading:
  //   [0, S/4) one-shot even calls | [S/4, S/2) one-shot odd calls | [S/2, S) two-shot partial slots + result
  //   flag words: one-shot even | +50000 one-shot odd | +100000 two-shot "partial stored" | +150000 "published"
  const unsigned long long S = staging_bytes;
  KR_REQUIRE(S % 1024 == 0, "staging size must be a multiple of 1024 bytes");
  KR_REQUIRE(tiles <= 50000 && (unsigned long long)flag_base + 200000ull <= pad_words,
             "signal pad too small for the tile flags");
  if (algo == 0) {
    KR_REQUIRE(S / 4 >= mn4, "staging buffer too small for one-shot GEMM all-reduce");
    p.stage_off = (call_parity & 1) ? S / 4 : 0;
    p.flag_base = flag_base + ((call_parity & 1) ? 50000u : 0u);
  } else {
    KR_REQUIRE(S / 2 >= (unsigned long long)(ws + 1) * mn4, "staging buffer too small for two-shot GEMM all-reduce");
    p.part_off = S / 2;
    p.res_off = S / 2 + (unsigned long long)ws * mn4;
    p.flag_base = flag_base + 100000u;
    p.flag2_base = flag_base + 150000u;
  }
  p.sync = sync_ctx(d);
  unsigned nb = (unsigned)tiles;
  unsigned cap = grid_cap(d);
  if (nb > cap) nb = cap;
  p.num_mma_ctas = (int)nb;
  return launch_gemm(bn, p, nb, stream);
}

