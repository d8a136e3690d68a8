// Single-CTA tcgen05 GEMM kernels for fp32 operands, multiplied as tf32 (kind::tf32, K = 8 per
// instruction, fp32 accumulation in TMEM): the plain GEMM and the decode GEMM -> all-reduce. The
// reference's GEMM + all-reduce and GEMM + reduce-scatter tests feed fp32 operands to tl.dot, which
// multiplies them as tf32 as well (test/test_gemm_allreduce.py:57-58).
#include "kraken/gemm_host.h"
#include "kraken/gemm_hooks.cuh"

namespace kraken {

template <int BN>
__device__ __forceinline__ void gemm_tf32_body(const GemmParams& p, unsigned bid, unsigned nb) {
  extern __shared__ unsigned char smem_raw[];
  if (p.mode == GEMM_AR) {
    ArHooksT<(BN <= 64)> h;   // the tagged push only exists for decode rows (column tiles up to 64)
    h.bn = BN;
    gemm_mainloop<BN, ArHooksT<(BN <= 64)>, 4>(p, bid, nb, h, smem_raw);
  } else {
    PlainHooks h;
    h.bn = BN;
    gemm_mainloop<BN, PlainHooks, 4>(p, bid, nb, h, smem_raw);
  }
}

#define KR_DEFINE_GEMM_TF32(BN)                                                                                \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm_tf32_##BN##_kernel(const __grid_constant__ GemmParams p) { \
    gemm_tf32_body<BN>(p, blockIdx.x, gridDim.x);                                                              \
  }                                                                                                            \
  __global__ void __launch_bounds__(kGemmThreads, 1) gemm_tf32_##BN##_emu_kernel(const GemmParams* ps) {         \
    gemm_tf32_body<BN>(ps[blockIdx.y], blockIdx.x, gridDim.x);                                                 \
  }
KR_DEFINE_GEMM_TF32(256)
KR_DEFINE_GEMM_TF32(64)
KR_DEFINE_GEMM_TF32(16)

int launch_gemm_tf32(int bn, const GemmParams& p, unsigned nb, cudaStream_t stream) {
  if (p.mode != GEMM_PLAIN && p.mode != GEMM_AR)
    return fail(KR_FAIL_UNSUPPORTED, "fp32 operands are supported by the plain GEMM and the GEMM all-reduce");
  switch (bn) {
    case 256: return launch_ranked(gemm_tf32_256_kernel, gemm_tf32_256_emu_kernel, p, nb, kGemmThreads, GemmCfg<256>::SMEM, stream);
    case 64: return launch_ranked(gemm_tf32_64_kernel, gemm_tf32_64_emu_kernel, p, nb, kGemmThreads, GemmCfg<64>::SMEM, stream);
    case 16: return launch_ranked(gemm_tf32_16_kernel, gemm_tf32_16_emu_kernel, p, nb, kGemmThreads, GemmCfg<16>::SMEM, stream);
    default: return fail(KR_FAIL_ARG, "tf32 GEMM supports column tiles of 16, 64 and 256");
  }
}

}  // namespace kraken
