// Row-normalisation building blocks shared by the RMSNorm kernels: a block-wide sum and the
// normalise-and-store step of a row held in registers (y = x * rsqrt(mean(x^2) + eps) * w, fp32
// math, reference: kraken/fused/rms_norm.py:34-43).
#pragma once
#include "kraken/vec.cuh"

namespace kraken {

constexpr int kNormMaxThreads = 1024;
constexpr int kNormVpt = 4;   // most 16-byte vectors a thread keeps in registers per row

__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();   // smem reuse across rows
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? smem[lane] : 0.f;
  return warp_sum(t);
}

// Normalises the row held in f[][] (vectors threadIdx.x + i*blockDim.x) and writes it to yrow.
template <int VPT>
__device__ __forceinline__ void rms_finish(float (&f)[VPT][8], int nvec, int D, float eps, const char* w,
                                           char* yrow, float* smem) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[i][j] * f[i][j];
    }
  }
  ss = block_sum(ss, smem);
  const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float g[8];
      unpack8(ld16_nc(w + (size_t)v * 16), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = f[i][j] * inv * g[j];
      st16(yrow + (size_t)v * 16, pack8(g));
    }
  }
}

}  // namespace kraken
