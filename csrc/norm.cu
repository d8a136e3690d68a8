// RMSNorm and the tensor-parallel decode epilogue: all-reduce + bias + RMSNorm in one kernel.
// A block owns whole rows (row r belongs to block r % gridDim.x on every rank), keeps the summed
// row in registers between the reduction and the normalisation, and loops over its rows, so the
// grid never exceeds the SM count whatever the batch size.
//
// Reference counterparts: kraken/fused/rms_norm.py:9-72,
// kraken/fused/one_shot_all_reduce_bias_rms_norm.py:23-169,
// kraken/fused/two_shot_all_reduce_bias_rms_norm.py:27-223.
// y = x * rsqrt(mean(x^2) + eps) * w, fp32 math, bf16 in/out.
#include "kraken/host.h"
#include "kraken/norm_core.cuh"

namespace kraken {

struct NormParams {
  void* const* bufs;       // [ws] symmetric buffers (AR variants)
  uint32_t* const* pads;   // [ws]
  const void* x;           // input rows [rows, D]
  void* y;                 // output rows [rows, D]
  const void* bias;        // optional
  const void* w;           // [D]
  void* mc_ptr;            // multicast address of the symmetric buffer (two-shot NVLS) or nullptr
  unsigned long long bias_period;
  int rows, D;
  int rank, ws;
  float eps;
  uint32_t pad_base;
  unsigned long long buf_off;   // byte offset of the tensor inside every rank's symmetric buffer
  SyncCtx sync;
};

__device__ __forceinline__ char* symm_buf(const NormParams& p, int r) { return (char*)p.bufs[r] + p.buf_off; }

// ---- standalone RMSNorm ----------------------------------------------------------------------
// A block walks rows r, r + gridDim.x, ...; the NEXT row's vectors are requested before the current
// row is reduced and stored, so every block always has a row of loads in flight (the reduction's
// two block barriers would otherwise leave the memory pipe idle once per row).
__global__ void __launch_bounds__(kNormMaxThreads) rms_norm_kernel(const __grid_constant__ NormParams p) {
  __shared__ float smem[32];
  const int nvec = p.D / 8;
  U4 nx[kNormVpt];
  int r = blockIdx.x;
  if (r < p.rows) {
    const char* xrow = (const char*)p.x + (size_t)r * p.D * 2;
#pragma unroll
    for (int i = 0; i < kNormVpt; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) nx[i] = ld16(xrow + (size_t)v * 16);
    }
  }
  for (; r < p.rows; r += gridDim.x) {
    float f[kNormVpt][8];
#pragma unroll
    for (int i = 0; i < kNormVpt; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) unpack8(nx[i], f[i]);
    }
    const int rn = r + gridDim.x;
    if (rn < p.rows) {
      const char* xrow = (const char*)p.x + (size_t)rn * p.D * 2;
#pragma unroll
      for (int i = 0; i < kNormVpt; ++i) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) nx[i] = ld16(xrow + (size_t)v * 16);
      }
    }
    rms_finish<kNormVpt>(f, nvec, p.D, p.eps, (const char*)p.w, (char*)p.y + (size_t)r * p.D * 2, smem);
  }
}

// Rows longer than the register budget: two passes over global memory.
__global__ void __launch_bounds__(kNormMaxThreads) rms_norm_long_kernel(const __grid_constant__ NormParams p) {
  __shared__ float smem[32];
  const int nvec = p.D / 8;
  for (int r = blockIdx.x; r < p.rows; r += gridDim.x) {
    const char* xrow = (const char*)p.x + (size_t)r * p.D * 2;
    char* yrow = (char*)p.y + (size_t)r * p.D * 2;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      unpack8(ld16(xrow + (size_t)v * 16), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
    ss = block_sum(ss, smem);
    const float inv = rsqrtf(ss / (float)p.D + p.eps);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8], g[8];
      unpack8(ld16(xrow + (size_t)v * 16), f);
      unpack8(ld16_nc((const char*)p.w + (size_t)v * 16), g);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = f[j] * inv * g[j];
      st16(yrow + (size_t)v * 16, pack8(g));
    }
  }
}

__device__ __forceinline__ void norm_add_bias8(const NormParams& p, size_t elem, float (&f)[8]) {
  acc8(ld16_nc((const char*)p.bias + (elem % p.bias_period) * 2), f);
}

// ---- one-shot all-reduce + bias + RMSNorm ------------------------------------------------------
// VPT: vectors a thread keeps per row. 1 covers rows of up to 8192 elements with every peer's load
// of the thread's vector in flight at once and no register spills (a spilled load becomes a
// synchronous one: ws NVLink round trips instead of one).
template <int VPT>
__device__ __forceinline__ void ar_norm_one_shot_impl(const NormParams& p, unsigned bid, unsigned nb) {
  __shared__ float smem[32];
  const int nvec = p.D / 8;
  const uint32_t sync_id = p.pad_base / p.ws + bid;
  char* own = symm_buf(p, p.rank);
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
      st16(own + off + (size_t)v * 16, ld16((const char*)p.x + off + (size_t)v * 16));
  }
  if (!symm_mem_sync<true, true>(p.pads, sync_id, p.rank, p.ws, p.sync, 30)) return;
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    float f[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[i][j] = 0.f;
        if (p.bias) norm_add_bias8(p, (size_t)r * p.D + (size_t)v * 8, f[i]);
        // all peers' loads are issued before any is consumed: one NVLink latency, not ws of them
        U4 x[8];
        for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) {
              int peer = p.rank + s0 + s;
              if (peer >= p.ws) peer -= p.ws;
              x[s] = ld16(symm_buf(p, peer) + off + (size_t)v * 16);
            }
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) acc8(x[s], f[i]);
        }
      }
    }
    rms_finish<VPT>(f, nvec, p.D, p.eps, (const char*)p.w, (char*)p.y + off, smem);
  }
  symm_mem_sync<true, false>(p.pads, sync_id, p.rank, p.ws, p.sync, 31);
}
__device__ void ar_norm_one_shot_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_one_shot_impl<1>(p, bid, nb); }
__device__ void ar_norm_one_shot_long_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_one_shot_impl<kNormVpt>(p, bid, nb); }
KR_DEFINE_RANKED_KERNEL(ar_norm_one_shot_long, NormParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(ar_norm_one_shot, NormParams, kNormMaxThreads)

// ---- two-shot all-reduce + bias + RMSNorm ------------------------------------------------------
// Rank k reduces columns [k*D/ws, (k+1)*D/ws) of every row the block owns (+bias), publishes the
// bf16 sums to all ranks (P2P stores, or one multimem.st), then each rank normalises its rows.
template <bool USE_MC, int VPT>
__device__ __forceinline__ void ar_norm_two_shot_impl(const NormParams& p, unsigned bid, unsigned nb) {
  __shared__ float smem[32];
  const int nvec = p.D / 8;
  const int svec = nvec / p.ws;   // host: D % (8*ws) == 0
  const uint32_t sync_id = p.pad_base / p.ws + bid;
  char* own = symm_buf(p, p.rank);
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
      st16(own + off + (size_t)v * 16, ld16((const char*)p.x + off + (size_t)v * 16));
  }
  if (!symm_mem_sync<true, true>(p.pads, sync_id, p.rank, p.ws, p.sync, 32)) return;
  for (int r = bid; r < p.rows; r += nb) {
    for (int sv = threadIdx.x; sv < svec; sv += blockDim.x) {
      const int v = p.rank * svec + sv;
      const size_t off = (size_t)r * p.D * 2 + (size_t)v * 16;
      U4 out;
      if (USE_MC) {
        out = multimem_ld_reduce_bf16x8((const char*)p.mc_ptr + p.buf_off + off);
        if (p.bias) {
          float f[8];
          unpack8(out, f);
          norm_add_bias8(p, (size_t)r * p.D + (size_t)v * 8, f);
          out = pack8(f);
        }
        multimem_st16((char*)p.mc_ptr + p.buf_off + off, out);
      } else {
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (p.bias) norm_add_bias8(p, (size_t)r * p.D + (size_t)v * 8, f);
        U4 x[8];
        for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) {
              int peer = p.rank + s0 + s;
              if (peer >= p.ws) peer -= p.ws;
              x[s] = ld16(symm_buf(p, peer) + off);
            }
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) acc8(x[s], f);
        }
        out = pack8(f);
        for (int s = 0; s < p.ws; ++s) {
          int peer = p.rank + s;
          if (peer >= p.ws) peer -= p.ws;
          st16(symm_buf(p, peer) + off, out);
        }
      }
    }
  }
  if (!symm_mem_sync<true, true>(p.pads, sync_id, p.rank, p.ws, p.sync, 33)) return;
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    float f[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) unpack8(ld16(own + off + (size_t)v * 16), f[i]);
    }
    rms_finish<VPT>(f, nvec, p.D, p.eps, (const char*)p.w, (char*)p.y + off, smem);
  }
  symm_mem_sync<true, false>(p.pads, sync_id, p.rank, p.ws, p.sync, 34);
}
__device__ void ar_norm_two_shot_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_two_shot_impl<false, 1>(p, bid, nb); }
__device__ void ar_norm_two_shot_mc_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_two_shot_impl<true, 1>(p, bid, nb); }
__device__ void ar_norm_two_shot_long_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_two_shot_impl<false, kNormVpt>(p, bid, nb); }
__device__ void ar_norm_two_shot_mc_long_body(const NormParams& p, unsigned bid, unsigned nb) { ar_norm_two_shot_impl<true, kNormVpt>(p, bid, nb); }
KR_DEFINE_RANKED_KERNEL(ar_norm_two_shot, NormParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(ar_norm_two_shot_mc, NormParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(ar_norm_two_shot_long, NormParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(ar_norm_two_shot_mc_long, NormParams, kNormMaxThreads)

}  // namespace kraken

using namespace kraken;

// Threads per row. vpt = 16-byte vectors each thread keeps: 1 when the loads cross NVLink (every
// load of a row in flight at once matters more than occupancy), up to kNormVpt for the local
// kernel (smaller blocks, several rows resident per SM, four independent loads per thread).
static unsigned norm_threads(int D, int vpt) {
  unsigned nvec = (unsigned)D / 8;
  unsigned t = (nvec + vpt - 1) / vpt;
  t = (t + 31) / 32 * 32;
  if (t < 64) t = 64;
  if (t > kNormMaxThreads) t = kNormMaxThreads;
  return t;
}

KR_API int kr_rms_norm(const void* x, const void* w, void* y, int rows, int D, float eps, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(rows >= 0 && D > 0 && D % 8 == 0, "rms_norm needs D % 8 == 0");
  KR_REQUIRE((((uintptr_t)x | (uintptr_t)y | (uintptr_t)w) & 15) == 0, "tensors must be 16-byte aligned");
  if (rows == 0) return KR_SUCCESS;
  NormParams p;
  memset(&p, 0, sizeof(p));
  p.x = x; p.y = y; p.w = w; p.rows = rows; p.D = D; p.eps = eps;
  const unsigned nt = norm_threads(D, rows >= 2 * d->num_sms ? kNormVpt : 1);
  // one wave of co-resident blocks (the register file, not the thread count, is what limits it)
  int per_sm = 0;
  KR_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rms_norm_kernel, (int)nt, 0));
  const unsigned resident = per_sm > 0 ? (unsigned)per_sm : 1u;
  const unsigned cap = (unsigned)d->num_sms * resident;
  unsigned nb = (unsigned)rows < cap ? (unsigned)rows : cap;
  if (D / 8 <= kNormVpt * kNormMaxThreads)
    rms_norm_kernel<<<nb, nt, 0, stream>>>(p);
  else
    rms_norm_long_kernel<<<nb, kNormMaxThreads, 0, stream>>>(p);
  KR_CUDA(cudaGetLastError());
  return KR_SUCCESS;
}

// y = rms_norm(bias + sum_r x_r) ; algo 0: one-shot pull, 1: two-shot, 2: two-shot NVLS (mc_ptr)
KR_API int kr_all_reduce_bias_rms_norm(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank, int ws, const void* x,
                                       const void* bias, unsigned long long bias_numel, const void* w, void* y,
                                       int rows, int D, float eps, int algo, void* mc_ptr, uint32_t pad_base,
                                       cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(rows >= 1 && D > 0 && D % 8 == 0, "needs D % 8 == 0");
  KR_REQUIRE(D / 8 <= kNormVpt * kNormMaxThreads, "row too long for the fused all-reduce + RMSNorm kernel");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  KR_REQUIRE(buf_off % 16 == 0, "symmetric tensor must start 16-byte aligned inside its buffer");
  KR_REQUIRE((((uintptr_t)x | (uintptr_t)y | (uintptr_t)w | (uintptr_t)bias) & 15) == 0,
             "tensors must be 16-byte aligned");
  if (bias) KR_REQUIRE(bias_numel > 0 && bias_numel % 8 == 0, "bias length must be a positive multiple of 8");
  if (algo != 0) KR_REQUIRE(D % (8 * ws) == 0, "two-shot needs D % (8 * world_size) == 0");
  if (algo == 2) KR_REQUIRE(mc_ptr != nullptr, "NVLS variant needs a multicast address");
  NormParams p;
  memset(&p, 0, sizeof(p));
  p.bufs = bufs; p.buf_off = buf_off; p.pads = pads; p.x = x; p.y = y; p.bias = bias; p.w = w; p.mc_ptr = mc_ptr;
  p.bias_period = bias ? bias_numel : 8;
  p.rows = rows; p.D = D; p.rank = rank; p.ws = ws; p.eps = eps; p.pad_base = pad_base;
  p.sync = sync_ctx(d);
  unsigned cap = (unsigned)d->num_sms;
  if (emu_recorder().active) cap = cap / (unsigned)emu_recorder().ws ? cap / (unsigned)emu_recorder().ws : 1;
  unsigned nb = (unsigned)rows < cap ? (unsigned)rows : cap;
  unsigned nt = norm_threads(D, 1);
  const bool longrow = (unsigned)D / 8 > nt;       // more than one vector per thread
  if (algo == 0)
    return longrow ? launch_ranked(ar_norm_one_shot_long_kernel, ar_norm_one_shot_long_emu_kernel, p, nb, nt, 0, stream)
                   : launch_ranked(ar_norm_one_shot_kernel, ar_norm_one_shot_emu_kernel, p, nb, nt, 0, stream);
  if (algo == 1)
    return longrow ? launch_ranked(ar_norm_two_shot_long_kernel, ar_norm_two_shot_long_emu_kernel, p, nb, nt, 0, stream)
                   : launch_ranked(ar_norm_two_shot_kernel, ar_norm_two_shot_emu_kernel, p, nb, nt, 0, stream);
  return longrow ? launch_ranked(ar_norm_two_shot_mc_long_kernel, ar_norm_two_shot_mc_long_emu_kernel, p, nb, nt, 0, stream)
                 : launch_ranked(ar_norm_two_shot_mc_kernel, ar_norm_two_shot_mc_emu_kernel, p, nb, nt, 0, stream);
}
