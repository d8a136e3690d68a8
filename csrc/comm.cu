// Memory-bound collectives over symmetric memory: all-reduce (one-shot pull, two-shot, NVLS
// multimem), reduce-scatter, SM-pull all-gather with progress flags — each optionally fused
// with a bias add. All kernels: bf16 data, fp32 accumulation, 16-byte vectors, peer order
// rotated by rank, bounded waits, persistent grid no larger than the SM count (so a
// 9216-byte signal pad suffices at 8 ranks), and identical grids on every rank because the
// cross-device barrier is keyed by block id.
//
// Reference counterparts: kraken/comm/one_shot_all_reduce.py:17-113,
// kraken/comm/two_shot_all_reduce.py:13-157, kraken/fused/one_shot_all_reduce_bias.py:20-173,
// kraken/fused/two_shot_all_reduce_bias.py:24-193, kraken/comm/copy_engine_all_gather.py:6-126.
// multimem_all_reduce and reduce_scatter have no reference kernel (the reference only names them).
#include <map>
#include <mutex>
#include <string>
#include "kraken/host.h"
#include "kraken/vec.cuh"

namespace kraken {

constexpr int kCommThreads = 512;

struct CommParams {
  void* const* bufs;        // device array [ws]: every rank's symmetric buffer
  uint32_t* const* pads;    // device array [ws]: every rank's signal pad
  const void* input;        // optional: copied into the own buffer first (nullptr: already there)
  void* output;             // local result
  const void* bias;         // optional bf16 bias
  void* mc_ptr;             // multicast (NVLS) address of the symmetric buffer, or nullptr
  uint32_t* progress;       // all-gather: flags [ws * splits]
  uint32_t* counters;       // all-gather: zeroed scratch [ws * splits], self-resetting
  unsigned long long numel; // elements of the (per-rank) tensor
  unsigned long long bias_period;  // bias index = element index % bias_period
  int rank, ws;
  int splits;               // all-gather: chunks per rank
  uint32_t pad_base;        // first slot of the signal pad this launch may use
  unsigned long long buf_off;  // byte offset of the tensor inside every rank's symmetric buffer
  SyncCtx sync;
};

__device__ __forceinline__ char* symm_buf(const CommParams& p, int r) { return (char*)p.bufs[r] + p.buf_off; }

__device__ __forceinline__ void add_bias8(const CommParams& p, size_t elem, float (&f)[8]) {
  // bias_period is a multiple of 8 (checked on the host), so a vector never straddles a period.
  const char* b = (const char*)p.bias + (elem % p.bias_period) * 2;
  acc8(ld16_nc(b), f);
}

__device__ __forceinline__ bool block_sync_T_T(const CommParams& p, unsigned bid, uint32_t site) {
  return symm_mem_sync<true, true>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, site);
}
__device__ __forceinline__ bool block_sync_F_T(const CommParams& p, unsigned bid, uint32_t site) {
  return symm_mem_sync<false, true>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, site);
}
__device__ __forceinline__ bool block_sync_T_F(const CommParams& p, unsigned bid, uint32_t site) {
  return symm_mem_sync<true, false>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, site);
}

// ---------------------------------------------------------------------------------------------
// One-shot all-reduce (+bias): every rank pulls the whole tensor from every peer and sums.
// ---------------------------------------------------------------------------------------------
__device__ void one_shot_ar_body(const CommParams& p, unsigned bid, unsigned nb) {
  const size_t nvec = p.numel / 8;
  const size_t tail0 = nvec * 8;
  const size_t stride = (size_t)nb * blockDim.x;
  const size_t first = (size_t)bid * blockDim.x + threadIdx.x;
  char* own = symm_buf(p, p.rank);
  if (p.input != nullptr) {
    for (size_t v = first; v < nvec; v += stride) st16(own + v * 16, ld16((const char*)p.input + v * 16));
    if (bid == 0)
      for (size_t e = tail0 + threadIdx.x; e < p.numel; e += blockDim.x)
        ((uint16_t*)own)[e] = ((const uint16_t*)p.input)[e];
    if (!block_sync_T_T(p, bid, 1)) return;
  } else {
    if (!block_sync_F_T(p, bid, 1)) return;
  }
  for (size_t v = first; v < nvec; v += stride) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (p.bias) add_bias8(p, v * 8, f);
    U4 x[8];
    for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s0 + s < p.ws) {
          int peer = p.rank + s0 + s;
          if (peer >= p.ws) peer -= p.ws;
          x[s] = ld16(symm_buf(p, peer) + v * 16);
        }
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s0 + s < p.ws) acc8(x[s], f);
    }
    st16((char*)p.output + v * 16, pack8(f));
  }
  if (bid == 0) {
    for (size_t e = tail0 + threadIdx.x; e < p.numel; e += blockDim.x) {
      float a = p.bias ? __bfloat162float(((const __nv_bfloat16*)p.bias)[e % p.bias_period]) : 0.f;
      for (int s = 0; s < p.ws; ++s) a += __bfloat162float(((const __nv_bfloat16*)symm_buf(p, (p.rank + s) % p.ws))[e]);
      ((__nv_bfloat16*)p.output)[e] = __float2bfloat16(a);
    }
  }
  block_sync_T_F(p, bid, 2);
}
KR_DEFINE_RANKED_KERNEL(one_shot_ar, CommParams, kCommThreads)

// ---------------------------------------------------------------------------------------------
// Two-shot all-reduce (+bias): the tensor is cut into chunks of blockDim.x vectors; chunk c is
// reduced by rank c % ws, which then writes the sum into every rank's buffer (or once to the
// multicast address). Block b owns the groups of ws consecutive chunks g with g % nb == b in
// all three phases, so the per-block barrier orders everything it needs.
// USE_MC: reduce with multimem.ld_reduce and publish with multimem.st (NVLS).
// ---------------------------------------------------------------------------------------------
template <bool USE_MC>
__device__ __forceinline__ void two_shot_ar_impl(const CommParams& p, unsigned bid, unsigned nb) {
  const size_t nvec = p.numel / 8;   // host guarantees numel % 8 == 0
  const size_t group = (size_t)blockDim.x * p.ws;   // vectors per chunk group
  const size_t ngroups = (nvec + group - 1) / group;
  char* own = symm_buf(p, p.rank);
  if (p.input != nullptr) {
    for (size_t g = bid; g < ngroups; g += nb)
      for (int c = 0; c < p.ws; ++c) {
        size_t v = g * group + (size_t)c * blockDim.x + threadIdx.x;
        if (v < nvec) st16(own + v * 16, ld16((const char*)p.input + v * 16));
      }
    if (!block_sync_T_T(p, bid, 3)) return;
  } else {
    if (!block_sync_F_T(p, bid, 3)) return;
  }
  // Four chunk groups per iteration: all their loads (4 x ws, or 4 multimem.ld_reduce) are in
  // flight before the first sum, which is what fills the NVLink pipe.
  constexpr int UNR = 4;
  for (size_t g0 = bid; g0 < ngroups; g0 += (size_t)nb * UNR) {
    size_t vs[UNR];
    bool act[UNR];
#pragma unroll
    for (int k = 0; k < UNR; ++k) {
      const size_t g = g0 + (size_t)k * nb;
      vs[k] = g * group + (size_t)p.rank * blockDim.x + threadIdx.x;
      act[k] = g < ngroups && vs[k] < nvec;
    }
    if (USE_MC) {
      U4 r[UNR];
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (act[k]) r[k] = multimem_ld_reduce_bf16x8((const char*)p.mc_ptr + p.buf_off + vs[k] * 16);
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (act[k]) {
          if (p.bias) {
            float f[8];
            unpack8(r[k], f);
            add_bias8(p, vs[k] * 8, f);
            r[k] = pack8(f);
          }
          multimem_st16((char*)p.mc_ptr + p.buf_off + vs[k] * 16, r[k]);
        }
    } else if (p.ws <= 4) {
      U4 x[UNR][4];
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (act[k]) {
#pragma unroll
          for (int s = 0; s < 4; ++s)
            if (s < p.ws) {
              int peer = p.rank + s;
              if (peer >= p.ws) peer -= p.ws;
              x[k][s] = ld16(symm_buf(p, peer) + vs[k] * 16);
            }
        }
#pragma unroll
      for (int k = 0; k < UNR; ++k)
        if (act[k]) {
          float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          if (p.bias) add_bias8(p, vs[k] * 8, f);
#pragma unroll
          for (int s = 0; s < 4; ++s)
            if (s < p.ws) acc8(x[k][s], f);
          const U4 r = pack8(f);
          for (int s = 0; s < p.ws; ++s) {
            int peer = p.rank + s;
            if (peer >= p.ws) peer -= p.ws;
            st16(symm_buf(p, peer) + vs[k] * 16, r);
          }
        }
    } else {
#pragma unroll 1
      for (int k = 0; k < UNR; ++k) {
        if (!act[k]) continue;
        const size_t v = vs[k];
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (p.bias) add_bias8(p, v * 8, f);
        U4 x[8];
        for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) {
              int peer = p.rank + s0 + s;
              if (peer >= p.ws) peer -= p.ws;
              x[s] = ld16(symm_buf(p, peer) + v * 16);
            }
#pragma unroll
          for (int s = 0; s < 8; ++s)
            if (s0 + s < p.ws) acc8(x[s], f);
        }
        const U4 r = pack8(f);
        for (int s = 0; s < p.ws; ++s) {
          int peer = p.rank + s;
          if (peer >= p.ws) peer -= p.ws;
          st16(symm_buf(p, peer) + v * 16, r);
        }
      }
    }
  }
  if (!block_sync_T_T(p, bid, 4)) return;
  if (p.output != (void*)own) {
    for (size_t g = bid; g < ngroups; g += nb)
      for (int c = 0; c < p.ws; ++c) {
        size_t v = g * group + (size_t)c * blockDim.x + threadIdx.x;
        if (v < nvec) st16((char*)p.output + v * 16, ld16(own + v * 16));
      }
    // Peers must not overwrite this buffer (next call's copy-in / publish) before it is drained.
    block_sync_T_F(p, bid, 5);
  }
}
__device__ void two_shot_ar_body(const CommParams& p, unsigned bid, unsigned nb) { two_shot_ar_impl<false>(p, bid, nb); }
__device__ void two_shot_ar_mc_body(const CommParams& p, unsigned bid, unsigned nb) { two_shot_ar_impl<true>(p, bid, nb); }
KR_DEFINE_RANKED_KERNEL(two_shot_ar, CommParams, kCommThreads)
KR_DEFINE_RANKED_KERNEL(two_shot_ar_mc, CommParams, kCommThreads)

// ---------------------------------------------------------------------------------------------
// Reduce-scatter: rank r sums slab r (numel/ws elements) of every rank's buffer into `output`.
// ---------------------------------------------------------------------------------------------
__device__ void reduce_scatter_body(const CommParams& p, unsigned bid, unsigned nb) {
  const size_t slab_vec = p.numel / p.ws / 8;   // host: numel % (8*ws) == 0
  const size_t stride = (size_t)nb * blockDim.x;
  const size_t first = (size_t)bid * blockDim.x + threadIdx.x;
  char* own = symm_buf(p, p.rank);
  if (p.input != nullptr) {
    // Block b stages, for EVERY slab, exactly the in-slab vectors that block b of the slab's
    // owner will read, so the per-block barrier is all the ordering the pull needs.
    for (int s = 0; s < p.ws; ++s) {
      const size_t off = (size_t)s * slab_vec;
      for (size_t v = first; v < slab_vec; v += stride)
        st16(own + (off + v) * 16, ld16((const char*)p.input + (off + v) * 16));
    }
    if (!block_sync_T_T(p, bid, 6)) return;
  } else {
    if (!block_sync_F_T(p, bid, 6)) return;
  }
  const size_t base = (size_t)p.rank * slab_vec;
  for (size_t v = first; v < slab_vec; v += stride) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    U4 x[8];
    for (int s0 = 0; s0 < p.ws; s0 += 8) {
      // fixed rank order 0..ws-1 keeps the sum bitwise reproducible
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s0 + s < p.ws) x[s] = ld16(symm_buf(p, s0 + s) + (base + v) * 16);
#pragma unroll
      for (int s = 0; s < 8; ++s)
        if (s0 + s < p.ws) acc8(x[s], f);
    }
    st16((char*)p.output + v * 16, pack8(f));
  }
  block_sync_T_F(p, bid, 7);
}
KR_DEFINE_RANKED_KERNEL(reduce_scatter, CommParams, kCommThreads)

// ---------------------------------------------------------------------------------------------
// SM-pull all-gather with progress flags: bufs[r] holds rank r's shard (numel elements);
// `output` is [ws * numel]. Chunk index = src * splits + split (the reference's layout,
// copy_engine_all_gather.py:30-54); chunks are fetched starting at rank+1 so the own shard comes
// last, and progress[idx] becomes 1 (release.gpu) once the whole chunk has landed.
// ---------------------------------------------------------------------------------------------
__device__ void all_gather_body(const CommParams& p, unsigned bid, unsigned nb) {
  if (!block_sync_F_T(p, bid, 8)) return;
  const size_t chunk_vec = p.numel / p.splits / 8;   // host: numel % (8*splits) == 0
  const size_t stride = (size_t)nb * blockDim.x;
  const size_t first = (size_t)bid * blockDim.x + threadIdx.x;
  for (int step = 0; step < p.ws; ++step) {
    const int src = (p.rank + step + 1) % p.ws;
    for (int sp = 0; sp < p.splits; ++sp) {
      const int idx = src * p.splits + sp;
      if (!kr_in_bounds(idx >= 0 && idx < p.ws * p.splits, p.sync, 74)) continue;
      const char* from = symm_buf(p, src) + (size_t)sp * chunk_vec * 16;
      char* to = (char*)p.output + (size_t)idx * chunk_vec * 16;
      size_t v = first;
      for (; v + 3 * stride < chunk_vec; v += 4 * stride) {
        U4 a = ld16(from + v * 16), b = ld16(from + (v + stride) * 16);
        U4 c = ld16(from + (v + 2 * stride) * 16), d = ld16(from + (v + 3 * stride) * 16);
        st16(to + v * 16, a); st16(to + (v + stride) * 16, b);
        st16(to + (v + 2 * stride) * 16, c); st16(to + (v + 3 * stride) * 16, d);
      }
      for (; v < chunk_vec; v += stride) st16(to + v * 16, ld16(from + v * 16));
      __syncthreads();
      if (threadIdx.x == 0) {
        uint32_t old = atom_add_acqrel_gpu(p.counters + idx, 1u);
        if (old == nb - 1) {
          p.counters[idx] = 0;
          st_release_gpu(p.progress + idx, 1u);
        }
      }
    }
  }
  block_sync_T_F(p, bid, 9);
}
KR_DEFINE_RANKED_KERNEL(all_gather, CommParams, kCommThreads)

// ---------------------------------------------------------------------------------------------
// Local slab reduction (K14 of the reference, gemm_reduce_scatter_ce_persistent.py:245-323):
// out[slab_numel] = sum_i slabs[(start + i) % ws], fp32 accumulate.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kCommThreads) reduce_slabs_kernel(const char* slabs, char* out, int ws, int start,
                                                                     size_t slab_vec) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < slab_vec; v += stride) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < ws; ++i) {
      int s = start + i;
      if (s >= ws) s -= ws;
      acc8(ld16(slabs + ((size_t)s * slab_vec + v) * 16), f);
    }
    st16(out + v * 16, pack8(f));
  }
}

// ---------------------------------------------------------------------------------------------
// Barrier / flag test kernels (the library's own checks of ptx_sync.cuh).
// ---------------------------------------------------------------------------------------------
struct SyncTestParams {
  uint32_t* const* pads;
  uint32_t* flags;       // gmem barrier test: one flag per producer
  uint32_t* out;         // results
  int rank, ws;
  int mode;              // 0: symm_mem_sync x3 patterns; 1: gmem arrive/wait; 2: wait on a flag nothing sets
  int num_producers;
  SyncCtx sync;
};
__device__ void sync_test_body(const SyncTestParams& p, unsigned bid, unsigned nb) {
  if (p.mode == 0) {
    bool ok = symm_mem_sync<false, true>(p.pads, bid, p.rank, p.ws, p.sync, 20);
    ok = ok && symm_mem_sync<true, true>(p.pads, bid, p.rank, p.ws, p.sync, 21);
    ok = ok && symm_mem_sync<true, false>(p.pads, bid, p.rank, p.ws, p.sync, 22);
    if (threadIdx.x == 0) p.out[bid] = ok ? 1u : 0u;
  } else if (p.mode == 1) {
    // blocks [0, num_producers) publish; every other block waits on flag (bid % num_producers)
    if ((int)bid < p.num_producers) {
      if (threadIdx.x == 0) p.out[bid] = 7u;
      arrive_gmem_barrier(p.flags + bid, 1u);
    } else {
      int src = bid % p.num_producers;
      bool ok = wait_gmem_barrier(p.flags + src, 1u, p.sync, 23);
      if (threadIdx.x == 0) p.out[bid] = ok ? ld_volatile_u32(p.out + src) : 0u;
    }
  } else if (p.mode == 2) {
    bool ok = wait_gmem_barrier(p.flags + bid, 1u, p.sync, 24);
    if (threadIdx.x == 0) p.out[bid] = ok ? 1u : 2u;
  } else if (p.mode >= 4) {
    // one barrier of the pattern the caller names: bit 1 = earlier accesses, bit 0 = later accesses
    bool ok;
    switch (p.mode & 3) {
      case 0: ok = symm_mem_sync<false, false>(p.pads, bid, p.rank, p.ws, p.sync, 26); break;
      case 1: ok = symm_mem_sync<false, true>(p.pads, bid, p.rank, p.ws, p.sync, 27); break;
      case 2: ok = symm_mem_sync<true, false>(p.pads, bid, p.rank, p.ws, p.sync, 28); break;
      default: ok = symm_mem_sync<true, true>(p.pads, bid, p.rank, p.ws, p.sync, 29); break;
    }
    if (threadIdx.x == 0) p.out[bid] = ok ? 1u : 0u;
  } else {
    // Bounds-check self-test: index num_producers is checked against a limit of num_producers
    // (one past the end). In the debug build the check fails, records KR_ERR_BOUNDS and the store is
    // skipped (out stays 0); in the regular build the check is compiled away and the store happens —
    // inside the buffer either way, which the host sizes with one spare word.
    if (threadIdx.x == 0 && kr_in_bounds(p.num_producers < p.num_producers, p.sync, 75)) p.out[p.num_producers] = 3u;
  }
}
KR_DEFINE_RANKED_KERNEL(sync_test, SyncTestParams, 128)

// One-block cross-device barrier with full release/acquire semantics (handle.barrier()).
__device__ void symm_barrier_body(const SyncTestParams& p, unsigned, unsigned) {
  symm_mem_sync<true, true>(p.pads, (uint32_t)p.mode, p.rank, p.ws, p.sync, 25);
}
KR_DEFINE_RANKED_KERNEL(symm_barrier, SyncTestParams, 128)

}  // namespace kraken

using namespace kraken;

static unsigned pick_blocks(const DeviceState* d, size_t nvec, int max_blocks, unsigned vec_per_block) {
  unsigned nb = cdiv(nvec, vec_per_block);
  unsigned cap = (unsigned)d->num_sms;
  if (max_blocks > 0 && (unsigned)max_blocks < cap) cap = (unsigned)max_blocks;
  if (emu_recorder().active) {
    unsigned per = (unsigned)d->num_sms / (unsigned)emu_recorder().ws;
    if (per < 1) per = 1;
    if (cap > per) cap = per;
  }
  if (nb < 1) nb = 1;
  return nb > cap ? cap : nb;
}

static int fill_common(CommParams& p, DeviceState* d, void* const* bufs, unsigned long long buf_off,
                       uint32_t* const* pads, int rank, int ws, unsigned long long numel, const void* bias,
                       unsigned long long bias_numel, uint32_t pad_base) {
  KR_REQUIRE(buf_off % 16 == 0, "symmetric tensor must start 16-byte aligned inside its buffer");
  KR_REQUIRE(ws >= 1 && ws <= 72 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  if (bias) {
    KR_REQUIRE(bias_numel > 0 && bias_numel % 8 == 0, "bias length must be a positive multiple of 8");
    KR_REQUIRE(((uintptr_t)bias & 15) == 0, "bias must be 16-byte aligned");
  }
  memset(&p, 0, sizeof(p));
  p.bufs = bufs;
  p.buf_off = buf_off;
  p.pads = pads;
  p.rank = rank;
  p.ws = ws;
  p.numel = numel;
  p.bias = bias;
  p.bias_period = bias ? bias_numel : 8;
  p.pad_base = pad_base;
  p.splits = 1;
  p.sync = sync_ctx(d);
  return KR_SUCCESS;
}

// Scratch counters (zeroed once, self-resetting) for kernels that count block arrivals.
static int scratch_counters(DeviceState* d, uint32_t** out) {
  static std::map<int, uint32_t*>* tbl = new std::map<int, uint32_t*>();
  auto it = tbl->find(d->device);
  if (it == tbl->end()) {
    uint32_t* ptr = nullptr;
    KR_CUDA(cudaMalloc(&ptr, 4096 * sizeof(uint32_t)));
    KR_CUDA(cudaMemset(ptr, 0, 4096 * sizeof(uint32_t)));
    it = tbl->emplace(d->device, ptr).first;
  }
  *out = it->second;
  return KR_SUCCESS;
}

// out = bias + sum_r bufs[r]   (bias optional; input optional: copied into bufs[rank] first)
KR_API int kr_one_shot_all_reduce(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank, int ws, const void* input,
                                  void* output, const void* bias, unsigned long long bias_numel,
                                  unsigned long long numel, int max_blocks, uint32_t pad_base,
                                  cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  CommParams p;
  int rc = fill_common(p, d, bufs, buf_off, pads, rank, ws, numel, bias, bias_numel, pad_base);
  if (rc) return rc;
  KR_REQUIRE(((uintptr_t)output & 15) == 0 && ((uintptr_t)input & 15) == 0, "tensors must be 16-byte aligned");
  p.input = input;
  p.output = output;
  unsigned nb = pick_blocks(d, numel / 8, max_blocks, kCommThreads * 2);
  return launch_ranked(one_shot_ar_kernel, one_shot_ar_emu_kernel, p, nb, kCommThreads, 0, stream);
}

// Two-shot all-reduce; mc_ptr != nullptr selects the NVLS (multimem) form. output may be the own
// symmetric buffer (in place: no copy-out).
KR_API int kr_two_shot_all_reduce(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank, int ws, const void* input,
                                  void* output, const void* bias, unsigned long long bias_numel,
                                  unsigned long long numel, void* mc_ptr, int max_blocks, uint32_t pad_base,
                                  cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  CommParams p;
  int rc = fill_common(p, d, bufs, buf_off, pads, rank, ws, numel, bias, bias_numel, pad_base);
  if (rc) return rc;
  KR_REQUIRE(numel % 8 == 0, "two-shot all-reduce needs numel % 8 == 0");
  KR_REQUIRE(((uintptr_t)output & 15) == 0 && ((uintptr_t)input & 15) == 0, "tensors must be 16-byte aligned");
  p.input = input;
  p.output = output;
  p.mc_ptr = mc_ptr;
  unsigned nb = pick_blocks(d, numel / 8, max_blocks, kCommThreads * ws);
  if (mc_ptr) return launch_ranked(two_shot_ar_mc_kernel, two_shot_ar_mc_emu_kernel, p, nb, kCommThreads, 0, stream);
  return launch_ranked(two_shot_ar_kernel, two_shot_ar_emu_kernel, p, nb, kCommThreads, 0, stream);
}

// output[numel/ws] = sum_r bufs[r][rank*numel/ws ...]
KR_API int kr_reduce_scatter(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank, int ws, const void* input,
                             void* output, unsigned long long numel, int max_blocks, uint32_t pad_base,
                             cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  CommParams p;
  int rc = fill_common(p, d, bufs, buf_off, pads, rank, ws, numel, nullptr, 0, pad_base);
  if (rc) return rc;
  KR_REQUIRE(numel % (8ull * ws) == 0, "reduce-scatter needs numel % (8 * world_size) == 0");
  KR_REQUIRE(((uintptr_t)output & 15) == 0 && ((uintptr_t)input & 15) == 0, "tensors must be 16-byte aligned");
  p.input = input;
  p.output = output;
  unsigned nb = pick_blocks(d, numel / 8 / ws, max_blocks, kCommThreads * 2);
  return launch_ranked(reduce_scatter_kernel, reduce_scatter_emu_kernel, p, nb, kCommThreads, 0, stream);
}

// output[ws * numel] = concat_r bufs[r][0 .. numel); progress[ws*splits] set to 1 chunk by chunk.
KR_API int kr_all_gather_sm(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank, int ws, void* output,
                            uint32_t* progress, uint32_t* counters, int splits, unsigned long long numel,
                            int max_blocks, uint32_t pad_base, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  CommParams p;
  int rc = fill_common(p, d, bufs, buf_off, pads, rank, ws, numel, nullptr, 0, pad_base);
  if (rc) return rc;
  KR_REQUIRE(splits >= 1 && numel % (8ull * splits) == 0, "all-gather needs numel % (8 * splits) == 0");
  KR_REQUIRE(ws * splits <= 2048, "too many chunks");
  KR_REQUIRE(((uintptr_t)output & 15) == 0, "output must be 16-byte aligned");
  p.output = output;
  p.progress = progress;
  p.splits = splits;
  if (counters) {
    p.counters = counters;
  } else {
    KR_REQUIRE(!emu_recorder().active, "emulated ranks need their own counters");
    rc = scratch_counters(d, &p.counters);
    if (rc) return rc;
  }
  unsigned nb = pick_blocks(d, numel / 8 / splits, max_blocks, kCommThreads * 4);
  return launch_ranked(all_gather_kernel, all_gather_emu_kernel, p, nb, kCommThreads, 0, stream);
}

KR_API int kr_reduce_slabs(const void* slabs, void* out, int ws, int start, unsigned long long slab_numel,
                           cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && start >= 0 && start < ws, "bad slab rotation");
  KR_REQUIRE(slab_numel % 8 == 0, "slab size must be a multiple of 8 elements");
  KR_REQUIRE((((uintptr_t)slabs | (uintptr_t)out) & 15) == 0, "tensors must be 16-byte aligned");
  if (slab_numel == 0) return KR_SUCCESS;
  unsigned nb = cdiv(slab_numel / 8, kCommThreads * 2);
  if (nb > (unsigned)d->num_sms * 4) nb = (unsigned)d->num_sms * 4;
  reduce_slabs_kernel<<<nb, kCommThreads, 0, stream>>>((const char*)slabs, (char*)out, ws, start, slab_numel / 8);
  KR_CUDA(cudaGetLastError());
  return KR_SUCCESS;
}

// mode 0: three symm_mem_sync patterns per block; 1: gmem arrive/wait; 2: wait that must time out;
// 3: bounds-check self-test (out needs num_producers + 1 words); 4..7: ONE symm_mem_sync per block,
// pattern = (mode & 2: the block accessed symmetric memory before, mode & 1: it will after).
KR_API int kr_sync_test(uint32_t* const* pads, int rank, int ws, uint32_t* flags, uint32_t* out, int mode,
                        int num_blocks, int num_producers, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  SyncTestParams p;
  memset(&p, 0, sizeof(p));
  p.pads = pads;
  p.rank = rank;
  p.ws = ws;
  p.flags = flags;
  p.out = out;
  p.mode = mode;
  p.num_producers = num_producers;
  p.sync = sync_ctx(d);
  KR_REQUIRE(num_blocks >= 1 && num_blocks <= d->num_sms, "sync test grid must fit the device");
  return launch_ranked(sync_test_kernel, sync_test_emu_kernel, p, (unsigned)num_blocks, 128, 0, stream);
}

// Cross-device barrier of all ranks on `stream`, using barrier slot `slot` of the signal pads.
KR_API int kr_symm_barrier(uint32_t* const* pads, int rank, int ws, int slot, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ws >= 1 && rank >= 0 && rank < ws && slot >= 0, "bad barrier arguments");
  SyncTestParams p;
  memset(&p, 0, sizeof(p));
  p.pads = pads;
  p.rank = rank;
  p.ws = ws;
  p.mode = slot;
  p.sync = sync_ctx(d);
  return launch_ranked(symm_barrier_kernel, symm_barrier_emu_kernel, p, 1, 128, 0, stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the SM all-gather (declared in kraken/no_alloc.h). The arrival
// counters and a status word live in a fixed device array instead of allocated memory.
// ---------------------------------------------------------------------------------------------
#include "kraken/no_alloc.h"

namespace kraken {
constexpr int kNoAllocStatusWords = 64;   // 256 bytes: word 0 is the default status word
static __device__ __align__(256) uint32_t g_noalloc_scratch[kNoAllocStatusWords + KR_NOALLOC_MAX_CHUNKS];
static_assert(sizeof(uint32_t) * (kNoAllocStatusWords + KR_NOALLOC_MAX_CHUNKS) == KR_NOALLOC_SCRATCH_BYTES,
              "scratch size stated in the header");

struct NoAllocDevice {
  bool ready = false;
  uint32_t* scratch = nullptr;   // DEVICE address of g_noalloc_scratch on this device
  int num_sms = 0;
};
static NoAllocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_mu;

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address: the
// address a kernel can use has to be asked for, per device, with that device current.
static int noalloc_device(NoAllocDevice** out) {
  int dev = -1;
  KR_CUDA(cudaGetDevice(&dev));
  KR_REQUIRE(dev >= 0 && dev < 64, "device index out of range");
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (!d.ready) {
    void* ptr = nullptr;
    KR_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
    KR_CUDA(cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev));
    d.scratch = (uint32_t*)ptr;
    d.ready = true;
  }
  *out = &d;
  return KR_SUCCESS;
}

static uint64_t g_noalloc_timeout_ns = 0;   // 0: follow the device's setting (or the environment default)

// Deadline of the waits in the allocation-free path: its own setting if one was made, else the
// current device's (when other entry points have created that state), else the environment default.
static uint64_t noalloc_timeout_ns() {
  if (g_noalloc_timeout_ns != 0) return g_noalloc_timeout_ns;
  return current_timeout_ns();
}
}  // namespace kraken

KR_API int kr_all_gather_sm_noalloc(void* const* bufs, unsigned long long buf_off, uint32_t* const* pads, int rank,
                                    int world_size, void* output, uint32_t* progress, int splits,
                                    unsigned long long numel, int max_blocks, uint32_t pad_base, uint32_t* status,
                                    cudaStream_t stream) {
  const int ws = world_size;
  KR_REQUIRE(ws >= 1 && ws <= 72 && rank >= 0 && rank < ws, "bad rank/world size");
  KR_REQUIRE(splits >= 1 && numel % (8ull * splits) == 0, "all-gather needs numel % (8 * splits) == 0");
  if ((unsigned long long)ws * (unsigned long long)splits > KR_NOALLOC_MAX_CHUNKS)
    return fail(KR_FAIL_ARG, "kr_all_gather_sm_noalloc: world_size * splits = " + std::to_string((long long)ws * splits) +
                                 " exceeds the built-in scratch of " + std::to_string(KR_NOALLOC_MAX_CHUNKS) +
                                 " chunks; use kr_all_gather_sm with caller-provided counters");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  KR_REQUIRE(buf_off % 16 == 0 && ((uintptr_t)output & 15) == 0, "tensors must be 16-byte aligned");
  KR_REQUIRE(bufs && pads && output && progress, "null argument");
  KR_REQUIRE(!emu_recorder().active, "not available while rank emulation is recording");
  NoAllocDevice* d = nullptr;
  int rc = noalloc_device(&d);
  if (rc) return rc;
  // The scratch address belongs to the current device: a stream of another device would run the
  // kernel there, against memory it was not meant for.
  int stream_dev = -1, cur_dev = -1;
  KR_CUDA(cudaGetDevice(&cur_dev));
  if (cudaStreamGetDevice(stream, &stream_dev) == cudaSuccess)
    KR_REQUIRE(stream_dev == cur_dev, "kr_all_gather_sm_noalloc: the stream belongs to another device than the current one");
  else
    (void)cudaGetLastError();
  uint32_t* counters = d->scratch + kNoAllocStatusWords;
  // The array keeps whatever the previous call left. The counters must start at zero; so must the
  // built-in status word when this call uses it (a code left there would make every wait give up).
  if (status == nullptr) {
    KR_CUDA(cudaMemsetAsync(d->scratch, 0, sizeof(uint32_t) * ((size_t)kNoAllocStatusWords + (size_t)ws * splits), stream));
  } else {
    KR_CUDA(cudaMemsetAsync(counters, 0, sizeof(uint32_t) * (size_t)ws * splits, stream));
  }
  CommParams p;
  memset(&p, 0, sizeof(p));
  p.bufs = bufs;
  p.buf_off = buf_off;
  p.pads = pads;
  p.rank = rank;
  p.ws = ws;
  p.numel = numel;
  p.bias_period = 8;
  p.pad_base = pad_base;
  p.splits = splits;
  p.output = output;
  p.progress = progress;
  p.counters = counters;
  p.sync = SyncCtx{status ? status : d->scratch, noalloc_timeout_ns()};
  unsigned nb = cdiv(numel / 8 / splits, kCommThreads * 4);
  unsigned cap = (unsigned)d->num_sms;
  if (max_blocks > 0 && (unsigned)max_blocks < cap) cap = (unsigned)max_blocks;
  if (nb < 1) nb = 1;
  if (nb > cap) nb = cap;
  void* args[] = {(void*)&p};
  KR_CUDA(cudaLaunchKernel((const void*)all_gather_kernel, dim3(nb), dim3(kCommThreads), args, 0, stream));
  return KR_SUCCESS;
}

// Reads the built-in status word of the current device (the one calls with status == NULL use)
// after synchronising `stream`; clear != 0 also zeroes it. No allocation.
KR_API int kr_noalloc_read_status(cudaStream_t stream, uint32_t* word, int clear) {
  KR_REQUIRE(word != nullptr, "null argument");
  NoAllocDevice* d = nullptr;
  int rc = noalloc_device(&d);
  if (rc) return rc;
  KR_CUDA(cudaStreamSynchronize(stream));
  KR_CUDA(cudaMemcpy(word, d->scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (clear) KR_CUDA(cudaMemset(d->scratch, 0, sizeof(uint32_t)));
  return KR_SUCCESS;
}

// Deadline of the device-side waits of kr_all_gather_sm_noalloc, in milliseconds; 0 restores the
// default (the current device's kr_set_timeout_ms value, else KRAKEN_SYNC_TIMEOUT_MS, else 4000).
KR_API int kr_noalloc_set_timeout_ms(double ms) {
  KR_REQUIRE(ms >= 0, "timeout must not be negative");
  g_noalloc_timeout_ns = (uint64_t)(ms * 1e6);
  return KR_SUCCESS;
}
