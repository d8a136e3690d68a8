// 16-byte vector access, bf16 <-> fp32 packing and NVLS multimem helpers (sm_100a).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace kraken {

struct alignas(16) U4 {
  uint32_t x, y, z, w;
};

// Plain (weak) 16-byte global load; ordering comes from the surrounding acquire barrier.
// L1::no_allocate: the data is streamed once (peer or staging memory).
__device__ __forceinline__ U4 ld16(const void* p) {
  U4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Read-only path for operands never written during the kernel (bias, norm weights).
__device__ __forceinline__ U4 ld16_nc(const void* p) {
  U4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st16(void* p, const U4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 8 bf16 <-> 8 fp32
__device__ __forceinline__ void unpack8(const U4& v, float (&f)[8]) {
  f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
  f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
}
__device__ __forceinline__ void acc8(const U4& v, float (&f)[8]) {
  f[0] += bf16lo(v.x); f[1] += bf16hi(v.x); f[2] += bf16lo(v.y); f[3] += bf16hi(v.y);
  f[4] += bf16lo(v.z); f[5] += bf16hi(v.z); f[6] += bf16lo(v.w); f[7] += bf16hi(v.w);
}
__device__ __forceinline__ U4 pack8(const float (&f)[8]) {
  U4 v;
  v.x = pack_bf16x2(f[0], f[1]); v.y = pack_bf16x2(f[2], f[3]);
  v.z = pack_bf16x2(f[4], f[5]); v.w = pack_bf16x2(f[6], f[7]);
  return v;
}

// ---- NVLS (multicast address) operations -------------------------------------------------------
// In-switch reduction of 8 bf16 across all devices bound to the multicast object, fp32 accumulate.
__device__ __forceinline__ U4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  U4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
  return v;
}
// In-switch reduction of 4 fp32.
__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const void* mc_ptr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc_ptr) : "memory");
  return v;
}
// Broadcast store of 16 bytes to every device bound to the multicast object.
__device__ __forceinline__ void multimem_st16(void* mc_ptr, const U4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
// The same as a weak store: no ordering of its own, made visible by a later release (a flag).
__device__ __forceinline__ void multimem_st16_weak(void* mc_ptr, const U4& v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
// Broadcast store of one 64-bit word (seen whole at every destination).
__device__ __forceinline__ void multimem_st_u64(void* mc_ptr, unsigned long long v) {
  asm volatile("multimem.st.relaxed.sys.global.u64 [%0], %1;" ::"l"(mc_ptr), "l"(v) : "memory");
}
// Broadcast +1 on a flag word in every bound device's memory.
__device__ __forceinline__ void multimem_red_add_release_u32(uint32_t* mc_ptr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace kraken
