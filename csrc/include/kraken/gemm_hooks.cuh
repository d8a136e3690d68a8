// Epilogue hooks shared by several GEMM translation units: the plain GEMM and the GEMM ->
// all-reduce exchange for decode shapes.
#pragma once
#include "kraken/gemm_core.cuh"

namespace kraken {

struct PlainHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    return TileDest{(char*)p.out, p.ldo, tr * kBM, tc * bn, p.out_rows, p.out_cols, p.use_tma_store ? &p.tmap_out[0] : nullptr};
  }
  __device__ __forceinline__ bool after_store(const GemmParams&, int, int, int, int) { return true; }
};

// GEMM -> all-reduce (decode). Two exchange algorithms behind the same main loop:
//  * one-shot (small M): the fp32 partial tile goes to the rank's OWN staging, a flag goes to
//    every peer, and every rank sums the tile from all ranks (in-switch with multimem.ld_reduce
//    when the staging buffer has a multicast mapping, else ws peer loads in rank order).
//  * two-shot (larger M): tile t belongs to rank t % ws. Every rank stores its partial tile into
//    the OWNER's staging slot [src]; the owner sums the ws slots from its own memory (rank order,
//    so every rank receives identical bits), writes the result into every rank's result buffer
//    (one multimem.st, or ws-1 peer stores) and raises "published" flags; the others copy the tile
//    out. NVLink bytes per rank drop from (ws-1)·M·N·4 to about 2·(ws-1)/ws·M·N·4.
// The staging buffer is dedicated to this op. One-shot alternates between two staging halves and
// two flag banks from call to call, and in two-shot nobody leaves before every tile it takes part
// in is published, so neither needs an exit barrier.
struct ArHooks : HookDefaults {
  int bn;
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ int tile_of(const GemmParams& p, int tr, int tc) const { return tr * p.tiles_c + tc; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    char* base;
    if (p.ar_algo == 0) {
      base = (char*)p.bufs[p.rank] + p.stage_off;
    } else {
      const int owner = tile_of(p, tr, tc) % p.ws;
      base = (char*)p.bufs[owner] + p.part_off + (size_t)p.rank * p.out_rows * p.out_cols * 4;
    }
    return TileDest{base, (long long)p.out_cols, tr * kBM, tc * bn, p.out_rows, p.out_cols, nullptr};
  }
  // region of tile (tr, tc) in the orientation of `out`
  __device__ __forceinline__ void region(const GemmParams& p, int tr, int tc, int& r_lo, int& r_n, int& c_lo, int& c_n) {
    if (p.transposed) { r_lo = tc * bn; r_n = bn; c_lo = tr * kBM; c_n = kBM; }
    else { r_lo = tr * kBM; r_n = kBM; c_lo = tc * bn; c_n = bn; }
  }
  __device__ __forceinline__ bool wait_count(uint32_t* f, uint32_t need, const GemmParams& p, uint32_t site) {
    if (need == 0) return true;
    if (spin_until([&] { return ld_acquire_sys(f) >= need; }, p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, site, 0, blockIdx.x))) {
      red_add_relaxed_sys(f, 0u - need);
      return true;
    }
    return false;
  }
  __device__ __forceinline__ bool after_store(const GemmParams& p, int tr, int tc, int q, int lane) {
    const int tile = tile_of(p, tr, tc);
    const int tid = q * 32 + lane;   // 0..127 over the epilogue warps
    int r_lo, r_n, c_lo, c_n;
    region(p, tr, tc, r_lo, r_n, c_lo, c_n);
    const int upr = c_n / 4;         // 16-byte units per tile row
    const bool vec = (p.out_cols % 4) == 0 && (p.ldo % 4) == 0;
    const size_t mn4 = (size_t)p.out_rows * p.out_cols * 4;
    epi_bar_sync();                  // the whole tile has been stored
    if (p.ar_algo == 0) {
      // ---------------- one-shot ----------------
      if (tid < p.ws && tid != p.rank) red_add_release_sys(p.pads[tid] + p.flag_base + tile, 1u);
      if (tid == 0) wait_count(p.pads[p.rank] + p.flag_base + tile, (uint32_t)(p.ws - 1), p, 51);
      epi_bar_sync();
      if (!status_ok(p.sync)) return false;
      for (int i0 = tid; i0 < r_n * upr; i0 += 256) {
        size_t off[2];
        int rr[2], cc[2];
        bool act[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int i = i0 + 128 * k;
          rr[k] = r_lo + i / upr;
          cc[k] = c_lo + (i % upr) * 4;
          act[k] = i < r_n * upr && rr[k] < p.out_rows && cc[k] < p.out_cols;
          off[k] = ((size_t)rr[k] * p.out_cols + cc[k]) * 4;
        }
        if (vec && p.mc_ptr != nullptr) {
          float4 a[2];
#pragma unroll
          for (int k = 0; k < 2; ++k)
            if (act[k]) a[k] = multimem_ld_reduce_f32x4((const char*)p.mc_ptr + p.stage_off + off[k]);
#pragma unroll
          for (int k = 0; k < 2; ++k)
            if (act[k]) *(float4*)((float*)p.out + (size_t)rr[k] * p.ldo + cc[k]) = a[k];
        } else if (vec) {
          U4 x[2][8];
          float4 a[2];
          a[0] = a[1] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
            for (int k = 0; k < 2; ++k)
#pragma unroll
              for (int s = 0; s < 8; ++s)
                if (act[k] && s0 + s < p.ws) x[k][s] = ld16((const char*)p.bufs[s0 + s] + p.stage_off + off[k]);
#pragma unroll
            for (int k = 0; k < 2; ++k)
#pragma unroll
              for (int s = 0; s < 8; ++s)
                if (act[k] && s0 + s < p.ws) {
                  a[k].x += __uint_as_float(x[k][s].x); a[k].y += __uint_as_float(x[k][s].y);
                  a[k].z += __uint_as_float(x[k][s].z); a[k].w += __uint_as_float(x[k][s].w);
                }
          }
#pragma unroll
          for (int k = 0; k < 2; ++k)
            if (act[k]) *(float4*)((float*)p.out + (size_t)rr[k] * p.ldo + cc[k]) = a[k];
        } else {
          for (int k = 0; k < 2; ++k) {
            if (!act[k]) continue;
            for (int e = 0; e < 4 && cc[k] + e < p.out_cols; ++e) {
              float acc = 0.f;
              for (int s = 0; s < p.ws; ++s)
                acc += ((const volatile float*)((const char*)p.bufs[s] + p.stage_off + off[k]))[e];
              ((float*)p.out)[(size_t)rr[k] * p.ldo + cc[k] + e] = acc;
            }
          }
        }
      }
      return true;
    }
    // ---------------- two-shot ----------------
    const int owner = tile % p.ws;
    if (tid == 0) red_add_release_sys(p.pads[owner] + p.flag_base + tile, 1u);
    if (owner == p.rank) {
      if (tid == 0) wait_count(p.pads[p.rank] + p.flag_base + tile, (uint32_t)p.ws, p, 58);
      epi_bar_sync();
      if (!status_ok(p.sync)) return false;
      const char* part = (const char*)p.bufs[p.rank] + p.part_off;
      for (int i = tid; i < r_n * upr; i += 128) {
        const int rr = r_lo + i / upr, cc = c_lo + (i % upr) * 4;
        if (rr >= p.out_rows || cc >= p.out_cols) continue;
        const size_t off = ((size_t)rr * p.out_cols + cc) * 4;
        if (vec) {
          U4 x[8];
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int s0 = 0; s0 < p.ws; s0 += 8) {
#pragma unroll
            for (int s = 0; s < 8; ++s)
              if (s0 + s < p.ws) x[s] = ld16(part + (size_t)(s0 + s) * mn4 + off);
#pragma unroll
            for (int s = 0; s < 8; ++s)
              if (s0 + s < p.ws) {
                a.x += __uint_as_float(x[s].x); a.y += __uint_as_float(x[s].y);
                a.z += __uint_as_float(x[s].z); a.w += __uint_as_float(x[s].w);
              }
          }
          *(float4*)((float*)p.out + (size_t)rr * p.ldo + cc) = a;
          const U4 v = U4{__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w)};
          if (p.mc_ptr != nullptr) {
            multimem_st16((char*)p.mc_ptr + p.res_off + off, v);
          } else {
            for (int s = 1; s < p.ws; ++s) {
              int peer = p.rank + s;
              if (peer >= p.ws) peer -= p.ws;
              st16((char*)p.bufs[peer] + p.res_off + off, v);
            }
          }
        } else {
          for (int e = 0; e < 4 && cc + e < p.out_cols; ++e) {
            float acc = 0.f;
            for (int s = 0; s < p.ws; ++s) acc += ((const float*)(part + (size_t)s * mn4 + off))[e];
            ((float*)p.out)[(size_t)rr * p.ldo + cc + e] = acc;
            for (int s = 1; s < p.ws; ++s)
              ((float*)((char*)p.bufs[(p.rank + s) % p.ws] + p.res_off + off))[e] = acc;
          }
        }
      }
      epi_bar_sync();                // every thread's result stores are issued
      if (tid < p.ws && tid != p.rank) red_add_release_sys(p.pads[tid] + p.flag2_base + tile, 1u);
      return true;
    }
    if (tid == 0) wait_count(p.pads[p.rank] + p.flag2_base + tile, 1u, p, 59);
    epi_bar_sync();
    if (!status_ok(p.sync)) return false;
    const char* res = (const char*)p.bufs[p.rank] + p.res_off;
    for (int i = tid; i < r_n * upr; i += 128) {
      const int rr = r_lo + i / upr, cc = c_lo + (i % upr) * 4;
      if (rr >= p.out_rows || cc >= p.out_cols) continue;
      const size_t off = ((size_t)rr * p.out_cols + cc) * 4;
      if (vec) {
        const U4 v = ld16(res + off);
        st16((char*)((float*)p.out + (size_t)rr * p.ldo + cc), v);
      } else {
        for (int e = 0; e < 4 && cc + e < p.out_cols; ++e)
          ((float*)p.out)[(size_t)rr * p.ldo + cc + e] = ((const float*)(res + off))[e];
      }
    }
    return true;
  }
};

}  // namespace kraken
