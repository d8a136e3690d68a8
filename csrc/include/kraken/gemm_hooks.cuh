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

// GEMM -> all-reduce (decode). Exchanges behind the same main loop (GemmParams::ar_algo):
//  0 one-shot (small outputs): the fp32 partial tile goes to the rank's OWN staging, a flag goes to
//    every peer, and every rank sums the tile from all ranks (in-switch with multimem.ld_reduce
//    when the staging buffer has a multicast mapping, else ws peer loads in rank order).
//  1 two-shot (large outputs): tile t belongs to rank t % ws. Every rank stores its partial tile into
//    the OWNER's staging slot [src]; the owner sums the slots from its own memory (slot order, so
//    every rank receives identical bits), writes the result into every rank's result buffer (one
//    multimem.st, or ws-1 peer stores) and raises "published" flags; the others copy the tile out.
//    NVLink bytes per rank drop from (ws-1)·M·N·4 to about 2·(ws-1)/ws·M·N·4.
//  2 tagged push and 3 tagged two-shot (TAGGED kernels: decode rows, transposed tiles): the same
//    two data flows without any flag — every partial element travels with the call's tag in one
//    8-byte store and the reader polls the pairs; the sums happen after the CTA's last tile, in
//    helper_role. See the comments at helper_role and two_shot_tagged.
// With K split over several CTAs per tile (k_split), every split is one more slot of the exchange.
// The staging buffer is dedicated to this op. One-shot and the tagged forms alternate between two
// staging regions (and flag banks) from call to call, and in two-shot nobody leaves before every
// tile it takes part in is published, so none needs an exit barrier.
template <bool TAGGED>
struct ArHooksT : HookDefaults {
  int bn;
  __device__ __forceinline__ bool begin_tile(const GemmParams&, int, int, int, int) { return true; }
  __device__ __forceinline__ void add_to_chunk(const GemmParams&, int, int, int, int, uint32_t (&)[32], int) {}
  __device__ __forceinline__ bool before_load(const GemmParams&, int, const CUtensorMap*&, int&) { return true; }
  __device__ __forceinline__ int tile_of(const GemmParams& p, int tr, int tc) const { return tr * p.tiles_c + tc; }
  __device__ __forceinline__ TileDest tile_dest(const GemmParams& p, int tr, int tc) {
    char* base;
    const int slot = p.rank * nsplit(p) + k_split;
    const size_t mn = (size_t)p.out_rows * p.out_cols;
    if (TAGGED && p.ar_algo == 2) {
      TileDest d{nullptr, (long long)p.out_cols, tr * kBM, tc * bn, p.out_rows, p.out_cols, nullptr};
      d.ll_tag = p.ll_tag;
      d.ll_off = p.ll_off + (unsigned long long)slot * mn * 8ull;
      return d;
    }
    if (TAGGED && p.ar_algo == 3) {
      // tagged two-shot: the pairs go to the tile's owner only, into the slot's packed array of
      // that owner's tiles (tile-local coordinates, 128 pairs per row)
      const int tile = tile_of(p, tr, tc);
      TileDest d{nullptr, (long long)p.out_cols, tr * kBM, tc * bn, p.out_rows, p.out_cols, nullptr};
      d.ll_tag = p.ll_tag;
      d.ll_off = p.ll_off + ((unsigned long long)slot * p.ll_slot_pairs + (unsigned long long)(tile / p.ws) * bn * kBM) * 8ull;
      d.ll_row0 = tc * bn;
      d.ll_col0 = tr * kBM;
      d.ll_ld = kBM;
      d.ll_dst = tile % p.ws;
      return d;
    }
    if (p.ar_algo == 0) {
      base = (char*)p.bufs[p.rank] + p.stage_off;
    } else {
      const int owner = tile_of(p, tr, tc) % p.ws;
      base = (char*)p.bufs[owner] + p.part_off + (size_t)slot * mn * 4;
    }
    return TileDest{base, (long long)p.out_cols, tr * kBM, tc * bn, p.out_rows, p.out_cols, nullptr};
  }
  __device__ __forceinline__ int nsplit(const GemmParams& p) const { return p.k_splits > 1 ? p.k_splits : 1; }
  // Polls `nsl` slots (stride `stride` bytes) of four consecutive tagged pairs at `src` until all
  // carry the tag and adds the values, slot after slot, into acc. False when the wait gave up.
  __device__ __forceinline__ bool poll_quad(const GemmParams& p, const char* src, size_t stride, int nsl, float (&acc)[4]) {
    {
      const size_t first = (size_t)(src - (const char*)p.peer_buf[p.rank]);
      if (!kr_in_bounds(first >= p.ll_off && first + (size_t)(nsl - 1) * stride + 32 <= p.ll_end, p.sync, 77)) return false;
    }
    for (int s0 = 0; s0 < nsl; s0 += 4) {
      unsigned long long v[4][4];
      const bool ok = spin_until(
          [&] {
            bool all = true;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (s0 + k < nsl) {
                const char* q = src + (size_t)(s0 + k) * stride;
                ld_relaxed_sys_u64x2(q, v[k][0], v[k][1]);
                ld_relaxed_sys_u64x2(q + 16, v[k][2], v[k][3]);
#pragma unroll
                for (int e = 0; e < 4; ++e) all = all && (uint32_t)(v[k][e] >> 32) == p.ll_tag;
              }
            return all;
          },
          p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 53, 0, blockIdx.x));
      if (!ok) return false;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (s0 + k < nsl) {
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[e] += __uint_as_float((uint32_t)v[k][e]);
        }
    }
    return true;
  }
  // Tagged two-shot (out_cols % 4 == 0): the epilogue sent each partial tile, as tagged pairs, to the
  // tile's owner (tile % ws) only. After its last tile every CTA walks its work items again: for a
  // tile this rank owns it sums its share of the tile over all slots as the pairs land, writes the
  // result and publishes it, tagged again, into every rank's result array (one multimem.st per
  // pair, or ws - 1 stores); for any other tile it polls its own result array and copies the values
  // out. All ranks walk the same items in the same order and no CTA waits before its own pairs are
  // out, so every wait is for data whose producer waits for nothing later: no cycle.
  __device__ __forceinline__ void two_shot_tagged(const GemmParams& p, unsigned bid, unsigned nb, int tid) {
    const int ks = nsplit(p), nslots = p.ws * ks;
    const int tiles_rc = p.tiles_r * p.tiles_c;
    const char* mine = (const char*)p.peer_buf[p.rank];
    const unsigned long long tagw = (unsigned long long)p.ll_tag << 32;
    for (int t = (int)bid; t < tiles_rc * ks; t += (int)nb) {
      const int split = t / tiles_rc;
      int tr, tc;
      tile_coords(p, t - split * tiles_rc, tr, tc);
      const int tile = tile_of(p, tr, tc), owner = tile % p.ws;
      int r_lo, r_n, c_lo, c_n;
      region(p, tr, tc, r_lo, r_n, c_lo, c_n);
      const int r_full = r_n;
      if (r_lo + r_n > p.out_rows) r_n = p.out_rows - r_lo;
      if (r_n <= 0) continue;
      const int nq = r_n * c_n / 4;
      const int lo = (int)((long long)nq * split / ks), hi = (int)((long long)nq * (split + 1) / ks);
      for (int qd = lo + tid; qd < hi; qd += kGemmThreads) {
        const int i = qd * 4;
        const int lr = i / c_n, lc = i % c_n;
        const int rr = r_lo + lr, cc = c_lo + lc;
        if (cc >= p.out_cols) continue;
        const size_t res = p.ll_res_off + ((size_t)rr * p.out_cols + cc) * 8;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (owner == p.rank) {
          const char* src = mine + p.ll_off + ((size_t)(tile / p.ws) * r_full * c_n + (size_t)lr * c_n + lc) * 8;
          if (!poll_quad(p, src, (size_t)p.ll_slot_pairs * 8, nslots, acc)) return;
          if (p.mc_ptr != nullptr) {
#pragma unroll
            for (int e = 0; e < 4; ++e) multimem_st_u64((char*)p.mc_ptr + res + 8 * e, tagw | __float_as_uint(acc[e]));
          } else {
            for (int s = 1; s < p.ws; ++s) {
              int peer = p.rank + s;
              if (peer >= p.ws) peer -= p.ws;
#pragma unroll
              for (int e = 0; e < 4; ++e) st_relaxed_sys_u64((char*)p.peer_buf[peer] + res + 8 * e, tagw | __float_as_uint(acc[e]));
            }
          }
        } else {
          if (!poll_quad(p, mine + res, 0, 1, acc)) return;
        }
        float* o = (float*)p.out + (size_t)rr * p.ldo + cc;
        if ((((uintptr_t)o) & 15) == 0) {
          *(float4*)o = make_float4(acc[0], acc[1], acc[2], acc[3]);
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = acc[e];
        }
      }
    }
  }
  // Tagged push: the epilogue has already written this CTA's partial tiles, as {value, tag} pairs,
  // into slot [rank * splits + split] of every rank's staging. Once all of this CTA's tiles are out
  // (so that no CTA ever waits while it still owes a peer data), the six pipeline warps sum, for
  // each work item of the CTA, that item's share of its tile over all ws * splits slots of the OWN
  // staging, polling each pair until it carries this call's tag. No flag, no fence: the 8-byte pair
  // is one atomic store. Slots are summed in slot order, so every rank gets identical bits.
  __device__ __forceinline__ void helper_role(const GemmParams& p, unsigned bid, unsigned nb, int, int tid) {
    if (!TAGGED || p.ar_algo < 2) return;
    if (p.ar_algo == 3) {
      two_shot_tagged(p, bid, nb, tid);
      return;
    }
    const int ks = nsplit(p), nslots = p.ws * ks;
    const int tiles_rc = p.tiles_r * p.tiles_c;
    const size_t mn = (size_t)p.out_rows * p.out_cols;
    const char* mine = (const char*)p.peer_buf[p.rank] + p.ll_off;
    for (int t = (int)bid; t < tiles_rc * ks; t += (int)nb) {
      const int split = t / tiles_rc;
      int tr, tc;
      tile_coords(p, t - split * tiles_rc, tr, tc);
      int r_lo, r_n, c_lo, c_n;
      region(p, tr, tc, r_lo, r_n, c_lo, c_n);
      if (r_lo + r_n > p.out_rows) r_n = p.out_rows - r_lo;
      if (r_n <= 0) continue;
      const int n = r_n * c_n;
      const char* tile_src = mine;
      if ((p.out_cols & 1) == 0) {
        // Four consecutive elements per thread and step: their {value, tag} pairs are two 16-byte
        // loads per slot, so one poll keeps up to eight loads in flight instead of one element's.
        const int nq = n / 4;                 // c_n = 128: rows are whole quads
        const int lo = (int)((long long)nq * split / ks), hi = (int)((long long)nq * (split + 1) / ks);
        for (int qd = lo + tid; qd < hi; qd += kGemmThreads) {
          const int i = qd * 4;
          const int rr = r_lo + i / c_n, cc = c_lo + i % c_n;
          if (cc >= p.out_cols) continue;
          const int nv = p.out_cols - cc < 4 ? p.out_cols - cc : 4;     // 2 or 4 (out_cols is even)
          const char* src = tile_src + ((size_t)rr * p.out_cols + cc) * 8;
          float acc[4] = {0.f, 0.f, 0.f, 0.f};
          for (int s0 = 0; s0 < nslots; s0 += 4) {
            unsigned long long v[4][4];
            const bool ok = spin_until(
                [&] {
                  bool all = true;
#pragma unroll
                  for (int k = 0; k < 4; ++k)
                    if (s0 + k < nslots) {
                      const char* q = src + (size_t)(s0 + k) * mn * 8;
                      ld_relaxed_sys_u64x2(q, v[k][0], v[k][1]);
                      if (nv == 4) ld_relaxed_sys_u64x2(q + 16, v[k][2], v[k][3]);
#pragma unroll
                      for (int e = 0; e < 4; ++e)
                        if (e < nv) all = all && (uint32_t)(v[k][e] >> 32) == p.ll_tag;
                    }
                  return all;
                },
                p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 52, 0, blockIdx.x));
            if (!ok) return;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              if (s0 + k < nslots) {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  if (e < nv) acc[e] += __uint_as_float((uint32_t)v[k][e]);
              }
          }
          float* o = (float*)p.out + (size_t)rr * p.ldo + cc;
          if (nv == 4 && (((uintptr_t)o) & 15) == 0) {
            *(float4*)o = make_float4(acc[0], acc[1], acc[2], acc[3]);
          } else {
            for (int e = 0; e < nv; ++e) o[e] = acc[e];
          }
        }
        continue;
      }
      const int lo = (int)((long long)n * split / ks), hi = (int)((long long)n * (split + 1) / ks);
      for (int i = lo + tid; i < hi; i += kGemmThreads) {
        const int rr = r_lo + i / c_n, cc = c_lo + i % c_n;
        if (cc >= p.out_cols) continue;
        const char* src = mine + ((size_t)rr * p.out_cols + cc) * 8;
        float acc = 0.f;
        for (int s0 = 0; s0 < nslots; s0 += 8) {
          unsigned long long v[8];
          const bool ok = spin_until(
              [&] {
                bool all = true;
#pragma unroll
                for (int k = 0; k < 8; ++k)
                  if (s0 + k < nslots) {
                    v[k] = ld_relaxed_sys_u64(src + (size_t)(s0 + k) * mn * 8);
                    all = all && (uint32_t)(v[k] >> 32) == p.ll_tag;
                  }
                return all;
              },
              p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 52, 0, blockIdx.x));
          if (!ok) return;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (s0 + k < nslots) acc += __uint_as_float((uint32_t)v[k]);
        }
        ((float*)p.out)[(size_t)rr * p.ldo + cc] = acc;
      }
    }
  }
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
    if (TAGGED && p.ar_algo >= 2) return true;   // tagged forms: nothing to signal, the sums happen in helper_role
    const int tile = tile_of(p, tr, tc);
    const int tid = q * 32 + lane;   // 0..127 over the epilogue warps
    const int ks = nsplit(p), nslots = p.ws * ks;
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
    if (k_split != 0) return true;   // split-K: the CTA of split 0 reduces (owner) or copies out (others)
    if (owner == p.rank) {
      if (tid == 0) wait_count(p.pads[p.rank] + p.flag_base + tile, (uint32_t)nslots, p, 58);
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
          for (int s0 = 0; s0 < nslots; s0 += 8) {
#pragma unroll
            for (int s = 0; s < 8; ++s)
              if (s0 + s < nslots) x[s] = ld16(part + (size_t)(s0 + s) * mn4 + off);
#pragma unroll
            for (int s = 0; s < 8; ++s)
              if (s0 + s < nslots) {
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
            for (int s = 0; s < nslots; ++s) acc += ((const float*)(part + (size_t)s * mn4 + off))[e];
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
