// Push-style one-shot all-reduce for small messages, optionally fused with a bias add and with
// bias + RMSNorm (the tensor-parallel decode epilogue).
//
// The pull form (comm.cu / norm.cu; reference: kraken/comm/one_shot_all_reduce.py:17-54,
// kraken/fused/one_shot_all_reduce_bias_rms_norm.py:23-99) costs a copy-in, a barrier, a round of
// remote loads and an exit barrier. Here every rank WRITES its data straight into slot [rank] of
// every peer's workspace (posted NVLink stores, or one multimem.st through the NVSwitch), meets its
// peers in ONE barrier, and then sums the ws slots out of its own memory. The workspace has two
// halves used alternately call by call, so a fast rank's next call never overwrites what a slow
// rank still reads and no exit barrier is needed: a rank can only be one call ahead, because
// finishing a call takes a signal from every peer sent in that same call.
// The peers' buffer and signal-pad addresses travel in the kernel parameters (world sizes up to
// 8), which saves two dependent global loads at the start of a latency-bound kernel.
#include "kraken/host.h"
#include "kraken/norm_core.cuh"

namespace kraken {

constexpr int kPushMaxWs = 8;
constexpr int kPushThreads = 512;

struct PushParams {
  void* bufs[kPushMaxWs];        // every rank's workspace
  uint32_t* pads[kPushMaxWs];    // every rank's signal pad
  void* mc_ptr;                  // multicast address of the workspace, or nullptr
  const void* input;             // this rank's data (any device memory)
  void* output;
  const void* bias;              // optional
  const void* w;                 // RMSNorm weight (norm kernel)
  unsigned long long numel;      // elements (all-reduce kernel)
  unsigned long long bias_period;
  unsigned long long half_off;   // byte offset of this call's workspace half
  unsigned long long slot_bytes; // bytes reserved per source rank inside a half
  uint32_t tag;                  // != 0: tagged form (no barrier): every 4 bytes of data travel with this tag
  int rows, D;                   // norm kernel
  float eps;
  int rank, ws;
  uint32_t pad_base;
  SyncCtx sync;
};

__device__ __forceinline__ char* slot_of(const PushParams& p, int dst, int src) {
  return (char*)p.bufs[dst] + p.half_off + (size_t)src * p.slot_bytes;
}

// Writes one 16-byte vector of this rank's data into slot [rank] of every peer.
__device__ __forceinline__ void push_vec(const PushParams& p, size_t byte_off, const U4& x) {
  if (!kr_in_bounds(byte_off + 16 <= p.slot_bytes, p.sync, 73)) return;
  if (p.mc_ptr != nullptr) {
    multimem_st16((char*)p.mc_ptr + p.half_off + (size_t)p.rank * p.slot_bytes + byte_off, x);
  } else {
#pragma unroll
    for (int s = 1; s < kPushMaxWs; ++s)
      if (s < p.ws) {
        int peer = p.rank + s;
        if (peer >= p.ws) peer -= p.ws;
        st16(slot_of(p, peer, p.rank) + byte_off, x);
      }
  }
}

// Sum over ranks (rank order) of one vector: the own contribution is still in registers.
__device__ __forceinline__ void gather_vec(const PushParams& p, size_t byte_off, const U4& own, float (&f)[8]) {
  U4 x[kPushMaxWs];
#pragma unroll
  for (int s = 0; s < kPushMaxWs; ++s)
    if (s < p.ws && s != p.rank) x[s] = ld16(slot_of(p, p.rank, s) + byte_off);
#pragma unroll
  for (int s = 0; s < kPushMaxWs; ++s)
    if (s < p.ws) acc8(s == p.rank ? own : x[s], f);
}

// ---- tagged form ------------------------------------------------------------------------------
// For the smallest messages even the one barrier is most of the time: its release (a system-scope
// fence behind the data stores) and the flag's own NVLink crossing. The tagged form sends no flag:
// every 4 bytes of data (two bf16) travel with the call's tag in ONE 8-byte store, which a peer sees
// whole or not at all, into a region that only tagged calls ever write (so no stale word can carry
// the tag: tags are call numbers, the region alternates with the call's parity and starts out
// zero). The receiver polls the pairs of its own slots until they carry the tag. Twice the bytes,
// no fence, no flag.
__device__ __forceinline__ void push_vec_tagged(const PushParams& p, size_t byte_off, const U4& x) {
  if (!kr_in_bounds(2 * byte_off + 32 <= p.slot_bytes, p.sync, 74)) return;
  const unsigned long long t = (unsigned long long)p.tag << 32;
  const unsigned long long w0 = t | x.x, w1 = t | x.y, w2 = t | x.z, w3 = t | x.w;
  if (p.mc_ptr != nullptr) {
    char* d = (char*)p.mc_ptr + p.half_off + (size_t)p.rank * p.slot_bytes + 2 * byte_off;
    multimem_st_u64(d, w0); multimem_st_u64(d + 8, w1); multimem_st_u64(d + 16, w2); multimem_st_u64(d + 24, w3);
  } else {
#pragma unroll
    for (int s = 1; s < kPushMaxWs; ++s)
      if (s < p.ws) {
        int peer = p.rank + s;
        if (peer >= p.ws) peer -= p.ws;
        char* d = slot_of(p, peer, p.rank) + 2 * byte_off;
        st_relaxed_sys_u64(d, w0); st_relaxed_sys_u64(d + 8, w1);
        st_relaxed_sys_u64(d + 16, w2); st_relaxed_sys_u64(d + 24, w3);
      }
  }
}

// Sum over ranks (rank order) of one vector whose peers' copies arrive tagged; up to four slots
// (eight 16-byte loads) are polled together. False when a wait gave up.
__device__ __forceinline__ bool gather_vec_tagged(const PushParams& p, size_t byte_off, const U4& own, float (&f)[8]) {
  for (int s0 = 0; s0 < p.ws; s0 += 4) {
    unsigned long long v[4][4];
    const bool ok = spin_until(
        [&] {
          bool all = true;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int s = s0 + k;
            if (s < p.ws && s != p.rank) {
              const char* q = slot_of(p, p.rank, s) + 2 * byte_off;
              ld_relaxed_sys_u64x2(q, v[k][0], v[k][1]);
              ld_relaxed_sys_u64x2(q + 16, v[k][2], v[k][3]);
#pragma unroll
              for (int e = 0; e < 4; ++e) all = all && (uint32_t)(v[k][e] >> 32) == p.tag;
            }
          }
          return all;
        },
        p.sync, make_status(KR_ERR_TIMEOUT_SIGNAL, 62, 0, blockIdx.x));
    if (!ok) return false;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int s = s0 + k;
      if (s < p.ws) {
        if (s == p.rank) acc8(own, f);
        else acc8(U4{(uint32_t)v[k][0], (uint32_t)v[k][1], (uint32_t)v[k][2], (uint32_t)v[k][3]}, f);
      }
    }
  }
  return true;
}

// ---- all-reduce (+bias) ---------------------------------------------------------------------
// Block b handles vectors b*T + t, (b + nb)*T + t, ... in both phases on every rank, so the
// per-block barrier is all the ordering the slots need.
__device__ void push_ar_body(const PushParams& p, unsigned bid, unsigned nb) {
  const size_t nvec = p.numel / 8;
  const size_t stride = (size_t)nb * blockDim.x;
  const size_t first = (size_t)bid * blockDim.x + threadIdx.x;
  if (p.tag != 0) {
    for (size_t v = first; v < nvec; v += stride) push_vec_tagged(p, v * 16, ld16((const char*)p.input + v * 16));
  } else {
    for (size_t v = first; v < nvec; v += stride) push_vec(p, v * 16, ld16((const char*)p.input + v * 16));
    if (!symm_mem_sync<true, true>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 60)) return;
  }
  for (size_t v = first; v < nvec; v += stride) {
    float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (p.bias) acc8(ld16_nc((const char*)p.bias + ((v * 8) % p.bias_period) * 2), f);
    if (p.tag != 0) {
      if (!gather_vec_tagged(p, v * 16, ld16((const char*)p.input + v * 16), f)) return;
    } else {
      gather_vec(p, v * 16, ld16((const char*)p.input + v * 16), f);
    }
    st16((char*)p.output + v * 16, pack8(f));
  }
}
KR_DEFINE_RANKED_KERNEL(push_ar, PushParams, kPushThreads)

// ---- all-reduce + bias + RMSNorm --------------------------------------------------------------
// One block per row (row r -> block r % nb on every rank); a thread keeps VPT vectors of the row
// in registers from the push to the normalisation (1 for rows of up to 8192 elements: no spills, all
// ws slot loads of the vector in flight together).
template <int VPT, bool TAGGED>
__device__ __forceinline__ void push_ar_norm_impl(const PushParams& p, unsigned bid, unsigned nb) {
  __shared__ float smem[32];
  const int nvec = p.D / 8;
  // phase 1: all rows of this block go out before the barrier
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const size_t bo = off + (size_t)v * 16;
      if (TAGGED) push_vec_tagged(p, bo, ld16((const char*)p.input + bo));
      else push_vec(p, bo, ld16((const char*)p.input + bo));
    }
  }
  if (!TAGGED && !symm_mem_sync<true, true>(p.pads, p.pad_base / p.ws + bid, p.rank, p.ws, p.sync, 61)) return;
  bool alive = true;
  for (int r = bid; r < p.rows; r += nb) {
    const size_t off = (size_t)r * p.D * 2;
    float f[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        const size_t bo = off + (size_t)v * 16;
#pragma unroll
        for (int j = 0; j < 8; ++j) f[i][j] = 0.f;
        if (p.bias) acc8(ld16_nc((const char*)p.bias + (((size_t)r * p.D + (size_t)v * 8) % p.bias_period) * 2), f[i]);
        if (TAGGED) alive = gather_vec_tagged(p, bo, ld16((const char*)p.input + bo), f[i]) && alive;
        else gather_vec(p, bo, ld16((const char*)p.input + bo), f[i]);
      }
    }
    if (TAGGED && __syncthreads_or(alive ? 0 : 1)) return;      // a wait gave up somewhere in the block: leave together
    rms_finish<VPT>(f, nvec, p.D, p.eps, (const char*)p.w, (char*)p.output + off, smem);
  }
}
__device__ void push_ar_norm_body(const PushParams& p, unsigned bid, unsigned nb) { push_ar_norm_impl<1, false>(p, bid, nb); }
__device__ void push_ar_norm_long_body(const PushParams& p, unsigned bid, unsigned nb) { push_ar_norm_impl<kNormVpt, false>(p, bid, nb); }
// tagged form: at most 512 threads (the polled pairs of four slots need registers), two vectors each
constexpr int kTaggedNormThreads = 512;
constexpr int kTaggedNormVpt = 2;
__device__ void push_ar_norm_tagged_body(const PushParams& p, unsigned bid, unsigned nb) { push_ar_norm_impl<kTaggedNormVpt, true>(p, bid, nb); }
KR_DEFINE_RANKED_KERNEL(push_ar_norm_long, PushParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(push_ar_norm, PushParams, kNormMaxThreads)
KR_DEFINE_RANKED_KERNEL(push_ar_norm_tagged, PushParams, kTaggedNormThreads)

}  // namespace kraken

using namespace kraken;

static int fill_push(PushParams& p, DeviceState* d, void* const* bufs_host, uint32_t* const* pads_host, void* mc_ptr,
                     int rank, int ws, const void* input, void* output, const void* bias,
                     unsigned long long bias_numel, unsigned long long bytes, unsigned call_seq,
                     unsigned long long tagged_max_bytes, unsigned long long workspace_bytes, uint32_t pad_base) {
  KR_REQUIRE(ws >= 1 && ws <= kPushMaxWs && rank >= 0 && rank < ws, "push all-reduce supports world sizes up to 8");
  KR_REQUIRE(bufs_host != nullptr && pads_host != nullptr, "null argument");
  KR_REQUIRE(pad_base % ws == 0, "pad_base must be a multiple of the world size");
  KR_REQUIRE((((uintptr_t)input | (uintptr_t)output | (uintptr_t)bias) & 15) == 0, "tensors must be 16-byte aligned");
  if (bias) KR_REQUIRE(bias_numel > 0 && bias_numel % 8 == 0, "bias length must be a positive multiple of 8");
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < ws; ++r) {
    p.bufs[r] = bufs_host[r];
    p.pads[r] = pads_host[r];
  }
  // Workspace quarters: [0] flag form, even calls | [1] flag form, odd | [2] tagged form, even |
  // [3] tagged, odd; each cut into ws slots. The tagged quarters are written by tagged calls only.
  const unsigned long long half = workspace_bytes / 4 / 1024 * 1024;
  const unsigned long long slot = half / ws / 1024 * 1024;
  KR_REQUIRE(slot >= bytes && slot > 0, "push workspace too small for this message");
  const bool tagged = bytes <= tagged_max_bytes && slot >= 2 * bytes;
  p.mc_ptr = mc_ptr;
  p.input = input;
  p.output = output;
  p.bias = bias;
  p.bias_period = bias ? bias_numel : 8;
  p.half_off = ((call_seq & 1u) ? half : 0) + (tagged ? 2 * half : 0);
  p.slot_bytes = slot;
  p.tag = tagged ? call_seq % 0x7fffffffu + 1u : 0u;     // call numbers: never 0, never what the region saw last
  p.rank = rank;
  p.ws = ws;
  p.pad_base = pad_base;
  p.sync = sync_ctx(d);
  return KR_SUCCESS;
}

static unsigned push_grid_cap(const DeviceState* d) {
  unsigned cap = (unsigned)d->num_sms;
  if (emu_recorder().active) {
    cap /= (unsigned)emu_recorder().ws;
    if (cap < 1) cap = 1;
  }
  return cap;
}

// output = bias + sum_r input_r. bufs_host / pads_host: HOST arrays [ws] with every rank's
// workspace and signal-pad address; workspace_bytes per rank (all zero before its first use),
// in quarters that alternate with the parity of call_seq (the number of calls made on this
// workspace so far, the same on every rank), each cut into ws slots that must hold numel * 2 bytes.
// Messages of up to tagged_max_bytes (and half a slot) take the tagged form. numel % 8 == 0.
KR_API int kr_push_all_reduce(void* const* bufs_host, uint32_t* const* pads_host, void* mc_ptr, int rank, int ws,
                              const void* input, void* output, const void* bias, unsigned long long bias_numel,
                              unsigned long long numel, unsigned call_seq, unsigned long long tagged_max_bytes,
                              unsigned long long workspace_bytes, uint32_t pad_base, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(numel >= 8 && numel % 8 == 0, "push all-reduce needs numel % 8 == 0");
  PushParams p;
  int rc = fill_push(p, d, bufs_host, pads_host, mc_ptr, rank, ws, input, output, bias, bias_numel, numel * 2,
                     call_seq, tagged_max_bytes, workspace_bytes, pad_base);
  if (rc) return rc;
  p.numel = numel;
  const unsigned long long nvec = numel / 8;
  unsigned nb = cdiv(nvec, (size_t)kPushThreads * 2);
  if (nvec <= (unsigned long long)kPushThreads) nb = 1;
  if (nb > push_grid_cap(d)) nb = push_grid_cap(d);
  return launch_ranked(push_ar_kernel, push_ar_emu_kernel, p, nb, kPushThreads, 0, stream);
}

// y = rms_norm(bias + sum_r x_r) * w over rows of D elements (D % 8 == 0, D / 8 <= 4096).
KR_API int kr_push_all_reduce_bias_rms_norm(void* const* bufs_host, uint32_t* const* pads_host, void* mc_ptr, int rank,
                                            int ws, const void* x, const void* bias, unsigned long long bias_numel,
                                            const void* w, void* y, int rows, int D, float eps, unsigned call_seq,
                                            unsigned long long tagged_max_bytes, unsigned long long workspace_bytes,
                                            uint32_t pad_base, cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(rows >= 1 && D > 0 && D % 8 == 0, "needs D % 8 == 0");
  KR_REQUIRE(D / 8 <= kNormVpt * kNormMaxThreads, "row too long for the fused all-reduce + RMSNorm kernel");
  KR_REQUIRE(((uintptr_t)w & 15) == 0, "tensors must be 16-byte aligned");
  PushParams p;
  int rc = fill_push(p, d, bufs_host, pads_host, mc_ptr, rank, ws, x, y, bias, bias_numel,
                     (unsigned long long)rows * D * 2, call_seq, tagged_max_bytes, workspace_bytes, pad_base);
  if (rc) return rc;
  p.w = w;
  p.rows = rows;
  p.D = D;
  p.eps = eps;
  const unsigned cap = push_grid_cap(d);
  const unsigned nb = (unsigned)rows < cap ? (unsigned)rows : cap;
  if (p.tag != 0) {
    if ((unsigned)D / 8 <= (unsigned)(kTaggedNormThreads * kTaggedNormVpt)) {
      unsigned nt = ((unsigned)D / 8 + 31) / 32 * 32;
      if (nt > (unsigned)kTaggedNormThreads) nt = (((unsigned)D / 8 + kTaggedNormVpt - 1) / kTaggedNormVpt + 31) / 32 * 32;
      if (nt < 64) nt = 64;
      return launch_ranked(push_ar_norm_tagged_kernel, push_ar_norm_tagged_emu_kernel, p, nb, nt, 0, stream);
    }
    // row too long for the tagged kernel: the flag form, in the flag form's quarter
    p.half_off -= 2 * (workspace_bytes / 4 / 1024 * 1024);
    p.tag = 0;
  }
  unsigned nt = ((unsigned)D / 8 + 31) / 32 * 32;      // one vector per thread when the row allows
  if (nt < 64) nt = 64;
  if (nt > kNormMaxThreads) nt = kNormMaxThreads;
  if ((unsigned)D / 8 > nt) return launch_ranked(push_ar_norm_long_kernel, push_ar_norm_long_emu_kernel, p, nb, nt, 0, stream);
  return launch_ranked(push_ar_norm_kernel, push_ar_norm_emu_kernel, p, nb, nt, 0, stream);
}
