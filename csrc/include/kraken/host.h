// Host-side runtime shared by every launcher in the library: error reporting, the per-device
// status word that bounded device waits write to, and "rank emulation" — a way to run the
// multi-rank code of a kernel on ONE GPU by launching all ranks as one cooperative grid
// (blockIdx.y = rank), because separate launches that spin on one another must never share a GPU.
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>
#include <cuda_runtime.h>
#include "kraken/ptx_sync.cuh"

#define KR_API extern "C" __attribute__((visibility("default")))

namespace kraken {

// Return codes of the C API.
enum : int { KR_SUCCESS = 0, KR_FAIL_CUDA = 1, KR_FAIL_ARG = 2, KR_FAIL_UNSUPPORTED = 3, KR_FAIL_STATE = 4 };

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define KR_CUDA(expr)                                              \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) return ::kraken::cuda_fail(_e, #expr);  \
  } while (0)

#define KR_REQUIRE(cond, msg)                                                     \
  do {                                                                            \
    if (!(cond)) return ::kraken::fail(::kraken::KR_FAIL_ARG, std::string(msg)); \
  } while (0)

struct DeviceState {
  int device = -1;
  int num_sms = 0;
  uint32_t* status = nullptr;   // 4 words of device memory, zeroed
  uint64_t timeout_ns = 0;
  void* emu_params = nullptr;   // device scratch holding the emulated ranks' parameter blocks
  size_t emu_params_bytes = 0;
};

// State of the CURRENT device (created on first use). Returns nullptr after setting the error.
DeviceState* device_state();
// Deadline of device-side waits on the current device; never allocates.
uint64_t current_timeout_ns();
inline SyncCtx sync_ctx(const DeviceState* d) { return SyncCtx{d->status, d->timeout_ns}; }

// ---- rank emulation ---------------------------------------------------------------------------
struct EmuRecorder {
  bool active = false;
  int ws = 0;
  const void* emu_kernel = nullptr;
  size_t param_size = 0;
  unsigned nblocks = 0, nthreads = 0;
  size_t smem = 0;
  std::vector<unsigned char> params;
  int count = 0;
};
EmuRecorder& emu_recorder();
int emu_record(const void* emu_kernel, const void* p, size_t psize, unsigned nblocks, unsigned nthreads,
               size_t smem);

// Raises the kernel's dynamic shared-memory limit once per (device, kernel).
int ensure_dynamic_smem(const void* func, size_t smem);

// Launches `real` with the parameter block by value, or — while an emulation is being recorded —
// stores the block so that kr_emu_end() can launch `emu` once for all ranks.
template <class P>
int launch_ranked(void (*real)(P), void (*emu)(const P*), const P& p, unsigned nblocks, unsigned nthreads,
                  size_t smem, cudaStream_t stream) {
  if (emu_recorder().active)
    return emu_record((const void*)emu, &p, sizeof(P), nblocks, nthreads, smem);
  if (smem > 48 * 1024) {
    int rc = ensure_dynamic_smem((const void*)real, smem);
    if (rc) return rc;
  }
  void* args[] = {(void*)&p};
  KR_CUDA(cudaLaunchKernel((const void*)real, dim3(nblocks), dim3(nthreads), args, smem, stream));
  return KR_SUCCESS;
}

// Defines NAME_kernel(Params) and NAME_emu_kernel(const Params*) around
//   __device__ void NAME_body(const Params& p, unsigned block_id, unsigned num_blocks);
#define KR_DEFINE_RANKED_KERNEL(NAME, PARAMS, THREADS)                                         \
  __global__ void __launch_bounds__(THREADS) NAME##_kernel(const __grid_constant__ PARAMS p) { \
    NAME##_body(p, blockIdx.x, gridDim.x);                                                     \
  }                                                                                            \
  __global__ void __launch_bounds__(THREADS) NAME##_emu_kernel(const PARAMS* ps) {             \
    NAME##_body(ps[blockIdx.y], blockIdx.x, gridDim.x);                                        \
  }

inline unsigned cdiv(size_t a, size_t b) { return (unsigned)((a + b - 1) / b); }

}  // namespace kraken
