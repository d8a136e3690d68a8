// A user-written kernel on top of the library's device primitives (what the reference's README
// shows with a Triton kernel and symm_mem_sync, README.md:77-129): every rank adds the values of
// ALL ranks' symmetric buffers into its own output, with the per-block cross-device barrier
// before (peers' data is ready) and after (peers may overwrite their buffers again).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -std=c++17 -O3 -shared -Xcompiler -fPIC \
//        -I csrc/include examples/custom_kernel.cu -o examples/libcustom_kernel.so
#include <cuda_bf16.h>
#include "kraken/ptx_sync.cuh"

using namespace kraken;

__global__ void sum_peers_kernel(float* const* bufs, uint32_t* const* pads, float* out, size_t n, int rank, int ws,
                                 uint32_t* status, unsigned long long timeout_ns) {
  const SyncCtx sync{status, timeout_ns};
  // pattern (previous=false, subsequent=true): peers' earlier writes are visible after this
  if (!symm_mem_sync<false, true>(pads, blockIdx.x, rank, ws, sync)) return;   // a peer never came: give up cleanly
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < ws; ++r) acc += bufs[r][i];     // plain loads from peer memory over NVLink
    out[i] = acc;
  }
  // pattern (previous=true, subsequent=false): nobody overwrites a buffer that is still being read
  symm_mem_sync<true, false>(pads, blockIdx.x, rank, ws, sync);
}

extern "C" int launch_sum_peers(float* const* bufs, uint32_t* const* pads, float* out, size_t n, int rank, int ws,
                                uint32_t* status, double timeout_ms, cudaStream_t stream) {
  // identical grid on every rank (the barrier pairs blocks by index) and no larger than the SM count
  sum_peers_kernel<<<32, 256, 0, stream>>>(bufs, pads, out, n, rank, ws, status, (unsigned long long)(timeout_ms * 1e6));
  return (int)cudaGetLastError();
}
