// Host runtime: error strings, per-device status word, wait deadline, rank emulation.
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <map>
#include "kraken/host.h"

namespace kraken {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
int cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return KR_FAIL_CUDA;
}

static std::mutex g_mu;
static std::map<int, DeviceState*> g_states;
static uint64_t g_default_timeout_ns = 0;

static uint64_t default_timeout_ns() {
  if (g_default_timeout_ns == 0) {
    const char* e = getenv("KRAKEN_SYNC_TIMEOUT_MS");
    double ms = e ? atof(e) : 4000.0;
    if (ms <= 0) ms = 4000.0;
    g_default_timeout_ns = (uint64_t)(ms * 1e6);
  }
  return g_default_timeout_ns;
}

DeviceState* device_state() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaGetDevice");
    return nullptr;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_states.find(dev);
  if (it != g_states.end()) return it->second;
  auto* d = new DeviceState();
  d->device = dev;
  e = cudaDeviceGetAttribute(&d->num_sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess) e = cudaMalloc(&d->status, 4 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(d->status, 0, 4 * sizeof(uint32_t));
  if (e != cudaSuccess) {
    cuda_fail(e, "device_state init");
    delete d;
    return nullptr;
  }
  d->timeout_ns = default_timeout_ns();
  g_states[dev] = d;
  return d;
}

// Wait deadline that applies on the current device, found without creating (allocating) its state.
uint64_t current_timeout_ns() {
  int dev = -1;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_states.find(dev);
    if (it != g_states.end()) return it->second->timeout_ns;
  }
  return default_timeout_ns();
}

int ensure_dynamic_smem(const void* func, size_t smem) {
  static std::map<std::pair<int, const void*>, size_t> done;
  int dev = 0;
  KR_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(g_mu);
  auto key = std::make_pair(dev, func);
  auto it = done.find(key);
  if (it != done.end() && it->second >= smem) return KR_SUCCESS;
  KR_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  done[key] = smem;
  return KR_SUCCESS;
}

EmuRecorder& emu_recorder() {
  static thread_local EmuRecorder r;
  return r;
}

int emu_record(const void* emu_kernel, const void* p, size_t psize, unsigned nblocks, unsigned nthreads,
               size_t smem) {
  EmuRecorder& r = emu_recorder();
  if (r.count == 0) {
    r.emu_kernel = emu_kernel;
    r.param_size = psize;
    r.nblocks = nblocks;
    r.nthreads = nthreads;
    r.smem = smem;
  } else if (r.emu_kernel != emu_kernel || r.param_size != psize || r.nblocks != nblocks ||
             r.nthreads != nthreads || r.smem != smem) {
    return fail(KR_FAIL_STATE, "rank emulation: ranks recorded different kernels or launch shapes");
  }
  if (r.count >= r.ws) return fail(KR_FAIL_STATE, "rank emulation: more launches than ranks");
  const unsigned char* b = (const unsigned char*)p;
  r.params.insert(r.params.end(), b, b + psize);
  r.count++;
  return KR_SUCCESS;
}

}  // namespace kraken

using namespace kraken;

KR_API const char* kr_last_error() { return g_last_error.c_str(); }

// 1 when the library was compiled with the device-side bounds checks (-DKRAKEN_DEBUG=1).
KR_API int kr_is_debug_build() {
#ifdef KRAKEN_DEBUG
  return 1;
#else
  return 0;
#endif
}

KR_API int kr_num_sms() {
  DeviceState* d = device_state();
  return d ? d->num_sms : -1;
}

// Sets the deadline of every device-side wait on the current device.
KR_API int kr_set_timeout_ms(double ms) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_REQUIRE(ms > 0, "timeout must be positive");
  d->timeout_ns = (uint64_t)(ms * 1e6);
  return KR_SUCCESS;
}
KR_API double kr_get_timeout_ms() {
  DeviceState* d = device_state();
  return d ? d->timeout_ns / 1e6 : -1.0;
}

KR_API void* kr_status_ptr() {
  DeviceState* d = device_state();
  return d ? (void*)d->status : nullptr;
}

// Reads the status word of the current device after synchronising `stream` (blocking).
KR_API int kr_read_status(cudaStream_t stream, uint32_t* out) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_CUDA(cudaStreamSynchronize(stream));
  KR_CUDA(cudaMemcpy(out, d->status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  return KR_SUCCESS;
}
KR_API int kr_clear_status(cudaStream_t stream) {
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  KR_CUDA(cudaMemsetAsync(d->status, 0, 4 * sizeof(uint32_t), stream));
  return KR_SUCCESS;
}

// ---- rank emulation: kr_emu_begin(ws); <launcher for rank 0> ... <launcher for rank ws-1>;
//      kr_emu_end(stream) launches the recorded kernel once with gridDim.y = ws, cooperatively,
//      so that all ranks' blocks are resident together.
KR_API int kr_emu_begin(int ws) {
  EmuRecorder& r = emu_recorder();
  KR_REQUIRE(!r.active, "rank emulation already active");
  KR_REQUIRE(ws >= 1 && ws <= 72, "bad emulated world size");
  r = EmuRecorder();
  r.active = true;
  r.ws = ws;
  return KR_SUCCESS;
}
KR_API int kr_emu_abort() {
  emu_recorder() = EmuRecorder();
  return KR_SUCCESS;
}
KR_API int kr_emu_end(cudaStream_t stream) {
  EmuRecorder& r = emu_recorder();
  KR_REQUIRE(r.active, "rank emulation not active");
  EmuRecorder rec = r;
  r = EmuRecorder();
  if (rec.count != rec.ws) return fail(KR_FAIL_STATE, "rank emulation: fewer launches than ranks");
  DeviceState* d = device_state();
  if (!d) return KR_FAIL_CUDA;
  if (rec.smem > 48 * 1024) {
    int rc = ensure_dynamic_smem(rec.emu_kernel, rec.smem);
    if (rc) return rc;
  }
  int per_sm = 0;
  KR_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, rec.emu_kernel, (int)rec.nthreads, rec.smem));
  if ((size_t)rec.nblocks * rec.ws > (size_t)per_sm * d->num_sms)
    return fail(KR_FAIL_ARG, "rank emulation: grid does not fit on the device at once");
  if (d->emu_params_bytes < rec.params.size()) {
    if (d->emu_params) KR_CUDA(cudaFree(d->emu_params));
    d->emu_params = nullptr;
    KR_CUDA(cudaMalloc(&d->emu_params, rec.params.size()));
    d->emu_params_bytes = rec.params.size();
  }
  KR_CUDA(cudaStreamSynchronize(stream));  // earlier emulated launches may still read the scratch
  KR_CUDA(cudaMemcpy(d->emu_params, rec.params.data(), rec.params.size(), cudaMemcpyHostToDevice));
  void* arg0 = d->emu_params;
  void* args[] = {&arg0};
  KR_CUDA(cudaLaunchCooperativeKernel(rec.emu_kernel, dim3(rec.nblocks, rec.ws), dim3(rec.nthreads), args,
                                      rec.smem, stream));
  return KR_SUCCESS;
}
