// Lazily resolved CUDA driver entry points. The library does not link libcuda: it asks the
// runtime for each symbol on first use, so the shared object also loads on machines without a
// driver (build checks, CPU-only tests).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <string>
#include "kraken/host.h"

namespace kraken {

void* driver_entry(const char* name);   // nullptr (and error set) when unavailable
std::string cu_error_string(CUresult r);

#define KR_DRV_FN(name) ((decltype(&name))::kraken::driver_entry(#name))

#define KR_CU(call_name, ...)                                                                      \
  do {                                                                                             \
    auto _fn = KR_DRV_FN(call_name);                                                               \
    if (!_fn) return ::kraken::fail(::kraken::KR_FAIL_UNSUPPORTED, std::string(#call_name) + " not available"); \
    CUresult _r = _fn(__VA_ARGS__);                                                                \
    if (_r != CUDA_SUCCESS)                                                                        \
      return ::kraken::fail(::kraken::KR_FAIL_CUDA, std::string(#call_name) + ": " + ::kraken::cu_error_string(_r)); \
  } while (0)

}  // namespace kraken
