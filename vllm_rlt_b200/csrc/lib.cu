// Library-wide state and the information entry points.
#include "common.cuh"

namespace rlt {

thread_local int g_last_cuda_error = 0;
std::atomic<long long> g_launches{0};

int sm_count(int* out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<int> cached[kMaxDevices];
  int device = 0;
  RLT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return RLT_E_LIMIT;
  int n = cached[device].load(std::memory_order_relaxed);
  if (n == 0) {
    RLT_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device));
    cached[device].store(n, std::memory_order_relaxed);
  }
  *out = n;
  return RLT_OK;
}

}  // namespace rlt

extern "C" {

int rlt_version(void) { return 1; }

const char* rlt_error_string(int code) {
  switch (code) {
    case RLT_OK: return "ok";
    case RLT_E_INVALID: return "invalid argument";
    case RLT_E_GEOMETRY: return "pool geometry is not dense or differs between source and destination";
    case RLT_E_LIMIT: return "size limit of the entry point exceeded";
    case RLT_E_CUDA: return "CUDA runtime call failed";
    case RLT_E_ALIGN: return "pointer or size is not aligned as the entry point requires";
    default: return "unknown error";
  }
}

int rlt_last_cuda_error(void) { return rlt::g_last_cuda_error; }

int64_t rlt_kernel_launches(void) { return rlt::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
