// Shared host/device helpers of the KV-handoff kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <nvtx3/nvToolsExt.h>

#include <atomic>

#include "rlt_kv_handoff.h"

namespace rlt {

constexpr int kThreads = 256;      // threads per CTA of every copy kernel
constexpr int kMaxRows = 256;      // token rows one work unit may hold
constexpr int kMaxBlockSize = 64;  // tokens per KV block

extern thread_local int g_last_cuda_error;
extern std::atomic<long long> g_launches;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return RLT_E_CUDA;
}

#define RLT_CUDA_TRY(expr)                          \
  do {                                              \
    cudaError_t rlt_err__ = (expr);                 \
    if (rlt_err__ != cudaSuccess) return ::rlt::cuda_fail(rlt_err__); \
  } while (0)

// Names the launches of one entry point for profilers (the reference's NIXL traffic is invisible to its
// torch profiler sessions; these launches are ordinary kernels and show up under these ranges).
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

// SM count of the current device, looked up once per device.
int sm_count(int* out);

// First error wins: later reports leave the status words alone.
__device__ __forceinline__ void report(int32_t* status, int code, int a, int b, int c) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = a;
    status[2] = b;
    status[3] = c;
  }
}

// Streaming 16-byte accesses: the payload is touched once, keep it out of L1.
__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4* p, uint4 v) { __stcs(p, v); }
// 32-byte accesses (256-bit global loads and stores exist from sm_100 on).
struct alignas(32) Vec32 {
  uint32_t v[8];
};
__device__ __forceinline__ Vec32 ld_stream(const Vec32* p) {
  Vec32 r;
  asm volatile("ld.global.L1::no_allocate.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                 "=r"(r.v[7])
               : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream(Vec32* p, const Vec32& r) {
  asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(r.v[0]), "r"(r.v[1]),
               "r"(r.v[2]), "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7])
               : "memory");
}
__device__ __forceinline__ uint32_t ld_stream(const uint32_t* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint32_t* p, uint32_t v) { __stcs(p, v); }
__device__ __forceinline__ uint8_t ld_stream(const uint8_t* p) { return *p; }
__device__ __forceinline__ void st_stream(uint8_t* p, uint8_t v) { *p = v; }

// Inclusive prefix sum across the 32 lanes of a warp.
__device__ __forceinline__ int warp_inclusive_scan(int v) {
  const unsigned lane = threadIdx.x & 31u;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, v, d);
    if (lane >= static_cast<unsigned>(d)) v += n;
  }
  return v;
}

// Multiplier m with floor(i / d) == __umulhi(i, m) whenever i * d < 2^32.
inline uint32_t div_magic(uint32_t d) { return static_cast<uint32_t>((1ull << 32) / d) + 1u; }

}  // namespace rlt
