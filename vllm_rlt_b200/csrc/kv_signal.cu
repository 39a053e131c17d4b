// Completion flags between the prefill GPU and the decode GPU.
//
// The reference learns that a chunk has landed from the notification NIXL
// delivers with each WRITE (vllm_rlt/pd/transport.py:186-195, :222-229). Here
// the sender issues a release store on the stream that carried the copy, and
// the receiver either polls the word from the host or runs the bounded wait
// below ahead of the work that consumes the KV.
//
// The wait never spins without a limit: it watches %globaltimer and gives up
// after the caller's timeout, recording what it last saw.

#include <cstring>

#include "common.cuh"

namespace rlt {
namespace {

__global__ void signal_kernel(unsigned long long* flag, unsigned long long value) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(value) : "memory");
  }
}

struct PostBody {
  unsigned long long words[7];
};

__global__ void post_kernel(unsigned long long* slot, const PostBody body, unsigned long long stamp) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
#pragma unroll
    for (int i = 0; i < 7; ++i) slot[1 + i] = body.words[i];
    __threadfence_system();
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(slot), "l"(stamp) : "memory");
  }
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void wait_kernel(const unsigned long long* flag, unsigned long long value, long long timeout_ns,
                            int* status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const unsigned long long start = global_timer_ns();
  unsigned long long seen = 0;
  // Two limits: elapsed time, and an iteration cap in case the timer does not advance.
  for (long long spin = 0; spin < (1ll << 34); ++spin) {
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(flag) : "memory");
    if (seen >= value) return;
    if (global_timer_ns() - start > static_cast<unsigned long long>(timeout_ns)) break;
    __nanosleep(200);
  }
  report(status, RLT_STATUS_TIMEOUT, static_cast<int>(seen & 0xffffffffull), 0, 0);
}

}  // namespace
}  // namespace rlt

extern "C" {

int rlt_kv_signal(uint64_t* flag, uint64_t value, rlt_stream_t stream) {
  if (flag == nullptr) return RLT_E_INVALID;
  if (reinterpret_cast<uintptr_t>(flag) & 7u) return RLT_E_ALIGN;
  rlt::signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<unsigned long long*>(flag), value);
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

int rlt_kv_post(void* slot, const uint8_t body[56], uint64_t stamp, rlt_stream_t stream) {
  if (slot == nullptr || body == nullptr) return RLT_E_INVALID;
  if (reinterpret_cast<uintptr_t>(slot) & 15u) return RLT_E_ALIGN;
  rlt::PostBody b;
  std::memcpy(b.words, body, sizeof(b.words));
  rlt::post_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<unsigned long long*>(slot), b, stamp);
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

int rlt_kv_wait(const uint64_t* flag, uint64_t value, int64_t timeout_ns, int32_t* status, rlt_stream_t stream) {
  if (flag == nullptr || status == nullptr) return RLT_E_INVALID;
  if (reinterpret_cast<uintptr_t>(flag) & 7u) return RLT_E_ALIGN;
  if (timeout_ns < 1 || timeout_ns > RLT_MAX_WAIT_NS) return RLT_E_LIMIT;
  rlt::wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const unsigned long long*>(flag), value, timeout_ns, status);
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // extern "C"
