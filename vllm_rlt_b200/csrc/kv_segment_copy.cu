// Copies of explicit byte ranges: one range (push) or a device-resident list of
// (source, destination, bytes) triples (copy_segments).
//
// copy_segments performs the WRITE of one NixlConnector.submit call
// (vllm_rlt/pd/transport.py:182-201) for the descriptor lists that
// partition_segments produces (:95-112): up to a few hundred ranges whose sizes
// differ by orders of magnitude (a 1.5 MiB block next to a 4 KiB partial row).
//
// Work split: the ranges are laid end to end, and CTA c of a persistent grid copies
// bytes [c * T / G, (c + 1) * T / G) of that line (cuts rounded to 256 bytes inside a
// range). Every CTA computes the same exclusive scan of the range sizes with
// warp-shuffle prefix sums in shared memory and finds its first range by binary
// search, so every CTA moves the same number of bytes to within 256 whatever the mix
// of range sizes; a split into fixed tiles left up to one tile of difference per CTA,
// which is 7 % of a launch that moves 0.8 GB.
//
// Roofline: one read and one write per byte. Local copies are HBM bound; a
// destination on a peer GPU is bound by NVLink (one direction).

#include "common.cuh"

namespace rlt {
namespace {

constexpr long long kCutBytes = 256;  // shares are cut at multiples of this inside a range: vector alignment survives
constexpr int kUnroll = 4;  // four 16-byte loads in flight per thread and three CTAs per SM measured best on HBM
constexpr int kCtasPerSm = 3;

template <typename T>
__device__ __forceinline__ void stream_range(const char* __restrict__ src, char* __restrict__ dst, long long n) {
  const T* s = reinterpret_cast<const T*>(src);
  T* d = reinterpret_cast<T*>(dst);
  for (long long base = threadIdx.x; base < n; base += kThreads * kUnroll) {
    T regs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = base + u * kThreads;
      if (i < n) regs[u] = ld_stream(s + i);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long i = base + u * kThreads;
      if (i < n) st_stream(d + i, regs[u]);
    }
  }
}

// One piece of one range. Pointers that are both 16-byte aligned take the vector path with a byte tail;
// otherwise the widest element both pointers and the length allow.
__device__ __forceinline__ void copy_piece(const char* src, char* dst, long long n) {
  const unsigned long long both = reinterpret_cast<unsigned long long>(src) | reinterpret_cast<unsigned long long>(dst);
  if ((both & 15ull) == 0) {
    const long long body = n & ~15ll;
    stream_range<uint4>(src, dst, body >> 4);
    if (static_cast<long long>(threadIdx.x) < n - body) dst[body + threadIdx.x] = src[body + threadIdx.x];
  } else if (((both | static_cast<unsigned long long>(n)) & 3ull) == 0) {
    stream_range<uint32_t>(src, dst, n >> 2);
  } else {
    stream_range<uint8_t>(src, dst, n);
  }
}

// Byte position `at` of a line of `total` bytes, moved down to a multiple of kCutBytes (the end of the line stays).
__device__ __forceinline__ long long cut_of(long long total, long long part, long long parts) {
  // total / parts * part + remainder term: no overflow for any int64 total
  const long long at = total / parts * part + total % parts * part / parts;
  return part >= parts ? total : at & ~(kCutBytes - 1);
}

__global__ void __launch_bounds__(kThreads, 3) push_kernel(const char* src, char* dst, long long nbytes) {
  const long long lo = cut_of(nbytes, blockIdx.x, gridDim.x), hi = cut_of(nbytes, blockIdx.x + 1, gridDim.x);
  if (hi > lo) copy_piece(src + lo, dst + lo, hi - lo);
}

__global__ void __launch_bounds__(kThreads, 3) segment_copy_kernel(const long long* __restrict__ segments, int count) {
  extern __shared__ long long seg_start[];  // [count + 1] exclusive scan of the range sizes
  __shared__ long long warp_sum[kThreads / 32];
  __shared__ long long carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    carry = 0;
    seg_start[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < count; base += kThreads) {
    const int s = base + threadIdx.x;
    long long n = 0;
    if (s < count) {
      n = segments[3ll * s + 2];
      if (n < 0) n = 0;
    }
    long long inc = n;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const long long up = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += up;
    }
    if (lane == 31) warp_sum[warp] = inc;
    __syncthreads();
    long long before = carry;
    for (int w = 0; w < warp; ++w) before += warp_sum[w];
    if (s < count) seg_start[s + 1] = before + inc;
    __syncthreads();
    if (threadIdx.x == kThreads - 1) carry = before + inc;
    __syncthreads();
  }
  const long long total = seg_start[count];
  // This CTA's share of the line. A cut is rounded down to a multiple of kCutBytes *inside its range*, so the
  // CTA on either side of it derives the same cut from the same numbers.
  long long share[2];
  int first = 0;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const long long part = static_cast<long long>(blockIdx.x) + k;
    long long at = part >= gridDim.x ? total : total / gridDim.x * part + total % gridDim.x * part / gridDim.x;
    int lo = 0, hi = count;  // last range that starts at or before `at`
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (seg_start[mid] <= at) lo = mid; else hi = mid;
    }
    if (at < total) at = seg_start[lo] + ((at - seg_start[lo]) & ~(kCutBytes - 1));
    share[k] = at;
    if (k == 0) first = lo;
  }
  for (int s = first; s < count && seg_start[s] < share[1]; ++s) {
    const long long lo = max(share[0], seg_start[s]) - seg_start[s];
    const long long hi = min(share[1], seg_start[s + 1]) - seg_start[s];
    if (hi > lo) {
      copy_piece(reinterpret_cast<const char*>(segments[3ll * s]) + lo, reinterpret_cast<char*>(segments[3ll * s + 1]) + lo,
                 hi - lo);
    }
  }
}

}  // namespace
}  // namespace rlt

extern "C" {

int rlt_kv_push(const void* src, void* dst, int64_t nbytes, rlt_stream_t stream) {
  const rlt::NvtxRange range("rlt.kv_push");
  if (nbytes == 0) return RLT_OK;
  if (src == nullptr || dst == nullptr || nbytes < 0) return RLT_E_INVALID;
  int sms = 0;
  const int rc = rlt::sm_count(&sms);
  if (rc != RLT_OK) return rc;
  // one persistent wave; a small range gets one CTA per 16 KiB (one pass of the copy loop)
  const long long passes = (nbytes + 16383) / 16384;
  const int grid = static_cast<int>(passes < sms * static_cast<long long>(rlt::kCtasPerSm) ? passes : sms * static_cast<long long>(rlt::kCtasPerSm));
  rlt::push_kernel<<<grid, rlt::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(src), static_cast<char*>(dst), nbytes);
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

int rlt_kv_copy_segments(const int64_t* segments, int32_t count, rlt_stream_t stream) {
  const rlt::NvtxRange range("rlt.kv_copy_segments");
  if (count == 0) return RLT_OK;
  if (segments == nullptr || count < 0) return RLT_E_INVALID;
  if (count > RLT_MAX_SEGMENTS) return RLT_E_LIMIT;
  int sms = 0;
  const int rc = rlt::sm_count(&sms);
  if (rc != RLT_OK) return rc;
  const size_t smem = (static_cast<size_t>(count) + 1) * sizeof(long long);
  rlt::segment_copy_kernel<<<sms * rlt::kCtasPerSm, rlt::kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const long long*>(segments), count);
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // extern "C"
