// Typed tensor movement: a flat copy with an optional second output of another type, and batches
// of strided 2-D copies described by a table of int64[8] rows
// (source address, destination address, rows, cols, source row/col stride, destination row/col
// stride; strides in elements). It takes the place of the reference's Triton
// tensor_transfer_kernel (vllm_rlt/kernels/tensor_transfer.py:8-42), which moves step metadata,
// block tables and hidden-state rows on one device or from mapped host memory to the device.
//
// Element types are int32, int64, float16, bfloat16 and float32. Values are converted by the
// usual cast rules (integer narrowing wraps, float -> integer truncates toward zero, integer and
// float -> float round to nearest even). Integers never pass through a floating type, so int64
// ids above 2^53 survive an int64 -> int64 copy exactly.

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace rlt {
namespace {

template <typename D, typename S>
struct Convert {
  __device__ static D run(S v) { return static_cast<D>(v); }
};
// float-like sources go through float; float-like destinations come from float or the integer itself
template <typename D>
struct Convert<D, __half> {
  __device__ static D run(__half v) { return Convert<D, float>::run(__half2float(v)); }
};
template <typename D>
struct Convert<D, __nv_bfloat16> {
  __device__ static D run(__nv_bfloat16 v) { return Convert<D, float>::run(__bfloat162float(v)); }
};
template <>
struct Convert<__half, float> {
  __device__ static __half run(float v) { return __float2half_rn(v); }
};
template <>
struct Convert<__nv_bfloat16, float> {
  __device__ static __nv_bfloat16 run(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Convert<__half, int> {
  __device__ static __half run(int v) { return __int2half_rn(v); }
};
template <>
struct Convert<__half, long long> {
  __device__ static __half run(long long v) { return __ll2half_rn(v); }
};
template <>
struct Convert<__nv_bfloat16, int> {
  __device__ static __nv_bfloat16 run(int v) { return __int2bfloat16_rn(v); }
};
template <>
struct Convert<__nv_bfloat16, long long> {
  __device__ static __nv_bfloat16 run(long long v) { return __ll2bfloat16_rn(v); }
};
template <>
struct Convert<__half, __half> {
  __device__ static __half run(__half v) { return v; }
};
template <>
struct Convert<__nv_bfloat16, __nv_bfloat16> {
  __device__ static __nv_bfloat16 run(__nv_bfloat16 v) { return v; }
};
template <>
struct Convert<__half, __nv_bfloat16> {
  __device__ static __half run(__nv_bfloat16 v) { return __float2half_rn(__bfloat162float(v)); }
};
template <>
struct Convert<__nv_bfloat16, __half> {
  __device__ static __nv_bfloat16 run(__half v) { return __float2bfloat16_rn(__half2float(v)); }
};

constexpr int kRows = 4;
constexpr int kTile = 256;

template <typename S, typename D>
__global__ void __launch_bounds__(kTile) segmented_transfer_kernel(const long long* __restrict__ descriptors) {
  const long long* d = descriptors + 8ll * blockIdx.x;
  const S* src = reinterpret_cast<const S*>(d[0]);
  D* dst = reinterpret_cast<D*>(d[1]);
  const long long rows = d[2], cols = d[3], sr = d[4], sc = d[5], dr = d[6], dc = d[7];
  const long long c = static_cast<long long>(blockIdx.z) * kTile + threadIdx.x;
  if (c >= cols) return;
#pragma unroll
  for (int k = 0; k < kRows; ++k) {
    const long long r = static_cast<long long>(blockIdx.y) * kRows + k;
    if (r < rows) dst[r * dr + c * dc] = Convert<D, S>::run(src[r * sr + c * sc]);
  }
}

// Flat copy with conversion. When every pointer is 16-byte aligned a thread handles N consecutive elements per
// step, N = 16 / (size of the widest of the three types): the widest side moves as one 16-byte access per thread
// and the narrower sides as 8-, 4- or 2-byte accesses, all of them contiguous across the warp, with kFlatUnroll
// steps in flight per thread. The last n % N elements, and unaligned tensors, go one element at a time.
constexpr int kFlatUnroll = 4;

template <int kBytes>
struct Bits;
template <>
struct Bits<16> { using type = uint4; };
template <>
struct Bits<8> { using type = uint2; };
template <>
struct Bits<4> { using type = uint32_t; };
template <>
struct Bits<2> { using type = uint16_t; };

template <typename T, int N>
struct alignas(sizeof(T) * N) Pack {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Pack<T, N> load_pack(const T* p) {
  using B = typename Bits<sizeof(T) * N>::type;
  union { B bits; Pack<T, N> pack; } u;
  u.bits = *reinterpret_cast<const B*>(p);
  return u.pack;
}

template <typename T, int N>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, N>& pack) {
  using B = typename Bits<sizeof(T) * N>::type;
  union { B bits; Pack<T, N> pack; } u;
  u.pack = pack;
  *reinterpret_cast<B*>(p) = u.bits;
}

template <typename S, typename D, typename E>
__global__ void __launch_bounds__(kTile) flat_transfer_kernel(const S* __restrict__ src, D* __restrict__ dst,
                                                              E* __restrict__ secondary, long long n, int vector_ok) {
  constexpr int kWidest = sizeof(S) > sizeof(D) ? (sizeof(S) > sizeof(E) ? sizeof(S) : sizeof(E))
                                                : (sizeof(D) > sizeof(E) ? sizeof(D) : sizeof(E));
  constexpr int N = 16 / kWidest;
  const long long first = static_cast<long long>(blockIdx.x) * kTile + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * kTile;
  long long done = 0;
  if (vector_ok) {
    const long long groups = n / N;
    for (long long base = first; base < groups; base += stride * kFlatUnroll) {
      Pack<S, N> in[kFlatUnroll];
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u) {
        const long long g = base + u * stride;
        if (g < groups) in[u] = load_pack<S, N>(src + g * N);
      }
#pragma unroll
      for (int u = 0; u < kFlatUnroll; ++u) {
        const long long g = base + u * stride;
        if (g >= groups) continue;
        Pack<D, N> out;
#pragma unroll
        for (int k = 0; k < N; ++k) out.v[k] = Convert<D, S>::run(in[u].v[k]);
        store_pack<D, N>(dst + g * N, out);
        if (secondary != nullptr) {
          Pack<E, N> second;
#pragma unroll
          for (int k = 0; k < N; ++k) second.v[k] = Convert<E, S>::run(in[u].v[k]);
          store_pack<E, N>(secondary + g * N, second);
        }
      }
    }
    done = groups * N;
  }
  for (long long i = done + first; i < n; i += stride) {
    const S v = src[i];
    dst[i] = Convert<D, S>::run(v);
    if (secondary != nullptr) secondary[i] = Convert<E, S>::run(v);
  }
}

template <typename S, typename D>
int launch_segmented(const long long* descriptors, int count, int max_rows, int max_cols, cudaStream_t stream) {
  const dim3 grid(count, (max_rows + kRows - 1) / kRows, (max_cols + kTile - 1) / kTile);
  if (grid.y > 65535u || grid.z > 65535u) return RLT_E_LIMIT;
  segmented_transfer_kernel<S, D><<<grid, kTile, 0, stream>>>(descriptors);
  return RLT_OK;
}

template <typename S, typename D>
int launch_flat(const void* src, void* dst, void* secondary, long long n, int secondary_dtype, int grid,
                cudaStream_t stream) {
  const S* s = static_cast<const S*>(src);
  D* d = static_cast<D*>(dst);
  const int vec = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                    reinterpret_cast<uintptr_t>(secondary)) & 15u) == 0;
  if (secondary == nullptr) {  // no second output: its type must not narrow the vector width
    flat_transfer_kernel<S, D, D><<<grid, kTile, 0, stream>>>(s, d, static_cast<D*>(nullptr), n, vec);
    return RLT_OK;
  }
  switch (secondary_dtype) {
    case RLT_DTYPE_I32: flat_transfer_kernel<S, D, int><<<grid, kTile, 0, stream>>>(s, d, static_cast<int*>(secondary), n, vec); break;
    case RLT_DTYPE_I64: flat_transfer_kernel<S, D, long long><<<grid, kTile, 0, stream>>>(s, d, static_cast<long long*>(secondary), n, vec); break;
    case RLT_DTYPE_F16: flat_transfer_kernel<S, D, __half><<<grid, kTile, 0, stream>>>(s, d, static_cast<__half*>(secondary), n, vec); break;
    case RLT_DTYPE_BF16: flat_transfer_kernel<S, D, __nv_bfloat16><<<grid, kTile, 0, stream>>>(s, d, static_cast<__nv_bfloat16*>(secondary), n, vec); break;
    case RLT_DTYPE_F32: flat_transfer_kernel<S, D, float><<<grid, kTile, 0, stream>>>(s, d, static_cast<float*>(secondary), n, vec); break;
    default: return RLT_E_INVALID;
  }
  return RLT_OK;
}

// Calls f.template operator()<S, D>() for the pair of type codes.
template <typename F>
int dispatch_pair(int src_dtype, int dst_dtype, F f) {
#define RLT_DST(S)                                                      \
  switch (dst_dtype) {                                                  \
    case RLT_DTYPE_I32: return f.template operator()<S, int>();         \
    case RLT_DTYPE_I64: return f.template operator()<S, long long>();   \
    case RLT_DTYPE_F16: return f.template operator()<S, __half>();      \
    case RLT_DTYPE_BF16: return f.template operator()<S, __nv_bfloat16>(); \
    case RLT_DTYPE_F32: return f.template operator()<S, float>();       \
    default: return RLT_E_INVALID;                                      \
  }
  switch (src_dtype) {
    case RLT_DTYPE_I32: RLT_DST(int)
    case RLT_DTYPE_I64: RLT_DST(long long)
    case RLT_DTYPE_F16: RLT_DST(__half)
    case RLT_DTYPE_BF16: RLT_DST(__nv_bfloat16)
    case RLT_DTYPE_F32: RLT_DST(float)
    default: return RLT_E_INVALID;
  }
#undef RLT_DST
}

struct SegmentedCall {
  const long long* descriptors;
  int count, max_rows, max_cols;
  cudaStream_t stream;
  template <typename S, typename D>
  int operator()() const { return launch_segmented<S, D>(descriptors, count, max_rows, max_cols, stream); }
};

struct FlatCall {
  const void* src;
  void* dst;
  void* secondary;
  long long n;
  int secondary_dtype, grid;
  cudaStream_t stream;
  template <typename S, typename D>
  int operator()() const { return launch_flat<S, D>(src, dst, secondary, n, secondary_dtype, grid, stream); }
};

}  // namespace
}  // namespace rlt

extern "C" {

int rlt_tensor_transfer(const int64_t* descriptors, int32_t count, int32_t max_rows, int32_t max_cols,
                        int32_t src_dtype, int32_t dst_dtype, rlt_stream_t stream) {
  if (count == 0) return RLT_OK;
  if (descriptors == nullptr || count < 0 || max_rows < 1 || max_cols < 1) return RLT_E_INVALID;
  const rlt::SegmentedCall call{reinterpret_cast<const long long*>(descriptors), count, max_rows, max_cols,
                                reinterpret_cast<cudaStream_t>(stream)};
  const int rc = rlt::dispatch_pair(src_dtype, dst_dtype, call);
  if (rc != RLT_OK) return rc;
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

int rlt_tensor_copy(const void* src, void* dst, void* secondary, int64_t count, int32_t src_dtype, int32_t dst_dtype,
                    int32_t secondary_dtype, rlt_stream_t stream) {
  if (count == 0) return RLT_OK;
  if (src == nullptr || dst == nullptr || count < 0) return RLT_E_INVALID;
  int sms = 0;
  const int rc0 = rlt::sm_count(&sms);
  if (rc0 != RLT_OK) return rc0;
  // a thread of the vector path covers kFlatUnroll groups of at least two elements per step
  const long long per_block = static_cast<long long>(rlt::kTile) * 2 * rlt::kFlatUnroll;
  const long long blocks = (count + per_block - 1) / per_block;
  const int grid = static_cast<int>(blocks < sms * 8ll ? blocks : sms * 8ll);
  const rlt::FlatCall call{src, dst, secondary, count, secondary_dtype, grid, reinterpret_cast<cudaStream_t>(stream)};
  const int rc = rlt::dispatch_pair(src_dtype, dst_dtype, call);
  if (rc != RLT_OK) return rc;
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // extern "C"
