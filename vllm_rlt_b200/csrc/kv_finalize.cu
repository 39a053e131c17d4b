// Batched exit-depth propagation inside one LAST_EXITED pool.
//
// When a token leaves the recurrence at plane e, every deeper plane must hold a copy of
// plane e's K/V row so that later tokens attending at those depths read the last computed
// state. The reference does this per token with basic-index copies
// (KVCacheManager.finalize_token, vllm_rlt/core/kv_cache_manager.py:1053-1076) or with a
// Triton kernel over (row, target plane, channel tile) plus a second launch for the scales
// (finalize_kernel, vllm_rlt/kernels/routing.py:147-179; ModelRunner.finalize_many,
// vllm_rlt/worker/model_runner.py:1349-1395). Here one launch covers K, V and both scale
// tensors: a work unit is (row, tensor); it loads the token's row of every selected layer once
// with 16-byte streaming loads and stores it to every deeper plane.
//
// HBM roofline: each selected (layer, tensor) row is read once and written once per deeper
// plane. Pools with more than kFanPlanes planes use the older kernel, whose unit is
// (row, target plane, tensor) and which reads the row once per target.

#include "common.cuh"

namespace rlt {
namespace {

struct FinalizeRegion {
  char* key;
  char* value;
  long long block_bytes, layer_bytes, token_bytes;
  int vec_bytes;
  int row_vecs;        // token_bytes / vec_bytes
  unsigned row_magic;  // div_magic(row_vecs), 0 for one-vector rows
};

struct FinalizeParams {
  FinalizeRegion region[2];
  int num_regions;
  int planes, block_size, num_blocks, num_layers;
  unsigned long long layer_mask;  // bit l set: layer l is copied (the recurrent layers)
  const int* tables;              // [requests, planes, table_width]
  int table_width, num_requests;
  const int* rows;                // [n][3]: request index, exit plane, token position
  int n;
  int* status;
};

constexpr int kUnroll = 4;

// Copies the token's row of every selected layer as one flat vector array: vector i belongs to selected
// layer i / row_vecs. kUnroll loads are in flight per thread before the first store.
template <typename T>
__device__ __forceinline__ void copy_layers(const char* src, char* dst, const int* layer_of, int layers, int row_vecs,
                                            unsigned row_magic, long long layer_bytes) {
  const int total = layers * row_vecs;
  for (int base = threadIdx.x; base < total; base += kThreads * kUnroll) {
    T regs[kUnroll];
    long long at[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      at[u] = -1;
      if (i < total) {
        const int slot = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        at[u] = layer_of[slot] * layer_bytes + static_cast<long long>(i - slot * row_vecs) * static_cast<long long>(sizeof(T));
        regs[u] = ld_stream(reinterpret_cast<const T*>(src + at[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (at[u] >= 0) st_stream(reinterpret_cast<T*>(dst + at[u]), regs[u]);
    }
  }
}

constexpr int kFanPlanes = 64;

// One load, several stores: vector i of the flat (selected layers x row vectors) array goes to the same
// in-block offset of every target plane whose block is valid (plane_base >= 0).
template <typename T>
__device__ __forceinline__ void copy_layers_fan(const char* src, char* pool, const long long* plane_base, int first,
                                                int planes, const int* layer_of, int layers, int row_vecs,
                                                unsigned row_magic, long long layer_bytes) {
  const int total = layers * row_vecs;
  for (int base = threadIdx.x; base < total; base += kThreads * kUnroll) {
    T regs[kUnroll];
    long long at[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      at[u] = -1;
      if (i < total) {
        const int slot = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        at[u] = layer_of[slot] * layer_bytes + static_cast<long long>(i - slot * row_vecs) * static_cast<long long>(sizeof(T));
        regs[u] = ld_stream(reinterpret_cast<const T*>(src + at[u]));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (at[u] >= 0) {
        for (int t = first; t < planes; ++t) {
          const long long pb = plane_base[t];
          if (pb >= 0) st_stream(reinterpret_cast<T*>(pool + pb + at[u]), regs[u]);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 4) finalize_fan_kernel(const FinalizeParams p) {
  __shared__ int layer_of[64];  // the selected layers, in order
  __shared__ int n_selected;
  __shared__ long long plane_base[2][kFanPlanes];  // per unit: byte offset of the token's row in each target plane
  if (threadIdx.x == 0) {
    int n = 0;
    for (int layer = 0; layer < p.num_layers; ++layer) {
      if ((p.layer_mask >> layer) & 1ull) layer_of[n++] = layer;
    }
    n_selected = n;
  }
  __syncthreads();
  const int layers = n_selected;
  const int tensors = 2 * p.num_regions;
  const long long units = static_cast<long long>(p.n) * tensors;
  int parity = 0;  // flipped only by units that reach the barrier, so two such units in a row never share a table
  for (long long w = blockIdx.x; w < units; w += gridDim.x) {
    const int tensor = static_cast<int>(w % tensors);
    const int row = static_cast<int>(w / tensors);
    const int request = p.rows[3 * row], exit_plane = p.rows[3 * row + 1], position = p.rows[3 * row + 2];
    if (request < 0 || request >= p.num_requests || exit_plane < 0 || exit_plane >= p.planes || position < 0 ||
        position >= p.table_width * p.block_size) {
      if (threadIdx.x == 0 && tensor == 0) report(p.status, RLT_STATUS_BAD_PLANE, row, position, exit_plane);
      continue;
    }
    if (exit_plane + 1 >= p.planes) continue;  // the deepest plane was computed: nothing to fill
    const int page = position / p.block_size, offset = position - page * p.block_size;
    const long long base = (static_cast<long long>(request) * p.planes) * p.table_width + page;
    const int sb = p.tables[base + static_cast<long long>(exit_plane) * p.table_width];
    if (sb < 0 || sb >= p.num_blocks) {
      if (threadIdx.x == 0) report(p.status, RLT_STATUS_BAD_BLOCK, request, page, sb);
      continue;
    }
    const FinalizeRegion& rg = p.region[tensor >> 1];
    long long* pb = plane_base[parity];
    const int t = static_cast<int>(threadIdx.x);
    if (t > exit_plane && t < p.planes) {
      const int db = p.tables[base + static_cast<long long>(t) * p.table_width];
      long long at = -1;
      if (db < 0 || db >= p.num_blocks) {
        report(p.status, RLT_STATUS_BAD_BLOCK, request, page, db);
      } else {
        at = db * rg.block_bytes + offset * rg.token_bytes;
      }
      pb[t] = at;
    }
    __syncthreads();
    parity ^= 1;
    char* pool = (tensor & 1) ? rg.value : rg.key;
    const char* src = pool + sb * rg.block_bytes + offset * rg.token_bytes;
    if (rg.vec_bytes == 16) {
      copy_layers_fan<uint4>(src, pool, pb, exit_plane + 1, p.planes, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    } else if (rg.vec_bytes == 4) {
      copy_layers_fan<uint32_t>(src, pool, pb, exit_plane + 1, p.planes, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    } else {
      copy_layers_fan<uint8_t>(src, pool, pb, exit_plane + 1, p.planes, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    }
  }
}

__global__ void __launch_bounds__(kThreads, 4) finalize_kernel(const FinalizeParams p) {
  __shared__ int layer_of[64];  // the selected layers, in order
  __shared__ int n_selected;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int layer = 0; layer < p.num_layers; ++layer) {
      if ((p.layer_mask >> layer) & 1ull) layer_of[n++] = layer;
    }
    n_selected = n;
  }
  __syncthreads();
  const int layers = n_selected;
  const int tensors = 2 * p.num_regions;
  const int targets = p.planes - 1;
  const long long units = static_cast<long long>(p.n) * targets * tensors;
  for (long long w = blockIdx.x; w < units; w += gridDim.x) {
    const int tensor = static_cast<int>(w % tensors);
    const long long rest = w / tensors;
    const int target = 1 + static_cast<int>(rest % targets);
    const int row = static_cast<int>(rest / targets);
    const int request = p.rows[3 * row], exit_plane = p.rows[3 * row + 1], position = p.rows[3 * row + 2];
    if (request < 0 || request >= p.num_requests || exit_plane < 0 || exit_plane >= p.planes || position < 0 ||
        position >= p.table_width * p.block_size) {
      if (threadIdx.x == 0 && target == 1 && tensor == 0) report(p.status, RLT_STATUS_BAD_PLANE, row, position, exit_plane);
      continue;
    }
    if (target <= exit_plane) continue;  // that plane was computed, not copied
    const int page = position / p.block_size, offset = position - page * p.block_size;
    const long long base = (static_cast<long long>(request) * p.planes) * p.table_width + page;
    const int sb = p.tables[base + static_cast<long long>(exit_plane) * p.table_width];
    const int db = p.tables[base + static_cast<long long>(target) * p.table_width];
    if (sb < 0 || sb >= p.num_blocks || db < 0 || db >= p.num_blocks) {
      if (threadIdx.x == 0) report(p.status, RLT_STATUS_BAD_BLOCK, request, page, sb < 0 || sb >= p.num_blocks ? sb : db);
      continue;
    }
    const FinalizeRegion& rg = p.region[tensor >> 1];
    char* pool = (tensor & 1) ? rg.value : rg.key;
    const char* src = pool + sb * rg.block_bytes + offset * rg.token_bytes;
    char* dst = pool + db * rg.block_bytes + offset * rg.token_bytes;
    if (rg.vec_bytes == 16) {
      copy_layers<uint4>(src, dst, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    } else if (rg.vec_bytes == 4) {
      copy_layers<uint32_t>(src, dst, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    } else {
      copy_layers<uint8_t>(src, dst, layer_of, layers, rg.row_vecs, rg.row_magic, rg.layer_bytes);
    }
  }
}

}  // namespace
}  // namespace rlt

extern "C" {

int rlt_kv_finalize(const RltPool* pool, const int32_t* tables, int32_t num_requests, int32_t table_width,
                    const int32_t* rows, int32_t count, uint64_t layer_mask, int32_t* status, rlt_stream_t stream) {
  const rlt::NvtxRange range("rlt.kv_finalize");
  if (count == 0) return RLT_OK;
  if (pool == nullptr || tables == nullptr || rows == nullptr || count < 0 || num_requests < 1 || table_width < 1)
    return RLT_E_INVALID;
  if (pool->codes.key == nullptr || pool->codes.value == nullptr) return RLT_E_INVALID;
  if (pool->num_layers < 1 || pool->num_layers > 64 || pool->block_size < 1 || pool->num_planes < 1 ||
      pool->num_blocks < 1)
    return RLT_E_LIMIT;
  if (pool->num_planes == 1) return RLT_OK;  // a SHARED pool has nothing deeper to fill
  rlt::FinalizeParams p{};
  p.num_regions = pool->scales.key != nullptr ? 2 : 1;
  if (p.num_regions == 2 && pool->scales.value == nullptr) return RLT_E_INVALID;
  for (int g = 0; g < p.num_regions; ++g) {
    const RltRegion& r = g == 0 ? pool->codes : pool->scales;
    if (r.token_bytes <= 0 || r.layer_bytes != r.token_bytes * pool->block_size ||
        r.block_bytes != r.layer_bytes * pool->num_layers)
      return RLT_E_GEOMETRY;
    rlt::FinalizeRegion& out = p.region[g];
    out.key = static_cast<char*>(r.key);
    out.value = static_cast<char*>(r.value);
    out.block_bytes = r.block_bytes;
    out.layer_bytes = r.layer_bytes;
    out.token_bytes = r.token_bytes;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(r.key) | reinterpret_cast<uintptr_t>(r.value) |
                           static_cast<uintptr_t>(r.token_bytes);
    out.vec_bytes = (bits & 15u) == 0 ? 16 : (bits & 3u) == 0 ? 4 : 1;
    out.row_vecs = static_cast<int>(r.token_bytes / out.vec_bytes);
    out.row_magic = out.row_vecs == 1 ? 0u : rlt::div_magic(static_cast<uint32_t>(out.row_vecs));
    // the flat index (selected layers x row vectors) times row_vecs must stay below 2^32 for the multiplier split
    if (64ll * out.row_vecs * out.row_vecs >= (1ll << 32)) return RLT_E_LIMIT;
  }
  p.planes = pool->num_planes;
  p.block_size = pool->block_size;
  p.num_blocks = pool->num_blocks;
  p.num_layers = pool->num_layers;
  const uint64_t all = pool->num_layers == 64 ? ~0ull : ((1ull << pool->num_layers) - 1ull);
  p.layer_mask = layer_mask == 0 ? all : (layer_mask & all);
  p.tables = tables;
  p.table_width = table_width;
  p.num_requests = num_requests;
  p.rows = rows;
  p.n = count;
  p.status = status;
  int sms = 0;
  const int rc = rlt::sm_count(&sms);
  if (rc != RLT_OK) return rc;
  const bool fan = p.planes <= rlt::kFanPlanes;
  const long long units = static_cast<long long>(count) * (fan ? 1 : p.planes - 1) * 2 * p.num_regions;
  const int grid = static_cast<int>(units < sms * 4ll ? units : sms * 4ll);
  if (fan) {
    rlt::finalize_fan_kernel<<<grid, rlt::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  } else {
    rlt::finalize_kernel<<<grid, rlt::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  }
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // extern "C"
