// Batched exit-depth propagation inside one LAST_EXITED pool.
//
// When a token leaves the recurrence at plane e, every deeper plane must hold a copy of
// plane e's K/V row so that later tokens attending at those depths read the last computed
// state. The reference does this per token with basic-index copies
// (KVCacheManager.finalize_token, vllm_rlt/core/kv_cache_manager.py:1053-1076) or with a
// Triton kernel over (row, target plane, channel tile) plus a second launch for the scales
// (finalize_kernel, vllm_rlt/kernels/routing.py:147-179; ModelRunner.finalize_many,
// vllm_rlt/worker/model_runner.py:1349-1395). Here one launch covers K, V and both scale
// tensors: each row's K, V and scale rows of every selected layer are loaded once with 16-byte
// streaming loads and stored to every deeper plane, and the rows are dealt to the CTAs by cost.
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
  int group_rows;                 // rows of one page taken together: at most kGroupRows, fewer for very long rows
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

// ---------------------------------------------------------------------------------------------
// finalize_fan_kernel: one load, one store per deeper plane; work split by cost; rows of one page move together.
//
// Cost. A row that exits at plane e costs (1 + deeper planes) row copies: nothing for the deepest plane, four for
// plane 0 of a four-plane pool. Every CTA derives the same exclusive scan of the row costs (each thread sums a
// contiguous slice of rows; one block scan of the 256 sums), cuts the total into gridDim.x equal shares and takes
// the contiguous run of rows - down to a fraction of the first and last row, in whole (tensor, layer) pieces - that
// makes up its share. No atomics, no scratch memory, and two neighbouring CTAs compute their common cut from the
// same numbers.
//
// Locality. A row is 24 pieces of 4 KiB that lie 64 KiB apart, so copying row after row sprays DRAM with 4 KiB
// accesses. Consecutive rows of a batch are usually consecutive tokens of one request, hence rows of one page, and
// on every deeper plane their copies are neighbours in one block. Rows of a CTA's run that share (request, page) are
// therefore taken as a group and walked layer by layer, token by token: the stores of one layer to one plane then
// cover up to block_size * token_bytes contiguous bytes (64 KiB for the Ouro shape). The block-table entries of a
// group (one per plane, shared by its rows) are fetched while the previous group streams.

constexpr int kGroupRows = 32;  // rows of one page taken together (one warp detects and compacts them)

// (1 + deeper planes) if the row is valid and has deeper planes, else 0. `say`: report an invalid row (one CTA does).
__device__ __forceinline__ int row_cost(const FinalizeParams& p, int row, bool say) {
  const int request = p.rows[3 * row], exit_plane = p.rows[3 * row + 1], position = p.rows[3 * row + 2];
  if (request < 0 || request >= p.num_requests || exit_plane < 0 || exit_plane >= p.planes || position < 0 ||
      position >= p.table_width * p.block_size) {
    if (say) report(p.status, RLT_STATUS_BAD_PLANE, row, position, exit_plane);
    return 0;
  }
  return exit_plane + 1 < p.planes ? p.planes - exit_plane : 0;
}

// What one group needs while it streams: per plane the byte offset of the page's block (either region), per carried
// row its exit plane and the byte offset of its token inside a block layer (either region).
struct GroupTables {
  long long plane_off[2][kFanPlanes];  // -1: that plane's block id is outside the pool
  int tok_off[2][kGroupRows];
  int exit_plane[kGroupRows];
  int carried;   // rows with something to copy (those are the ones listed above)
  int rows;      // rows of the batch the group spans, carried or not
  unsigned magic;  // div_magic(carried), 0 when carried <= 1
};

// Pieces [a, b) of every carried row of a group, for one region: piece = (K|V, selected layer). The flat vector array
// is ordered piece, row, vector, so consecutive threads walk consecutive tokens of one layer. Each vector is loaded
// once from the row's exit plane and stored to the same in-block offset of every deeper plane whose block is valid.
// This form serves rows shorter than a warp's reach (scale rows); fan_group_rows below serves the long ones.
template <typename T>
__device__ __forceinline__ void fan_group(const FinalizeRegion& rg, const GroupTables& gt, int g, int planes,
                                          const int* layer_of, int layers, int a, int b) {
  const int carried = gt.carried;
  const int total = (b - a) * carried * rg.row_vecs;
  // where vector i lives: (source/destination offset inside a plane's block, row of the group, K|V)
  auto locate = [&](int i, int* row, int* kv) -> long long {
    const int q = rg.row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), rg.row_magic)) : i;  // piece x row
    const int piece_rel = gt.magic ? static_cast<int>(__umulhi(static_cast<unsigned>(q), gt.magic)) : q;
    const int r = q - piece_rel * carried;
    const int piece = a + piece_rel;
    *kv = piece >= layers;
    *row = r;
    return layer_of[piece - *kv * layers] * rg.layer_bytes + gt.tok_off[g][r] +
           static_cast<long long>(i - q * rg.row_vecs) * static_cast<long long>(sizeof(T));
  };
  for (int base = threadIdx.x; base < total; base += kThreads * kUnroll) {
    T regs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total) {
        int r, kv;
        const long long at = locate(i, &r, &kv);
        const long long src = gt.plane_off[g][gt.exit_plane[r]];
        if (src >= 0) regs[u] = ld_stream(reinterpret_cast<const T*>((kv ? rg.value : rg.key) + src + at));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total) {
        int r, kv;
        const long long at = locate(i, &r, &kv);  // recomputed rather than kept live across the loads
        const int e = gt.exit_plane[r];
        if (gt.plane_off[g][e] >= 0) {
          char* pool = kv ? rg.value : rg.key;
          for (int t = e + 1; t < planes; ++t) {
            const long long pb = gt.plane_off[g][t];
            if (pb >= 0) st_stream(reinterpret_cast<T*>(pool + pb + at), regs[u]);
          }
        }
      }
    }
  }
}

// The same pieces with one warp per (piece, row): where the row lives is worked out once per warp and row instead of
// once per vector, and each lane then keeps kRowUnroll 16-byte loads in flight (4 KiB per warp for the Ouro shape).
// Consecutive warps take consecutive rows of one layer, so the CTA still covers neighbouring tokens together.
constexpr int kRowUnroll = 8;

__device__ __forceinline__ void fan_group_rows(const FinalizeRegion& rg, const GroupTables& gt, int g, int planes,
                                               const int* layer_of, int layers, int a, int b) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int carried = gt.carried;
  const int jobs = (b - a) * carried;
  for (int job = warp; job < jobs; job += kThreads / 32) {
    const int piece_rel = gt.magic ? static_cast<int>(__umulhi(static_cast<unsigned>(job), gt.magic)) : job;
    const int r = job - piece_rel * carried;
    const int piece = a + piece_rel;
    const int kv = piece >= layers;
    const int e = gt.exit_plane[r];
    const long long src_block = gt.plane_off[g][e];
    if (src_block < 0) continue;
    char* pool = kv ? rg.value : rg.key;
    const long long in_block = layer_of[piece - kv * layers] * rg.layer_bytes + gt.tok_off[g][r];
    const uint4* from = reinterpret_cast<const uint4*>(pool + src_block + in_block);
    for (int base = lane; base < rg.row_vecs; base += 32 * kRowUnroll) {
      uint4 regs[kRowUnroll];
#pragma unroll
      for (int u = 0; u < kRowUnroll; ++u) {
        const int v = base + u * 32;
        if (v < rg.row_vecs) regs[u] = ld_stream(from + v);
      }
      for (int t = e + 1; t < planes; ++t) {
        const long long pb = gt.plane_off[g][t];
        if (pb < 0) continue;
        uint4* to = reinterpret_cast<uint4*>(pool + pb + in_block);
#pragma unroll
        for (int u = 0; u < kRowUnroll; ++u) {
          const int v = base + u * 32;
          if (v < rg.row_vecs) st_stream(to + v, regs[u]);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 3) finalize_fan_kernel(const FinalizeParams p) {
  __shared__ int layer_of[64];  // the selected layers, in order
  __shared__ int n_selected;
  __shared__ long long slice_start[kThreads + 1];  // cost of all rows before each thread's slice; [kThreads] = total
  __shared__ long long warp_part[kThreads / 32];
  __shared__ int cut_row[2];        // first row of this CTA's share, and the row its share ends in
  __shared__ long long cut_rem[2];  // (cost x pieces) of that row that lies before the cut
  __shared__ GroupTables tables[2];  // double buffered: the next group's are written while this one streams
  const int tid = static_cast<int>(threadIdx.x);
  const int lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    int n = 0;
    for (int layer = 0; layer < p.num_layers; ++layer) {
      if ((p.layer_mask >> layer) & 1ull) layer_of[n++] = layer;
    }
    n_selected = n;
  }

  // ---- the same cost scan in every CTA ----
  const int per = (p.n + kThreads - 1) / kThreads;
  const int mine_lo = min(p.n, tid * per), mine_hi = min(p.n, mine_lo + per);
  long long mine = 0;
  for (int i = mine_lo; i < mine_hi; ++i) mine += row_cost(p, i, blockIdx.x == 0);
  {
    long long inc = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const long long up = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += up;
    }
    if (lane == 31) warp_part[warp] = inc;
    __syncthreads();
    long long before = 0;
    for (int w = 0; w < warp; ++w) before += warp_part[w];
    slice_start[tid] = before + inc - mine;
    if (tid == kThreads - 1) slice_start[kThreads] = before + inc;
  }
  __syncthreads();
  const long long total = slice_start[kThreads];
  if (total == 0) return;
  // Where this CTA's share begins and ends, in units of one (tensor, layer) piece of one row copy, then as
  // (cost position, piece remainder). total * pieces * gridDim.x stays far below 2^63.
  const int layers = n_selected;
  const int pieces_per_region = 2 * layers;
  const int pieces = pieces_per_region * p.num_regions;
  const long long fine_total = total * pieces;
  const long long fine[2] = {fine_total * blockIdx.x / gridDim.x, fine_total * (blockIdx.x + 1) / gridDim.x};
  if (fine[0] == fine[1]) return;  // an empty share (fewer pieces than CTAs)
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const long long c = fine[k] / pieces;
    if (c >= total) {
      if (tid == 0) {
        cut_row[k] = p.n;
        cut_rem[k] = 0;
      }
    } else if (slice_start[tid] <= c && c < slice_start[tid + 1]) {  // exactly one thread: the cut is in its slice
      long long acc = slice_start[tid];
      for (int i = mine_lo; i < mine_hi; ++i) {
        const int cost = row_cost(p, i, false);
        if (acc + cost > c) {
          cut_row[k] = i;
          cut_rem[k] = (c - acc) * pieces + fine[k] % pieces;  // pieces of this row's cost * pieces before the cut
          break;
        }
        acc += cost;
      }
    }
  }
  __syncthreads();
  // The share: pieces [head_lo, pieces) of row `first` if head_lo > 0, whole rows [whole_lo, whole_hi), and pieces
  // [0, tail_hi) of row whole_hi if tail_hi > 0. A share inside one row is the head alone, cut at both ends.
  const int first = cut_row[0], last = cut_row[1];
  const int head_lo = static_cast<int>(cut_rem[0] / row_cost(p, first, false));
  const int tail_hi = last < p.n ? static_cast<int>(cut_rem[1] / max(row_cost(p, last, false), 1)) : 0;
  const bool one_row = first == last;
  const int whole_lo = first + (head_lo > 0 || one_row ? 1 : 0);
  const int whole_hi = last;  // exclusive

  // A group starts at row `start`. Its extent: the head and the tail are groups of their own; otherwise up to
  // kGroupRows consecutive whole rows of the same request and page. `limit` is where it may reach at most.
  auto limit_of = [&](int start) -> int {
    if (start < whole_lo || start >= whole_hi) return start + 1;
    return min(whole_hi, start + p.group_rows);
  };
  // Step 1 of fetching a group (before the current one streams): the loads are issued, nothing waits for them.
  // Threads below `planes` look up the page's block on their plane; warp 0 reads the group's candidate rows.
  auto fetch = [&](int start, int* block, int* request, int* exit_plane, int* position) {
    *block = -2;
    *request = -1;
    if (start > last || start >= p.n) return;
    const int r0 = p.rows[3 * start], pos0 = p.rows[3 * start + 2];
    const bool head_ok = r0 >= 0 && r0 < p.num_requests && pos0 >= 0 && pos0 < p.table_width * p.block_size;
    if (head_ok && tid < p.planes)
      *block = p.tables[(static_cast<long long>(r0) * p.planes + tid) * p.table_width + pos0 / p.block_size];
    if (warp == 0 && start + lane < limit_of(start)) {
      *request = p.rows[3 * (start + lane)];
      *exit_plane = p.rows[3 * (start + lane) + 1];
      *position = p.rows[3 * (start + lane) + 2];
    }
  };
  // Step 2 (after the current group has streamed): write the group's tables. Warp 0 finds how far the run of rows
  // with the head row's (request, page) goes and compacts the rows that have something to copy.
  auto publish = [&](int start, GroupTables& out, int block, int request, int exit_plane, int position) {
    if (start > last || start >= p.n) {
      if (tid == 0) out.rows = out.carried = 0;
      return;
    }
    if (tid < p.planes) {
      long long at0 = -1, at1 = -1;
      if (block >= 0 && block < p.num_blocks) {
        at0 = block * p.region[0].block_bytes;
        if (p.num_regions == 2) at1 = block * p.region[1].block_bytes;
      } else if (block != -2) {
        report(p.status, RLT_STATUS_BAD_BLOCK, p.rows[3 * start], p.rows[3 * start + 2] / p.block_size, block);
      }
      out.plane_off[0][tid] = at0;
      out.plane_off[1][tid] = at1;
    }
    if (warp == 0) {
      const int r0 = __shfl_sync(0xffffffffu, request, 0), pos0 = __shfl_sync(0xffffffffu, position, 0);
      const bool listed = request >= 0 && start + lane < limit_of(start);
      const bool valid = listed && request < p.num_requests && exit_plane >= 0 && exit_plane < p.planes && position >= 0 &&
                         position < p.table_width * p.block_size;
      const bool head_valid = __shfl_sync(0xffffffffu, static_cast<int>(valid), 0) != 0;
      const bool same = lane == 0 || (head_valid && valid && request == r0 && position / p.block_size == pos0 / p.block_size);
      const unsigned run = __ballot_sync(0xffffffffu, same);
      const int rows = run == 0xffffffffu ? 32 : __ffs(~run) - 1;  // leading ones: how far the run goes
      const bool carry = lane < rows && valid && exit_plane + 1 < p.planes;
      const unsigned keep = __ballot_sync(0xffffffffu, carry);
      if (carry) {
        const int slot = __popc(keep & ((1u << lane) - 1u));
        const int offset = position % p.block_size;
        out.exit_plane[slot] = exit_plane;
        out.tok_off[0][slot] = offset * static_cast<int>(p.region[0].token_bytes);
        out.tok_off[1][slot] = p.num_regions == 2 ? offset * static_cast<int>(p.region[1].token_bytes) : 0;
      }
      if (lane == 0) {
        const int carried = __popc(keep);
        out.rows = rows;
        out.carried = carried;
        out.magic = carried > 1 ? static_cast<unsigned>((1ull << 32) / carried) + 1u : 0u;
      }
    }
  };

  int parity = 0;
  {
    int block, request, exit_plane = 0, position = 0;
    fetch(first, &block, &request, &exit_plane, &position);
    publish(first, tables[0], block, request, exit_plane, position);
  }
  __syncthreads();
  for (int start = first; start <= last && start < p.n;) {
    const GroupTables& gt = tables[parity];
    const int next = start + max(gt.rows, 1);
    int block, request, exit_plane = 0, position = 0;
    fetch(next, &block, &request, &exit_plane, &position);  // in flight while this group streams
    if (gt.carried > 0) {
      // pieces of each row that fall inside the share: everything, except for the head and the tail
      int lo = 0, hi = pieces;
      if (start == first && (head_lo > 0 || one_row)) lo = head_lo;
      if (start == last) hi = tail_hi;
      for (int g = 0; g < p.num_regions; ++g) {
        const int a = max(lo - g * pieces_per_region, 0), b = min(hi - g * pieces_per_region, pieces_per_region);
        if (a >= b) continue;
        const FinalizeRegion& rg = p.region[g];
        if (rg.vec_bytes == 16 && rg.row_vecs >= 32) {
          fan_group_rows(rg, gt, g, p.planes, layer_of, layers, a, b);
        } else if (rg.vec_bytes == 16) {
          fan_group<uint4>(rg, gt, g, p.planes, layer_of, layers, a, b);
        } else if (rg.vec_bytes == 4) {
          fan_group<uint32_t>(rg, gt, g, p.planes, layer_of, layers, a, b);
        } else {
          fan_group<uint8_t>(rg, gt, g, p.planes, layer_of, layers, a, b);
        }
      }
    }
    publish(next, tables[parity ^ 1], block, request, exit_plane, position);
    __syncthreads();  // the next group's tables are visible; this group's buffer is free for the one after
    parity ^= 1;
    start = next;
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
  int group_rows = 32;
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
    // the flat index (pieces x rows of a group x row vectors) times row_vecs must stay below 2^32 for the
    // multiplier split: long rows get smaller groups
    if (128ll * out.row_vecs * out.row_vecs >= (1ll << 32)) return RLT_E_LIMIT;
    const long long fit = ((1ll << 32) - 1) / (128ll * out.row_vecs * out.row_vecs);
    if (fit < group_rows) group_rows = static_cast<int>(fit);
  }
  p.group_rows = group_rows;
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
    // one persistent wave of three CTAs per SM; a CTA's share may be a fraction of a row, so small batches
    // still use every SM (a share of less than one (tensor, layer) piece is simply empty)
    rlt::finalize_fan_kernel<<<sms * 3, rlt::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  } else {
    rlt::finalize_kernel<<<grid, rlt::kThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  }
  RLT_CUDA_TRY(cudaGetLastError());
  rlt::g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // extern "C"
