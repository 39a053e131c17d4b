// Block-table driven KV copy: pool -> pool (handoff), pool -> packed (pack) and
// packed -> pool (scatter), one persistent kernel for all three.
//
// What it replaces in the reference: the Python walk of kv_segments over the
// source and the peer tables (vllm_rlt/pd/transport.py:29-63), the
// coalesce/partition step (:66-112) and the WRITE that NIXL performs with the
// resulting descriptors (:182-201). Here the walk runs on the GPU: each CTA
// derives its own slice of the (request, plane, block, tensor, layer) space
// from the block tables, so no descriptor list is ever built.
//
// Work decomposition
//   unit  = (request, logical block, destination plane, region, K|V, layer chunk)
//   row   = one token's bytes of one layer inside a unit (token_bytes long)
// A unit holds at most kMaxRows rows. For each unit the CTA first writes the
// source and destination byte offset of every row to shared memory (this is
// where block tables and per-token exit planes are read), then streams the
// unit as a flat array of 16-byte vectors: thread t handles vectors t, t+256,
// ... with kUnroll loads in flight before the first store. Row boundaries do
// not matter to the flat loop, so 64-byte scale rows use every lane just like
// 4 KiB code rows.
//
// Ragged requests: every CTA computes, with warp-shuffle prefix sums, the
// exclusive scan of per-request block counts (and token counts, for packed
// offsets) into shared memory, and finds a unit's request by binary search.
//
// HBM roofline: the kernel reads and writes each payload byte once; tables add
// 4 bytes per (request, plane, block). Algorithmic bytes per token per plane
// are 2 * layers * kv_heads * (head_dim * elt + scale) read and the same written.
//
// Flavours (RltOptions.variant, low 4 bits), all bit-identical in result:
//   0      register path, 4 x 16-byte streaming loads in flight per thread, 3 CTAs per SM (default;
//          measured at the HBM copy peak)
//   1, 2   the same with 8 loads in flight, with and without streaming cache hints
//   3, 4   rows move global -> shared -> global with cp.async.bulk, per-warp rings tracked by mbarriers
//   5      register path with 32-byte loads and stores
//
// The dedup wire image (pack / scatter in RLT_MODE_DEDUP) carries, per token, only the planes up to
// its exit plane. Where each (request, plane, block) starts in that image is computed on the device by
// three small kernels (count, tile scan, finish) into a caller-provided workspace; see plan_dedup.

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace rlt {
namespace {

struct RegionParams {
  const char* src_key;
  const char* src_value;
  char* dst_key;
  char* dst_value;
  long long block_bytes;
  long long layer_bytes;
  long long token_bytes;
  int vec_bytes;        // 16, 4 or 1
  int row_vecs;         // token_bytes / vec_bytes
  unsigned row_magic;   // div_magic(row_vecs)
  int wide_ok;          // rows and bases are 32-byte multiples: the 32-byte vector flavour may be used
  int layers_per_unit;  // layers one unit covers
  int chunks;           // ceil(layers in slice / layers_per_unit)
};

struct TableCopyParams {
  RegionParams region[2];
  int num_regions;
  int num_requests;
  int table_width;
  int src_planes;
  int dst_planes;   // destination planes, or wire planes for pack
  int plane_begin;  // planes iterated by this launch: [plane_begin, plane_begin + plane_count)
  int plane_count;
  int block_size;
  int src_blocks;
  int dst_blocks;
  const int* src_tables;
  const int* dst_tables;
  const int* tok_begin;
  const int* tok_end;
  const int* exit_planes;
  const long long* exit_offsets;
  long long exit_count;  // entries in exit_planes
  int plane_bias;   // 0: source plane = min(p, exit); src_planes: source plane = exit
  int layer_begin;
  int layer_end;
  int src_packed;   // source is the packed image (scatter)
  int dst_packed;   // destination is the packed image (pack)
  long long packed_token_bytes;  // 2 * layers in slice * (codes row + scales row)
  long long packed_bytes;        // size of the packed image; rows past it are skipped
  unsigned long long deep_layer_mask;  // layers carried for planes >= 1; 0 = all
  int dedup_wire;                // the packed image holds, per token, only planes up to its exit plane
  const int* dedup_prefix;       // [planes * total blocks] wire tokens before each (request, plane, block)
  int fan;                       // pool-to-pool dedup that reads each row once and stores it to every plane it fills
  int* status;
};

template <typename T, int kUnroll, bool kStreaming>
__device__ __forceinline__ void stream_rows(const char* __restrict__ src, char* __restrict__ dst,
                                            const long long* __restrict__ src_off,
                                            const long long* __restrict__ dst_off, int total_vecs,
                                            int row_vecs, unsigned row_magic) {
  // A skipped row has -1 in both offset tables. Row and offset are recomputed for the
  // stores instead of being kept live, which keeps the kernel at 64 registers.
  // row_magic == 0 marks one-vector rows, for which no 32-bit multiplier exists.
  for (int base = threadIdx.x; base < total_vecs; base += kThreads * kUnroll) {
    T regs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total_vecs) {
        const int row = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        const long long so = src_off[row];
        if (so >= 0) {
          const T* from = reinterpret_cast<const T*>(src + so) + (i - row * row_vecs);
          regs[u] = kStreaming ? ld_stream(from) : *from;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total_vecs) {
        const int row = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        const long long to = dst_off[row];
        if (to >= 0) {
          T* at = reinterpret_cast<T*>(dst + to) + (i - row * row_vecs);
          if (kStreaming) st_stream(at, regs[u]); else *at = regs[u];
        }
      }
    }
  }
}

// Exclusive scans of per-request block counts and token counts, into shared memory.
template <int kBlock>
__device__ void scan_requests(const TableCopyParams& p, int* blk_off, int* tok_off) {
  constexpr int kThreads = kBlock;  // shadows the file-wide constant: this routine serves CTAs of either size
  __shared__ int warp_sum[2][kThreads / 32];
  __shared__ int carry[2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    carry[0] = carry[1] = 0;
    blk_off[0] = tok_off[0] = 0;
  }
  __syncthreads();
  for (int tile = 0; tile < p.num_requests; tile += kThreads) {
    const int r = tile + threadIdx.x;
    int nb = 0, nt = 0;
    if (r < p.num_requests) {
      const int b = p.tok_begin[r], e = p.tok_end[r];
      if (e > b) {
        bool ok = b >= 0 && e <= p.table_width * p.block_size;
        if (ok && p.exit_planes != nullptr) {
          // every later read of exit_planes for this request lies in [offset, offset + e)
          const long long at = p.exit_offsets[r];
          ok = at >= 0 && at + e <= p.exit_count;
        }
        if (ok) {
          nb = (e - 1) / p.block_size - b / p.block_size + 1;
        } else {
          report(p.status, RLT_STATUS_BAD_RANGE, r, b, e);
        }
        nt = e - b;  // a skipped request still owns its slot in the packed image
      }
    }
    const int sb = warp_inclusive_scan(nb), st = warp_inclusive_scan(nt);
    if (lane == 31) {
      warp_sum[0][warp] = sb;
      warp_sum[1][warp] = st;
    }
    __syncthreads();
    if (warp == 0) {
      const int vb = lane < kThreads / 32 ? warp_sum[0][lane] : 0;
      const int vt = lane < kThreads / 32 ? warp_sum[1][lane] : 0;
      const int ib = warp_inclusive_scan(vb), it = warp_inclusive_scan(vt);
      if (lane < kThreads / 32) {
        warp_sum[0][lane] = ib - vb;
        warp_sum[1][lane] = it - vt;
      }
    }
    __syncthreads();
    if (r < p.num_requests) {
      blk_off[r + 1] = carry[0] + warp_sum[0][warp] + sb;
      tok_off[r + 1] = carry[1] + warp_sum[1][warp] + st;
    }
    __syncthreads();
    if (threadIdx.x == kThreads - 1) {
      carry[0] += warp_sum[0][warp] + sb;
      carry[1] += warp_sum[1][warp] + st;
    }
    __syncthreads();
  }
}

// One work unit, decoded from its flat index.
struct Unit {
  int r, plane, g, kv, logical;
  int begin, end;      // token range of the request
  int tok_lo, n_tok;   // tokens of this block that lie in the range
  int layer0, n_layers;
  int rows;            // n_layers * tokens carried by this unit
  int blk_first, n_blk;             // first flat block index and block count of the request
  unsigned long long sel_mask;      // dedup pack: tokens of the block whose exit plane reaches this plane
  int n_sel;
};

// Bit i set: token tok_lo + i of request r exits at or beyond `plane`, so `plane` holds a row of its own for it.
__device__ __forceinline__ unsigned long long exit_mask(const TableCopyParams& p, int r, int tok_lo, int n_tok, int plane) {
  unsigned long long mask = 0;
  const int* e = p.exit_planes + p.exit_offsets[r] + tok_lo;
  for (int i = 0; i < n_tok; ++i) mask |= static_cast<unsigned long long>(e[i] >= plane) << i;
  return mask;
}

// Position of the k-th (0-based) set bit of mask.
__device__ __forceinline__ int nth_set_bit(unsigned long long mask, int k) {
  const unsigned lo = static_cast<unsigned>(mask), hi = static_cast<unsigned>(mask >> 32);
  const int in_lo = __popc(lo);
  return k < in_lo ? static_cast<int>(__fns(lo, 0, k + 1)) : 32 + static_cast<int>(__fns(hi, 0, k - in_lo + 1));
}

__device__ __forceinline__ int units_per_plane(const TableCopyParams& p) {
  int n = 0;
  for (int g = 0; g < p.num_regions; ++g) n += 2 * p.region[g].chunks;
  return n;
}

template <bool kDedup>
__device__ __forceinline__ Unit decode_unit(const TableCopyParams& p, const int* blk_off, long long w,
                                            int per_plane, int per_block) {
  Unit u;
  const int blk_idx = static_cast<int>(w / per_block);
  int sub = static_cast<int>(w - static_cast<long long>(blk_idx) * per_block);
  const int plane_rel = sub / per_plane;
  sub -= plane_rel * per_plane;
  u.plane = p.plane_begin + plane_rel;
  u.g = 0;
  if (sub >= 2 * p.region[0].chunks) {
    u.g = 1;
    sub -= 2 * p.region[0].chunks;
  }
  const RegionParams& rg = p.region[u.g];
  u.kv = sub / rg.chunks;
  const int chunk = sub - u.kv * rg.chunks;
  // Request that owns block blk_idx: last r with blk_off[r] <= blk_idx.
  int lo_r = 0, hi_r = p.num_requests;
  while (hi_r - lo_r > 1) {
    const int mid = (lo_r + hi_r) >> 1;
    if (blk_off[mid] <= blk_idx) lo_r = mid; else hi_r = mid;
  }
  u.r = lo_r;
  u.begin = p.tok_begin[u.r];
  u.end = p.tok_end[u.r];
  u.logical = u.begin / p.block_size + (blk_idx - blk_off[u.r]);
  u.tok_lo = max(u.begin, u.logical * p.block_size);
  u.n_tok = min(u.end, (u.logical + 1) * p.block_size) - u.tok_lo;
  u.layer0 = p.layer_begin + chunk * rg.layers_per_unit;
  u.n_layers = min(rg.layers_per_unit, p.layer_end - u.layer0);
  u.blk_first = blk_off[u.r];
  u.n_blk = blk_off[u.r + 1] - u.blk_first;
  u.sel_mask = 0;
  u.n_sel = u.n_tok;
  if (kDedup && (p.dst_packed || p.fan)) {
    u.sel_mask = exit_mask(p, u.r, u.tok_lo, u.n_tok, u.plane);
    // Fan-out: every token has a row on plane 0, so an exit plane below 0 is seen (and reported) there.
    if (p.fan && !p.src_packed && u.plane == 0) u.sel_mask = u.n_tok >= 64 ? ~0ull : (1ull << u.n_tok) - 1ull;
    u.n_sel = __popcll(u.sel_mask);
  }
  u.rows = u.n_layers * u.n_sel;
  return u;
}

// Byte offsets (from the unit's source and destination tensor bases) of row `row` of a unit.
// This is where block tables and exit planes are read. A row that must be skipped gets -1 / -1.
template <bool kDedup>
__device__ __forceinline__ void row_offsets(const TableCopyParams& p, const Unit& u, const int* tok_off, int row,
                                            long long* src_off, long long* dst_off) {
  const RegionParams& rg = p.region[u.g];
  const int l_rel = row / u.n_sel;
  int tok = row - l_rel * u.n_sel;  // index among the unit's carried tokens
  const int layer = u.layer0 + l_rel;
  const int slice_layers = p.layer_end - p.layer_begin;
  long long so = -1, dof = -1;
  // Packed image: request, plane, block, region, tensor, layer, token (reference walk order).
  long long packed = 0;
  bool ok = true;
  if (kDedup) {
    // Only rows whose plane is not deeper than the token's exit plane are on the wire. The wire
    // plane of this row, the tokens of the block that plane carries, and this token's rank among them:
    int wire_plane = u.plane, rank = tok, carried = u.n_sel;
    if (p.dst_packed) {
      tok = nth_set_bit(u.sel_mask, rank);
    } else {
      int e = p.exit_planes[p.exit_offsets[u.r] + u.tok_lo + tok];
      if (e < 0) {  // such a token has no row on the wire; index as plane 0 and skip it
        report(p.status, RLT_STATUS_BAD_PLANE, u.r, u.tok_lo + tok, e);
        ok = false;
        e = 0;
      }
      wire_plane = min(u.plane, e);
      const unsigned long long mask = exit_mask(p, u.r, u.tok_lo, u.n_tok, wire_plane);
      carried = __popcll(mask);
      rank = __popcll(mask & ((1ull << tok) - 1ull));
    }
    const int entry = p.src_planes * u.blk_first + wire_plane * u.n_blk + (u.logical - u.begin / p.block_size);
    packed = static_cast<long long>(p.dedup_prefix[entry]) * p.packed_token_bytes;
    if (u.g == 1) packed += 2ll * slice_layers * carried * p.region[0].token_bytes;
    packed += (static_cast<long long>(u.kv) * slice_layers * carried +
               static_cast<long long>(layer - p.layer_begin) * carried + rank) * rg.token_bytes;
  } else if (p.src_packed | p.dst_packed) {
    const long long n_req = u.end - u.begin;
    packed = (static_cast<long long>(tok_off[u.r]) * p.dst_planes + static_cast<long long>(u.plane) * n_req +
              (u.tok_lo - u.begin)) * p.packed_token_bytes;
    if (u.g == 1) packed += 2ll * slice_layers * u.n_tok * p.region[0].token_bytes;
    packed += (static_cast<long long>(u.kv) * slice_layers * u.n_tok +
               static_cast<long long>(layer - p.layer_begin) * u.n_tok + tok) * rg.token_bytes;
  }
  const int t_abs = u.tok_lo + tok;
  if (p.src_packed | p.dst_packed) {
    if (packed + rg.token_bytes > p.packed_bytes) {
      report(p.status, RLT_STATUS_BAD_RANGE, u.r, u.begin, u.end);
      ok = false;
    }
  }
  if (p.deep_layer_mask != 0 && u.plane > 0 && !((p.deep_layer_mask >> layer) & 1ull)) ok = false;  // not carried
  const long long in_block = layer * rg.layer_bytes + (t_abs - u.logical * p.block_size) * rg.token_bytes;
  if (p.src_packed) {
    so = packed;
  } else {
    int exit_plane = p.src_planes - 1;
    if (p.exit_planes != nullptr) {
      exit_plane = p.exit_planes[p.exit_offsets[u.r] + t_abs];
      if (exit_plane < 0 || exit_plane >= p.src_planes) {
        report(p.status, RLT_STATUS_BAD_PLANE, u.r, t_abs, exit_plane);
        ok = false;
        exit_plane = 0;
      }
    }
    const int sp = min(u.plane + p.plane_bias, exit_plane);
    const int sb = p.src_tables[(static_cast<long long>(u.r) * p.src_planes + sp) * p.table_width + u.logical];
    if (sb < 0 || sb >= p.src_blocks) {
      report(p.status, RLT_STATUS_BAD_BLOCK, u.r, u.logical, sb);
      ok = false;
    }
    so = sb * rg.block_bytes + in_block;
  }
  if (p.dst_packed) {
    dof = packed;
  } else {
    const int db = p.dst_tables[(static_cast<long long>(u.r) * p.dst_planes + u.plane) * p.table_width + u.logical];
    if (db < 0 || db >= p.dst_blocks) {
      report(p.status, RLT_STATUS_BAD_BLOCK, u.r, u.logical, db);
      ok = false;
    }
    dof = db * rg.block_bytes + in_block;
  }
  *src_off = ok ? so : -1;
  *dst_off = ok ? dof : -1;
}

__device__ __forceinline__ const char* unit_src(const TableCopyParams& p, const Unit& u) {
  const RegionParams& rg = p.region[u.g];
  return p.src_packed ? rg.src_key : (u.kv ? rg.src_value : rg.src_key);
}

__device__ __forceinline__ char* unit_dst(const TableCopyParams& p, const Unit& u) {
  const RegionParams& rg = p.region[u.g];
  return p.dst_packed ? rg.dst_key : (u.kv ? rg.dst_value : rg.dst_key);
}

template <int kUnroll, bool kStreaming, bool kDedup, bool kWide = false>
__global__ void __launch_bounds__(kThreads, 4) table_copy_kernel(const TableCopyParams p) {
  extern __shared__ int dyn_smem[];
  int* blk_off = dyn_smem;                       // [num_requests + 1]
  int* tok_off = dyn_smem + p.num_requests + 1;  // [num_requests + 1]
  __shared__ long long row_src[2][kMaxRows];
  __shared__ long long row_dst[2][kMaxRows];

  scan_requests<kThreads>(p, blk_off, tok_off);

  const int per_plane = units_per_plane(p);
  const int per_block = per_plane * p.plane_count;
  const long long total_units = static_cast<long long>(blk_off[p.num_requests]) * per_block;

  int parity = 0;
  for (long long w = blockIdx.x; w < total_units; w += gridDim.x, parity ^= 1) {
    const Unit u = decode_unit<kDedup>(p, blk_off, w, per_plane, per_block);
    const RegionParams& rg = p.region[u.g];
    long long* rs = row_src[parity];
    long long* rd = row_dst[parity];
    if (threadIdx.x < u.rows) row_offsets<kDedup>(p, u, tok_off, threadIdx.x, &rs[threadIdx.x], &rd[threadIdx.x]);
    // A token with a negative exit plane has no row in a dedup wire image, so no row above sees it: one unit per
    // block looks (the scatter of such an image does the same in table_fan_kernel).
    if (kDedup && p.dst_packed && u.plane == p.plane_begin && u.g == 0 && u.kv == 0 && u.layer0 == p.layer_begin &&
        static_cast<int>(threadIdx.x) < u.n_tok) {
      const int t_abs = u.tok_lo + static_cast<int>(threadIdx.x);
      const int e = p.exit_planes[p.exit_offsets[u.r] + t_abs];
      if (e < 0) report(p.status, RLT_STATUS_BAD_PLANE, u.r, t_abs, e);
    }
    __syncthreads();  // one barrier per unit: the offset tables are double buffered

    const char* src = unit_src(p, u);
    char* dst = unit_dst(p, u);
    const int total_vecs = u.rows * rg.row_vecs;
    if (kWide && rg.wide_ok) {
      const int wide_vecs = rg.row_vecs >> 1;
      const unsigned wide_magic = wide_vecs == 1 ? 0u : static_cast<unsigned>((1ull << 32) / wide_vecs) + 1u;
      stream_rows<Vec32, kUnroll, true>(src, dst, rs, rd, u.rows * wide_vecs, wide_vecs, wide_magic);
    } else if (rg.vec_bytes == 16) {
      stream_rows<uint4, kUnroll, kStreaming>(src, dst, rs, rd, total_vecs, rg.row_vecs, rg.row_magic);
    } else if (rg.vec_bytes == 4) {
      stream_rows<uint32_t, kUnroll, kStreaming>(src, dst, rs, rd, total_vecs, rg.row_vecs, rg.row_magic);
    } else {
      stream_rows<uint8_t, kUnroll, kStreaming>(src, dst, rs, rd, total_vecs, rg.row_vecs, rg.row_magic);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Fan-out flavour of the dedup handoff and of the dedup scatter. The destination of RLT_MODE_DEDUP holds, on every
// plane deeper than a token's exit plane, a copy of the exit-plane row. The kernel above produces that by
// walking destination planes, which reads the exit-plane row once per plane it fills. Here the walk is over
// SOURCE planes: the unit of plane q loads the rows of the tokens that reach q (exit plane >= q) once,
// stores them to plane q, and stores the rows of the tokens that stop at q to every deeper plane as well.
// Bytes read = the dedup wire image, bytes written = the full destination; with the source behind a peer
// pointer only the wire image crosses the link. The scatter of a dedup wire image is the same walk with the
// rows of plane q taken from the image (they are stored there compacted, plane by plane) instead of a pool.
constexpr long long kFanBit = 1ll << 62;          // in a destination offset: the row also goes to the deeper planes
constexpr long long kNoPlane = -(1ll << 62);      // in a plane delta: that plane's block is invalid, skip it
constexpr int kFanMaxPlanes = 64;

template <typename T, int kUnroll>
__device__ __forceinline__ void stream_rows_fan(const char* __restrict__ src, char* __restrict__ dst,
                                                const long long* __restrict__ src_off,
                                                const long long* __restrict__ dst_off,
                                                const long long* __restrict__ plane_delta, int fan_begin,
                                                int fan_end, int total_vecs, int row_vecs, unsigned row_magic) {
  for (int base = threadIdx.x; base < total_vecs; base += kThreads * kUnroll) {
    T regs[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total_vecs) {
        const int row = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        const long long so = src_off[row];
        if (so >= 0) regs[u] = ld_stream(reinterpret_cast<const T*>(src + so) + (i - row * row_vecs));
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int i = base + u * kThreads;
      if (i < total_vecs) {
        const int row = row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i;
        long long to = dst_off[row];
        if (to >= 0) {
          const bool fan = (to & kFanBit) != 0;
          to &= ~kFanBit;
          char* at = dst + to + static_cast<long long>(i - row * row_vecs) * static_cast<long long>(sizeof(T));
          st_stream(reinterpret_cast<T*>(at), regs[u]);
          if (fan) {
            for (int pl = fan_begin; pl < fan_end; ++pl) {
              const long long d = plane_delta[pl];
              if (d != kNoPlane) st_stream(reinterpret_cast<T*>(at + d), regs[u]);
            }
          }
        }
      }
    }
  }
}

// Offsets of row `row` of a fan-out unit; the unit's rows are (layer, token that reaches the unit's plane).
__device__ __forceinline__ void fan_row_offsets(const TableCopyParams& p, const Unit& u, int row,
                                                long long* src_off, long long* dst_off) {
  const RegionParams& rg = p.region[u.g];
  const int l_rel = row / u.n_sel;
  const int rank = row - l_rel * u.n_sel;
  const int tok = nth_set_bit(u.sel_mask, rank);
  const int layer = u.layer0 + l_rel;
  const int t_abs = u.tok_lo + tok;
  const bool deep_ok = p.deep_layer_mask == 0 || ((p.deep_layer_mask >> layer) & 1ull) != 0;
  bool ok = u.plane == 0 || deep_ok;  // planes >= 1 carry only the deep layers
  const int e = p.exit_planes[p.exit_offsets[u.r] + t_abs];
  if (e < 0 || e >= p.src_planes) {
    report(p.status, RLT_STATUS_BAD_PLANE, u.r, t_abs, e);
    ok = false;
  }
  const long long in_block = layer * rg.layer_bytes + (t_abs - u.logical * p.block_size) * rg.token_bytes;
  long long so;
  if (p.src_packed) {
    // The wire image holds this plane's rows of the block compacted: same walk order as the pack side.
    const int slice_layers = p.layer_end - p.layer_begin;
    const int entry = p.src_planes * u.blk_first + u.plane * u.n_blk + (u.logical - u.begin / p.block_size);
    so = static_cast<long long>(p.dedup_prefix[entry]) * p.packed_token_bytes;
    if (u.g == 1) so += 2ll * slice_layers * u.n_sel * p.region[0].token_bytes;
    so += (static_cast<long long>(u.kv) * slice_layers * u.n_sel +
           static_cast<long long>(layer - p.layer_begin) * u.n_sel + rank) * rg.token_bytes;
    if (so + rg.token_bytes > p.packed_bytes) {
      report(p.status, RLT_STATUS_BAD_RANGE, u.r, u.begin, u.end);
      ok = false;
    }
  } else {
    const int sb = p.src_tables[(static_cast<long long>(u.r) * p.src_planes + u.plane) * p.table_width + u.logical];
    if (sb < 0 || sb >= p.src_blocks) {
      report(p.status, RLT_STATUS_BAD_BLOCK, u.r, u.logical, sb);
      ok = false;
    }
    so = sb * rg.block_bytes + in_block;
  }
  const int db = p.dst_tables[(static_cast<long long>(u.r) * p.dst_planes + u.plane) * p.table_width + u.logical];
  if (db < 0 || db >= p.dst_blocks) {
    report(p.status, RLT_STATUS_BAD_BLOCK, u.r, u.logical, db);
    ok = false;
  }
  long long dof = db * rg.block_bytes + in_block;
  if (e == u.plane && u.plane + 1 < p.dst_planes && deep_ok) dof |= kFanBit;
  *src_off = ok ? so : -1;
  *dst_off = ok ? dof : -1;
}

template <int kUnroll>
__global__ void __launch_bounds__(kThreads, 3) table_fan_kernel(const TableCopyParams p) {
  extern __shared__ int dyn_smem[];
  int* blk_off = dyn_smem;
  int* tok_off = dyn_smem + p.num_requests + 1;
  __shared__ long long row_src[2][kMaxRows];
  __shared__ long long row_dst[2][kMaxRows];
  __shared__ long long plane_delta[2][kFanMaxPlanes];

  scan_requests<kThreads>(p, blk_off, tok_off);

  const int per_plane = units_per_plane(p);
  const int per_block = per_plane * p.plane_count;
  const long long total_units = static_cast<long long>(blk_off[p.num_requests]) * per_block;

  int parity = 0;
  for (long long w = blockIdx.x; w < total_units; w += gridDim.x, parity ^= 1) {
    const Unit u = decode_unit<true>(p, blk_off, w, per_plane, per_block);
    const RegionParams& rg = p.region[u.g];
    long long* rs = row_src[parity];
    long long* rd = row_dst[parity];
    long long* pd = plane_delta[parity];
    if (threadIdx.x < u.rows) fan_row_offsets(p, u, threadIdx.x, &rs[threadIdx.x], &rd[threadIdx.x]);
    // A token with a negative exit plane has no row in a wire image, so no row above sees it: one unit per block looks.
    if (p.src_packed && u.plane == 0 && u.g == 0 && u.kv == 0 && u.layer0 == p.layer_begin &&
        static_cast<int>(threadIdx.x) < u.n_tok) {
      const int t_abs = u.tok_lo + static_cast<int>(threadIdx.x);
      const int e = p.exit_planes[p.exit_offsets[u.r] + t_abs];
      if (e < 0) report(p.status, RLT_STATUS_BAD_PLANE, u.r, t_abs, e);
    }
    // Threads of the back of the CTA fetch the deeper planes' blocks, as byte distances from this plane's block.
    const int pl = kThreads - 1 - static_cast<int>(threadIdx.x);
    if (u.rows > 0 && pl > u.plane && pl < p.dst_planes) {
      const long long row_base = static_cast<long long>(u.r) * p.dst_planes;
      const int here = p.dst_tables[(row_base + u.plane) * p.table_width + u.logical];
      const int there = p.dst_tables[(row_base + pl) * p.table_width + u.logical];
      long long d = kNoPlane;
      if (there < 0 || there >= p.dst_blocks) {
        report(p.status, RLT_STATUS_BAD_BLOCK, u.r, u.logical, there);
      } else {
        d = (static_cast<long long>(there) - here) * rg.block_bytes;
      }
      pd[pl] = d;
    }
    __syncthreads();  // one barrier per unit: all three tables are double buffered

    const char* src = unit_src(p, u);
    char* dst = unit_dst(p, u);
    const int total_vecs = u.rows * rg.row_vecs;
    if (rg.vec_bytes == 16) {
      stream_rows_fan<uint4, kUnroll>(src, dst, rs, rd, pd, u.plane + 1, p.dst_planes, total_vecs, rg.row_vecs, rg.row_magic);
    } else if (rg.vec_bytes == 4) {
      stream_rows_fan<uint32_t, kUnroll>(src, dst, rs, rd, pd, u.plane + 1, p.dst_planes, total_vecs, rg.row_vecs, rg.row_magic);
    } else {
      stream_rows_fan<uint8_t, kUnroll>(src, dst, rs, rd, pd, u.plane + 1, p.dst_planes, total_vecs, rg.row_vecs, rg.row_magic);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Bulk-copy flavour: the same walk, but rows move global -> shared -> global with cp.async.bulk
// (the TMA unit's untiled copy), tracked by mbarriers, instead of through registers.
//
// Every warp is an independent worker with a private ring of kBulkStages shared-memory stages.
// All 32 lanes decode units and compute row offsets (32 rows at a time); lane 0 merges rows that
// are adjacent on both sides into jobs of at most kBulkStageBytes and drives the ring:
//     load(job k) ... wait full[k - kBulkLag] ; store(job k - kBulkLag)
// so kBulkLag loads are in flight per warp while earlier stores drain. A stage is reused only
// after cp.async.bulk.wait_group.read has confirmed that the store which last used it has read
// it. Regions whose rows are too small or not 16-byte multiples (scale rows) are copied by the
// warp with ordinary loads and stores. Every bulk copy is a plain one-CTA copy, and every wait
// on an mbarrier is bounded: if a load never lands the warp records RLT_STATUS_STALL and stops.
constexpr int kBulkWarps = 6;
constexpr int kBulkThreads = kBulkWarps * 32;
constexpr int kBulkMinRow = 512;
constexpr int kBulkWarpBytes = 32768;  // shared memory of one warp's ring: stages x stage bytes
constexpr size_t kBulkStageTotal = static_cast<size_t>(kBulkWarps) * kBulkWarpBytes;

template <int kBulkStages>
struct BulkRing {
  unsigned long long full[kBulkStages];  // mbarriers: "the load into this stage has landed"
  unsigned long long dst[kBulkStages];   // destination address of the job parked in the stage
  int bytes[kBulkStages];
  int pad[kBulkStages];
};

__device__ __forceinline__ unsigned smem_addr(const void* p) {
  return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// Bounded wait for the phase with the given parity; false if it never completed.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, int parity) {
  const unsigned addr = smem_addr(bar);
  for (int spin = 0; spin < (1 << 22); ++spin) {
    unsigned done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, int bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, int bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst), "r"(smem_addr(smem_src)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

template <int kBulkStages>
struct BulkWorker {
  static constexpr int kBulkStageBytes = kBulkWarpBytes / kBulkStages;
  static constexpr int kBulkLag = kBulkStages - 2;
  BulkRing<kBulkStages>* ring;
  unsigned char* stages;  // kBulkStages * kBulkStageBytes of this warp
  long long issued = 0;   // jobs whose load was issued
  bool dead = false;

  __device__ __forceinline__ unsigned char* stage(int s) const { return stages + static_cast<size_t>(s) * kBulkStageBytes; }

  // Complete job k: its load has landed, send it on.
  __device__ __forceinline__ void finish(long long k) {
    const int s = static_cast<int>(k % kBulkStages);
    if (!mbar_wait(&ring->full[s], static_cast<int>((k / kBulkStages) & 1))) {
      dead = true;
      return;
    }
    bulk_store(reinterpret_cast<void*>(ring->dst[s]), stage(s), ring->bytes[s]);
  }

  __device__ __forceinline__ void emit(const char* src, char* dst, int bytes) {
    if (dead) return;
    const int s = static_cast<int>(issued % kBulkStages);
    if (issued >= kBulkStages) {
      // The store of job issued - kBulkStages must have read the stage; one younger store may still be pending.
      asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBulkStages - kBulkLag - 1) : "memory");
    }
    ring->dst[s] = reinterpret_cast<unsigned long long>(dst);
    ring->bytes[s] = bytes;
    mbar_expect_tx(&ring->full[s], bytes);
    bulk_load(stage(s), src, bytes, &ring->full[s]);
    ++issued;
    if (issued > kBulkLag) finish(issued - 1 - kBulkLag);
  }

  __device__ __forceinline__ void drain() {
    const long long first = issued > kBulkLag ? issued - kBulkLag : 0;
    for (long long k = first; k < issued && !dead; ++k) finish(k);
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
};

template <typename T>
__device__ __forceinline__ void warp_copy_rows(const char* src, char* dst, long long so, long long dof, int count,
                                               int row_vecs, unsigned row_magic) {
  // Lane j holds the offsets of row j; the warp streams the count rows as one flat vector array.
  const int lane = threadIdx.x & 31;
  const int total = count * row_vecs;
  for (int i = lane; i < total + 31 - (total + 31) % 32; i += 32) {  // uniform trip count: shuffles need every lane
    const bool in = i < total;
    const int row = in ? (row_magic ? static_cast<int>(__umulhi(static_cast<unsigned>(i), row_magic)) : i) : 0;
    const long long s = __shfl_sync(0xffffffffu, so, row);
    const long long d = __shfl_sync(0xffffffffu, dof, row);
    if (in && s >= 0) {
      const int off = i - row * row_vecs;
      reinterpret_cast<T*>(dst + d)[off] = reinterpret_cast<const T*>(src + s)[off];
    }
  }
}

template <int kBulkStages, bool kDedup>
__global__ void __launch_bounds__(kBulkThreads, 1) table_bulk_kernel(const TableCopyParams p) {
  constexpr int kBulkStageBytes = kBulkWarpBytes / kBulkStages;
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  BulkRing<kBulkStages>* rings = reinterpret_cast<BulkRing<kBulkStages>*>(bulk_smem + kBulkStageTotal);
  int* blk_off = reinterpret_cast<int*>(rings + kBulkWarps);
  int* tok_off = blk_off + p.num_requests + 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  BulkWorker<kBulkStages> worker;
  worker.ring = &rings[warp];
  worker.stages = bulk_smem + static_cast<size_t>(warp) * kBulkWarpBytes;
  if (lane == 0) {
    for (int s = 0; s < kBulkStages; ++s) mbar_init(&worker.ring->full[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  scan_requests<kBulkThreads>(p, blk_off, tok_off);  // ends with __syncthreads: barriers are initialised for everyone

  const int per_plane = units_per_plane(p);
  const int per_block = per_plane * p.plane_count;
  const long long total_units = static_cast<long long>(blk_off[p.num_requests]) * per_block;
  const long long first = static_cast<long long>(blockIdx.x) * kBulkWarps + warp;
  const long long stride = static_cast<long long>(gridDim.x) * kBulkWarps;

  for (long long w = first; w < total_units; w += stride) {
    const Unit u = decode_unit<kDedup>(p, blk_off, w, per_plane, per_block);
    const RegionParams& rg = p.region[u.g];
    const char* src = unit_src(p, u);
    char* dst = unit_dst(p, u);
    const bool bulk = rg.vec_bytes == 16 && rg.token_bytes >= kBulkMinRow;
    const int row_bytes = static_cast<int>(rg.token_bytes);
    if (kDedup && p.dst_packed && u.plane == p.plane_begin && u.g == 0 && u.kv == 0 && u.layer0 == p.layer_begin) {
      for (int i = lane; i < u.n_tok; i += 32) {  // tokens without a row on the wire: see table_copy_kernel
        const int e = p.exit_planes[p.exit_offsets[u.r] + u.tok_lo + i];
        if (e < 0) report(p.status, RLT_STATUS_BAD_PLANE, u.r, u.tok_lo + i, e);
      }
    }
    long long run_s = 0, run_d = 0;
    int run_n = 0;
    for (int base = 0; base < u.rows; base += 32) {
      long long so = -1, dof = -1;
      if (base + lane < u.rows) row_offsets<kDedup>(p, u, tok_off, base + lane, &so, &dof);
      const int count = min(32, u.rows - base);
      if (!bulk) {
        if (rg.vec_bytes == 16) {
          warp_copy_rows<uint4>(src, dst, so, dof, count, rg.row_vecs, rg.row_magic);
        } else if (rg.vec_bytes == 4) {
          warp_copy_rows<uint32_t>(src, dst, so, dof, count, rg.row_vecs, rg.row_magic);
        } else {
          warp_copy_rows<uint8_t>(src, dst, so, dof, count, rg.row_vecs, rg.row_magic);
        }
        continue;
      }
      for (int j = 0; j < count; ++j) {
        const long long s_j = __shfl_sync(0xffffffffu, so, j);
        const long long d_j = __shfl_sync(0xffffffffu, dof, j);
        if (s_j < 0 || lane != 0) continue;
        for (int off = 0; off < row_bytes; off += kBulkStageBytes) {
          const int n = min(kBulkStageBytes, row_bytes - off);
          if (run_n > 0 && s_j + off == run_s + run_n && d_j + off == run_d + run_n && run_n + n <= kBulkStageBytes) {
            run_n += n;
          } else {
            if (run_n > 0) worker.emit(src + run_s, dst + run_d, run_n);
            run_s = s_j + off;
            run_d = d_j + off;
            run_n = n;
          }
        }
      }
    }
    if (lane == 0 && run_n > 0) worker.emit(src + run_s, dst + run_d, run_n);
    if (__shfl_sync(0xffffffffu, static_cast<int>(worker.dead), 0)) break;
  }
  if (lane == 0) {
    worker.drain();
    if (worker.dead) report(p.status, RLT_STATUS_STALL, static_cast<int>(blockIdx.x), warp, 0);
  }
}

// ---------------------------------------------------------------------------------------------
// Dedup wire plan: where each (request, plane, block) starts in a wire image that carries, for
// every token, only the planes up to its exit plane. Three small launches:
//   count : tokens carried per (request, plane, block) entry, and the sum of every 1024-entry tile
//   tiles : exclusive scan of the tile sums (one CTA); total wire tokens -> header
//   finish: exclusive scan inside every tile, offset by its tile start (in place over the counts)
// Entries are ordered request, plane, block - the wire order. All scans use warp shuffles.
// Workspace layout: int64 header[2] = {wire tokens, entries}; int32 prefix[entries]; int32 tile[tiles + 1].
constexpr int kPlanTile = 1024;
constexpr int kPlanHeaderBytes = 16;

__device__ __forceinline__ int block_exclusive_scan(int v, int* total) {
  // Exclusive scan of one value per thread across a kThreads-wide CTA.
  __shared__ int warp_part[kThreads / 32];
  __shared__ int all;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int inc = warp_inclusive_scan(v);
  if (lane == 31) warp_part[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    const int w = lane < kThreads / 32 ? warp_part[lane] : 0;
    const int iw = warp_inclusive_scan(w);
    if (lane < kThreads / 32) warp_part[lane] = iw - w;
    if (lane == kThreads / 32 - 1) all = iw;
  }
  __syncthreads();
  const int out = warp_part[warp] + inc - v;
  *total = all;
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(kThreads) dedup_count_kernel(const TableCopyParams p, long long* header, int* prefix,
                                                               int* tile_sum) {
  extern __shared__ int dyn_smem[];
  int* blk_off = dyn_smem;
  int* tok_off = dyn_smem + p.num_requests + 1;
  scan_requests<kThreads>(p, blk_off, tok_off);
  const long long entries = static_cast<long long>(p.src_planes) * blk_off[p.num_requests];
  if (blockIdx.x == 0 && threadIdx.x == 0) header[1] = entries;
  const long long tiles = (entries + kPlanTile - 1) / kPlanTile;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    int mine = 0;
    for (int k = 0; k < kPlanTile / kThreads; ++k) {
      const long long idx = tile * kPlanTile + k * kThreads + threadIdx.x;
      if (idx >= entries) continue;
      int lo_r = 0, hi_r = p.num_requests;
      while (hi_r - lo_r > 1) {
        const int mid = (lo_r + hi_r) >> 1;
        if (static_cast<long long>(p.src_planes) * blk_off[mid] <= idx) lo_r = mid; else hi_r = mid;
      }
      const int r = lo_r;
      const int n_blk = blk_off[r + 1] - blk_off[r];
      const int local = static_cast<int>(idx - static_cast<long long>(p.src_planes) * blk_off[r]);
      const int plane = local / n_blk;
      const int begin = p.tok_begin[r], end = p.tok_end[r];
      const int logical = begin / p.block_size + (local - plane * n_blk);
      const int lo = max(begin, logical * p.block_size);
      const int hi = min(end, (logical + 1) * p.block_size);
      const int count = __popcll(exit_mask(p, r, lo, hi - lo, plane));
      prefix[idx] = count;
      mine += count;
    }
    int total;
    block_exclusive_scan(mine, &total);
    if (threadIdx.x == 0) tile_sum[tile] = total;
  }
}

__global__ void __launch_bounds__(kThreads) dedup_tiles_kernel(long long* header, int* tile_sum) {
  const long long tiles = (header[1] + kPlanTile - 1) / kPlanTile;
  int carry = 0;
  for (long long base = 0; base < tiles; base += kThreads) {
    const long long i = base + threadIdx.x;
    const int v = i < tiles ? tile_sum[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, &total);
    if (i < tiles) tile_sum[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) {
    tile_sum[tiles] = carry;
    header[0] = carry;
  }
}

__global__ void __launch_bounds__(kThreads) dedup_finish_kernel(const long long* header, int* prefix, const int* tile_sum) {
  const long long entries = header[1];
  const long long tiles = (entries + kPlanTile - 1) / kPlanTile;
  constexpr int kPer = kPlanTile / kThreads;
  for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
    const long long first = tile * kPlanTile + static_cast<long long>(threadIdx.x) * kPer;
    int v[kPer], sum = 0;
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      v[k] = first + k < entries ? prefix[first + k] : 0;
      sum += v[k];
    }
    int total;
    int run = tile_sum[tile] + block_exclusive_scan(sum, &total);
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      if (first + k < entries) prefix[first + k] = run;
      run += v[k];
    }
  }
}

long long dedup_workspace_bytes(long long requests, long long width, long long planes) {
  const long long entries = requests * width * planes;
  const long long tiles = (entries + kPlanTile - 1) / kPlanTile;
  return kPlanHeaderBytes + 4 * entries + 4 * (tiles + 1);
}

// Launch the three plan kernels into `workspace`; fills p.dedup_prefix.
int plan_dedup(TableCopyParams& p, void* workspace, long long workspace_bytes, int sms, size_t scan_smem,
               cudaStream_t stream) {
  if (workspace == nullptr) return RLT_E_INVALID;
  if (reinterpret_cast<uintptr_t>(workspace) & 15u) return RLT_E_ALIGN;
  const long long entries_max = static_cast<long long>(p.num_requests) * p.table_width * p.src_planes;
  if (workspace_bytes < dedup_workspace_bytes(p.num_requests, p.table_width, p.src_planes)) return RLT_E_LIMIT;
  long long* header = static_cast<long long*>(workspace);
  int* prefix = reinterpret_cast<int*>(static_cast<char*>(workspace) + kPlanHeaderBytes);
  int* tile_sum = prefix + entries_max;
  const long long tiles_max = (entries_max + kPlanTile - 1) / kPlanTile;
  const int grid = static_cast<int>(tiles_max < sms * 4ll ? tiles_max : sms * 4ll);
  dedup_count_kernel<<<grid, kThreads, scan_smem, stream>>>(p, header, prefix, tile_sum);
  dedup_tiles_kernel<<<1, kThreads, 0, stream>>>(header, tile_sum);
  dedup_finish_kernel<<<grid, kThreads, 0, stream>>>(header, prefix, tile_sum);
  RLT_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(3, std::memory_order_relaxed);
  p.dedup_prefix = prefix;
  return RLT_OK;
}

bool dense(const RltRegion& r, const RltPool& pool) {
  return r.token_bytes > 0 && r.layer_bytes == r.token_bytes * pool.block_size &&
         r.block_bytes == r.layer_bytes * pool.num_layers;
}

int vector_width(const void* a, const void* b, const void* c, const void* d, long long token_bytes) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                         reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d) |
                         static_cast<uintptr_t>(token_bytes);
  if ((bits & 15u) == 0) return 16;
  if ((bits & 3u) == 0) return 4;
  return 1;
}

enum Direction { kDirect, kPack, kScatter };

int launch_table_copy(Direction dir, const RltPool* src, const RltPool* dst, const RltBatch* batch,
                      const RltOptions* opt, void* packed, long long packed_bytes, cudaStream_t stream,
                      void* workspace = nullptr, long long workspace_bytes = 0) {
  const NvtxRange range(dir == kDirect ? "rlt.kv_handoff" : dir == kPack ? "rlt.kv_pack" : "rlt.kv_scatter");
  if (batch == nullptr || opt == nullptr) return RLT_E_INVALID;
  if (workspace == nullptr) {
    workspace = opt->workspace;
    workspace_bytes = opt->workspace_bytes;
  }
  const RltPool* any = dir == kScatter ? dst : src;
  if (any == nullptr || (dir == kDirect && dst == nullptr)) return RLT_E_INVALID;
  if (batch->num_requests < 1 || batch->table_width < 1 || batch->tok_begin == nullptr ||
      batch->tok_end == nullptr)
    return RLT_E_INVALID;
  if (batch->num_requests > RLT_MAX_REQUESTS) return RLT_E_LIMIT;
  if (any->block_size < 1 || any->block_size > kMaxBlockSize) return RLT_E_LIMIT;
  if (any->num_layers < 1 || any->num_planes < 1 || any->num_blocks < 1) return RLT_E_INVALID;
  if (dir != kScatter && batch->src_tables == nullptr) return RLT_E_INVALID;
  if (dir != kPack && batch->dst_tables == nullptr) return RLT_E_INVALID;
  if (opt->mode < RLT_MODE_ALL_PLANES || opt->mode > RLT_MODE_EXIT_ONLY) return RLT_E_INVALID;
  if (opt->mode != RLT_MODE_ALL_PLANES && dir != kScatter &&
      (batch->exit_planes == nullptr || batch->exit_offsets == nullptr))
    return RLT_E_INVALID;
  const bool dedup_wire = dir != kDirect && opt->mode == RLT_MODE_DEDUP;
  if (dedup_wire && (batch->exit_planes == nullptr || batch->exit_offsets == nullptr)) return RLT_E_INVALID;
  if (batch->exit_planes != nullptr && batch->exit_count < 1) return RLT_E_INVALID;

  const int layer_begin = opt->layer_begin;
  const int layer_end = opt->layer_end == 0 ? any->num_layers : opt->layer_end;
  if (layer_begin < 0 || layer_end <= layer_begin || layer_end > any->num_layers) return RLT_E_INVALID;

  const bool scales = any->scales.key != nullptr;
  if (scales && any->scales.value == nullptr) return RLT_E_INVALID;
  if (any->codes.key == nullptr || any->codes.value == nullptr) return RLT_E_INVALID;
  if (!dense(any->codes, *any) || (scales && !dense(any->scales, *any))) return RLT_E_GEOMETRY;
  if (dir == kDirect) {
    if (dst->codes.key == nullptr || dst->codes.value == nullptr) return RLT_E_INVALID;
    if ((dst->scales.key != nullptr) != scales) return RLT_E_GEOMETRY;
    if (scales && dst->scales.value == nullptr) return RLT_E_INVALID;
    if (dst->block_size != src->block_size || dst->num_layers != src->num_layers ||
        dst->codes.token_bytes != src->codes.token_bytes || !dense(dst->codes, *dst) ||
        dst->num_blocks < 1 || dst->num_planes < 1)
      return RLT_E_GEOMETRY;
    if (scales && (dst->scales.token_bytes != src->scales.token_bytes || !dense(dst->scales, *dst)))
      return RLT_E_GEOMETRY;
  }

  TableCopyParams p{};
  p.num_regions = scales ? 2 : 1;
  p.num_requests = batch->num_requests;
  p.table_width = batch->table_width;
  p.block_size = any->block_size;
  p.src_tables = batch->src_tables;
  p.dst_tables = batch->dst_tables;
  p.tok_begin = batch->tok_begin;
  p.tok_end = batch->tok_end;
  p.exit_planes = opt->mode == RLT_MODE_ALL_PLANES ? nullptr : batch->exit_planes;
  p.exit_offsets = reinterpret_cast<const long long*>(batch->exit_offsets);
  p.exit_count = batch->exit_count;
  p.layer_begin = layer_begin;
  p.layer_end = layer_end;
  p.status = opt->status;
  p.src_packed = dir == kScatter;
  p.dst_packed = dir == kPack;

  int wire_planes = opt->wire_planes;
  if (dir == kDirect) {
    p.src_planes = src->num_planes;
    p.dst_planes = dst->num_planes;
    p.src_blocks = src->num_blocks;
    p.dst_blocks = dst->num_blocks;
    if (opt->mode == RLT_MODE_EXIT_ONLY) {
      if (dst->num_planes != 1) return RLT_E_GEOMETRY;
    } else if (dst->num_planes != src->num_planes) {
      return RLT_E_GEOMETRY;
    }
  } else if (dir == kPack) {
    if (wire_planes == 0) wire_planes = opt->mode == RLT_MODE_EXIT_ONLY ? 1 : src->num_planes;
    if (opt->mode == RLT_MODE_EXIT_ONLY ? wire_planes != 1 : wire_planes != src->num_planes)
      return RLT_E_GEOMETRY;
    p.src_planes = src->num_planes;
    p.dst_planes = wire_planes;
    p.src_blocks = src->num_blocks;
  } else {
    if (wire_planes == 0) wire_planes = dst->num_planes;
    if (wire_planes != dst->num_planes) return RLT_E_GEOMETRY;
    p.src_planes = wire_planes;
    p.dst_planes = dst->num_planes;
    p.dst_blocks = dst->num_blocks;
    p.exit_planes = dedup_wire ? batch->exit_planes : nullptr;
  }
  p.plane_bias = opt->mode == RLT_MODE_EXIT_ONLY ? p.src_planes : 0;
  p.plane_begin = opt->plane_begin;
  const int plane_end = opt->plane_end == 0 ? p.dst_planes : opt->plane_end;
  if (p.plane_begin < 0 || plane_end <= p.plane_begin || plane_end > p.dst_planes) return RLT_E_INVALID;
  p.plane_count = plane_end - p.plane_begin;
  if (opt->deep_layer_mask != 0) {
    if (dir != kDirect || any->num_layers > 64) return RLT_E_INVALID;
    p.deep_layer_mask = opt->deep_layer_mask;
  }

  const int slice_layers = layer_end - layer_begin;
  const long long row_total = any->codes.token_bytes + (scales ? any->scales.token_bytes : 0);
  p.packed_token_bytes = 2ll * slice_layers * row_total;
  if (dir != kDirect) {
    if (packed == nullptr) return RLT_E_INVALID;
    if (reinterpret_cast<uintptr_t>(packed) & 15u) return RLT_E_ALIGN;
    if (packed_bytes < 0) return RLT_E_INVALID;
    p.packed_bytes = packed_bytes;
  }

  const int unit_kib = (opt->variant >> 4) & 0xff;
  // 128 KiB of rows per unit; a dedup pack carries only the tokens that reach a unit's plane (5/8 of a block on
  // average with uniform exits), so its units are sized at twice that (measured: 0.94 -> 0.97 of the HBM copy peak;
  // the same change costs the other launches 2 - 4 %).
  const long long unit_default = dedup_wire && dir == kPack ? 262144ll : 131072ll;
  const long long unit_target = unit_kib ? unit_kib * 16384ll : unit_default;
  for (int g = 0; g < p.num_regions; ++g) {
    const RltRegion& s = g == 0 ? any->codes : any->scales;
    RegionParams& rg = p.region[g];
    rg.block_bytes = s.block_bytes;
    rg.layer_bytes = s.layer_bytes;
    rg.token_bytes = s.token_bytes;
    if (dir == kScatter) {
      rg.src_key = rg.src_value = static_cast<const char*>(packed);
    } else {
      const RltRegion& sr = g == 0 ? src->codes : src->scales;
      rg.src_key = static_cast<const char*>(sr.key);
      rg.src_value = static_cast<const char*>(sr.value);
    }
    if (dir == kPack) {
      rg.dst_key = rg.dst_value = static_cast<char*>(packed);
    } else {
      const RltRegion& dr = g == 0 ? dst->codes : dst->scales;
      rg.dst_key = static_cast<char*>(dr.key);
      rg.dst_value = static_cast<char*>(dr.value);
    }
    // The packed offset of a scale row is a multiple of the scale row size plus a multiple of
    // the code row size, so both row sizes bound the vector width of a packed-side region.
    long long align_bytes = s.token_bytes;
    if (dir != kDirect && scales) align_bytes |= any->codes.token_bytes | any->scales.token_bytes;
    rg.vec_bytes = vector_width(rg.src_key, rg.src_value, rg.dst_key, rg.dst_value, align_bytes);
    rg.row_vecs = static_cast<int>(s.token_bytes / rg.vec_bytes);
    rg.wide_ok = ((reinterpret_cast<uintptr_t>(rg.src_key) | reinterpret_cast<uintptr_t>(rg.src_value) |
                   reinterpret_cast<uintptr_t>(rg.dst_key) | reinterpret_cast<uintptr_t>(rg.dst_value) |
                   static_cast<uintptr_t>(align_bytes)) & 31u) == 0;
    rg.row_magic = rg.row_vecs == 1 ? 0u : div_magic(static_cast<uint32_t>(rg.row_vecs));
    long long lpu = unit_target / (s.token_bytes * any->block_size);
    if (lpu < 1) lpu = 1;
    if (lpu > slice_layers) lpu = slice_layers;
    if (lpu * any->block_size > kMaxRows) lpu = kMaxRows / any->block_size;
    // __umulhi row split is exact while (vector index) * row_vecs < 2^32.
    while (lpu > 1 && lpu * any->block_size * rg.row_vecs * static_cast<long long>(rg.row_vecs) >= (1ll << 32)) --lpu;
    if (lpu * any->block_size * rg.row_vecs * static_cast<long long>(rg.row_vecs) >= (1ll << 32)) return RLT_E_LIMIT;
    rg.layers_per_unit = static_cast<int>(lpu);
    rg.chunks = (slice_layers + rg.layers_per_unit - 1) / rg.layers_per_unit;
  }
  if (p.num_regions == 1) p.region[1].chunks = 0;

  int sms = 0;
  const int rc = sm_count(&sms);
  if (rc != RLT_OK) return rc;
  int per_sm = (opt->variant >> 12) & 0xf;
  if (per_sm == 0) per_sm = 3;
  int grid = sms * per_sm;
  if (opt->grid_limit > 0 && grid > opt->grid_limit) grid = opt->grid_limit;
  const size_t smem = 2 * (static_cast<size_t>(batch->num_requests) + 1) * sizeof(int);
  if (dedup_wire) {
    p.dedup_wire = 1;
    const int planned = plan_dedup(p, workspace, workspace_bytes, sms, smem, stream);
    if (planned != RLT_OK) return planned;
  }
  int flavour = opt->variant & 0xf;
  if (flavour > 6) return RLT_E_INVALID;
  // Dedup into a pool (from a pool or from the wire image) over every plane: read each row once and fan it out,
  // unless flavour 6 asks for the walk over destination planes (kept for comparison; the bulk flavours 3 and 4
  // keep that walk too).
  const bool fan = (dir == kDirect || dir == kScatter) && opt->mode == RLT_MODE_DEDUP && p.plane_begin == 0 &&
                   p.plane_count == p.dst_planes && p.dst_planes > 1 && p.dst_planes <= kFanMaxPlanes &&
                   flavour != 3 && flavour != 4 && flavour != 6;
  if (flavour == 6) flavour = 0;
  if (fan) {
    p.fan = 1;
    table_fan_kernel<4><<<grid, kThreads, smem, stream>>>(p);
  } else if (flavour <= 2) {
    void (*kernel)(const TableCopyParams) = nullptr;
    if (dedup_wire) {
      kernel = flavour == 1 ? table_copy_kernel<8, true, true>
               : flavour == 2 ? table_copy_kernel<8, false, true> : table_copy_kernel<4, true, true>;
    } else {
      // Default: four 16-byte loads in flight per thread and three CTAs per SM. On the benchmark workload
      // this measured 6.5-6.6 TB/s of HBM traffic; eight loads in flight or four CTAs per SM were 5-8 % slower.
      kernel = flavour == 1 ? table_copy_kernel<8, true, false>
               : flavour == 2 ? table_copy_kernel<8, false, false> : table_copy_kernel<4, true, false>;
    }
    kernel<<<grid, kThreads, smem, stream>>>(p);
  } else if (flavour == 5) {
    // 32-byte vector loads and stores (two per thread in flight), same walk
    if (dedup_wire) {
      table_copy_kernel<2, true, true, true><<<grid, kThreads, smem, stream>>>(p);
    } else {
      table_copy_kernel<2, true, false, true><<<grid, kThreads, smem, stream>>>(p);
    }
  } else if (flavour <= 4) {
    // 3: eight 4 KiB stages per warp (six loads in flight); 4: four 8 KiB stages (two in flight).
    void (*kernel)(const TableCopyParams) = nullptr;
    if (dedup_wire) {
      kernel = flavour == 3 ? table_bulk_kernel<8, true> : table_bulk_kernel<4, true>;
    } else {
      kernel = flavour == 3 ? table_bulk_kernel<8, false> : table_bulk_kernel<4, false>;
    }
    const size_t bulk_smem_bytes = kBulkStageTotal + kBulkWarps * sizeof(BulkRing<8>) + smem;
    // Opting in to large dynamic shared memory is per device; the call is cheap, so it is simply repeated.
    RLT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(bulk_smem_bytes)));
    int bulk_grid = sms;  // one CTA of kBulkWarps pipelines per SM
    if (opt->grid_limit > 0 && bulk_grid > opt->grid_limit) bulk_grid = opt->grid_limit;
    kernel<<<bulk_grid, kBulkThreads, bulk_smem_bytes, stream>>>(p);
  } else {
    return RLT_E_INVALID;
  }
  RLT_CUDA_TRY(cudaGetLastError());
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return RLT_OK;
}

}  // namespace
}  // namespace rlt

namespace rlt {
namespace {

// Scratch of rlt_kv_pack_dedup_static: lives in the library image, one copy per GPU that loads it.
constexpr long long kStaticPlanEntries = 1ll << 20;
constexpr long long kStaticPlanBytes =
    kPlanHeaderBytes + 4 * kStaticPlanEntries + 4 * (kStaticPlanEntries / kPlanTile + 1);
static __device__ __align__(256) unsigned char g_static_plan[kStaticPlanBytes];

// Device address of g_static_plan on the current device, looked up once per device. In host code
// the array's name is only a handle for the runtime; the address has to be asked for.
int static_plan_address(void** out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<void*> cached[kMaxDevices];
  int device = 0;
  RLT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return RLT_E_LIMIT;
  void* ptr = cached[device].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    RLT_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_plan));
    if (ptr == nullptr) return RLT_E_CUDA;
    cached[device].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return RLT_OK;
}

}  // namespace
}  // namespace rlt

namespace rlt {
namespace {

// Staging of rlt_kv_handoff_host: per device a ring of slots, each a piece of pinned host memory and a piece of
// device memory of the same size, allocated at the first call on that device. A slot is written by the host,
// copied to the device on the caller's stream and read by the launch that follows; its event says when that
// launch has finished, and the slot is reused only then.
constexpr int kHostSlots = 16;
constexpr size_t kHostSlotBytes = 64 * 1024;

struct HostRing {
  unsigned char* pinned = nullptr;
  unsigned char* device = nullptr;
  cudaEvent_t done[kHostSlots] = {};
  int next = 0;
};

std::mutex g_host_ring_mutex;

int host_ring(HostRing** out) {
  constexpr int kMaxDevices = 64;
  static HostRing rings[kMaxDevices];
  int device = 0;
  RLT_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return RLT_E_LIMIT;
  HostRing& ring = rings[device];
  if (ring.pinned == nullptr) {
    void* host = nullptr;
    void* dev = nullptr;
    RLT_CUDA_TRY(cudaHostAlloc(&host, kHostSlots * kHostSlotBytes, cudaHostAllocDefault));
    if (cudaError_t e = cudaMalloc(&dev, kHostSlots * kHostSlotBytes); e != cudaSuccess) {
      cudaFreeHost(host);
      return cuda_fail(e);
    }
    for (int i = 0; i < kHostSlots; ++i) {
      if (cudaError_t e = cudaEventCreateWithFlags(&ring.done[i], cudaEventDisableTiming); e != cudaSuccess) {
        for (int j = 0; j < i; ++j) cudaEventDestroy(ring.done[j]);
        cudaFree(dev);
        cudaFreeHost(host);
        return cuda_fail(e);
      }
    }
    ring.device = static_cast<unsigned char*>(dev);
    ring.pinned = static_cast<unsigned char*>(host);
  }
  *out = &ring;
  return RLT_OK;
}

}  // namespace
}  // namespace rlt

extern "C" {

int rlt_kv_pack_dedup_static(const RltPool* src, const RltBatch* batch, const RltOptions* options, void* packed,
                             int64_t packed_bytes, rlt_stream_t stream) {
  if (src == nullptr || batch == nullptr || options == nullptr) return RLT_E_INVALID;
  if (options->mode != RLT_MODE_DEDUP) return RLT_E_INVALID;
  if (batch->num_requests < 1 || batch->table_width < 1 || src->num_planes < 1) return RLT_E_INVALID;
  const long long entries = static_cast<long long>(batch->num_requests) * batch->table_width * src->num_planes;
  if (entries > rlt::kStaticPlanEntries) return RLT_E_LIMIT;
  void* scratch = nullptr;
  const int rc = rlt::static_plan_address(&scratch);
  if (rc != RLT_OK) return rc;
  return rlt::launch_table_copy(rlt::kPack, src, nullptr, batch, options, packed, packed_bytes,
                                reinterpret_cast<cudaStream_t>(stream), scratch, rlt::kStaticPlanBytes);
}

int64_t rlt_kv_static_plan_entries(void) { return rlt::kStaticPlanEntries; }

int64_t rlt_kv_host_batch_limit(void) { return static_cast<int64_t>(rlt::kHostSlotBytes); }

int rlt_kv_handoff_host(const RltPool* src, const RltPool* dst, const RltHostBatch* hb, const RltOptions* options,
                        rlt_stream_t stream) {
  if (src == nullptr || dst == nullptr || hb == nullptr || options == nullptr) return RLT_E_INVALID;
  if (hb->num_requests < 1 || hb->num_requests > RLT_MAX_REQUESTS || hb->table_width < 1) return RLT_E_INVALID;
  if (hb->src_tables == nullptr || hb->dst_tables == nullptr || hb->tok_begin == nullptr || hb->tok_end == nullptr)
    return RLT_E_INVALID;
  if (hb->src_planes != src->num_planes || hb->dst_planes != dst->num_planes) return RLT_E_GEOMETRY;
  if (options->mode != RLT_MODE_ALL_PLANES) return RLT_E_INVALID;  // the other modes need per-token exit planes
  const size_t n = static_cast<size_t>(hb->num_requests);
  const size_t src_bytes = n * hb->src_planes * hb->table_width * sizeof(int32_t);
  const size_t dst_bytes = n * hb->dst_planes * hb->table_width * sizeof(int32_t);
  const size_t range_bytes = n * sizeof(int32_t);
  const size_t total = src_bytes + dst_bytes + 2 * range_bytes;
  if (total > rlt::kHostSlotBytes) return RLT_E_LIMIT;

  const std::lock_guard<std::mutex> lock(rlt::g_host_ring_mutex);
  rlt::HostRing* ring = nullptr;
  const int rc = rlt::host_ring(&ring);
  if (rc != RLT_OK) return rc;
  const int slot = ring->next;
  ring->next = (slot + 1) % rlt::kHostSlots;
  // the launch that last read this slot (kHostSlots calls ago) must be over before the host overwrites it
  RLT_CUDA_TRY(cudaEventSynchronize(ring->done[slot]));
  unsigned char* host = ring->pinned + slot * rlt::kHostSlotBytes;
  unsigned char* dev = ring->device + slot * rlt::kHostSlotBytes;
  memcpy(host, hb->src_tables, src_bytes);
  memcpy(host + src_bytes, hb->dst_tables, dst_bytes);
  memcpy(host + src_bytes + dst_bytes, hb->tok_begin, range_bytes);
  memcpy(host + src_bytes + dst_bytes + range_bytes, hb->tok_end, range_bytes);
  const cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  RLT_CUDA_TRY(cudaMemcpyAsync(dev, host, total, cudaMemcpyHostToDevice, s));
  RltBatch batch = {};
  batch.num_requests = hb->num_requests;
  batch.table_width = hb->table_width;
  batch.src_tables = reinterpret_cast<const int32_t*>(dev);
  batch.dst_tables = reinterpret_cast<const int32_t*>(dev + src_bytes);
  batch.tok_begin = reinterpret_cast<const int32_t*>(dev + src_bytes + dst_bytes);
  batch.tok_end = reinterpret_cast<const int32_t*>(dev + src_bytes + dst_bytes + range_bytes);
  const int launched = rlt::launch_table_copy(rlt::kDirect, src, dst, &batch, options, nullptr, 0, s);
  // recorded even when the launch was refused: the copy above still reads the slot
  RLT_CUDA_TRY(cudaEventRecord(ring->done[slot], s));
  return launched;
}

int rlt_kv_handoff(const RltPool* src, const RltPool* dst, const RltBatch* batch,
                   const RltOptions* options, rlt_stream_t stream) {
  return rlt::launch_table_copy(rlt::kDirect, src, dst, batch, options, nullptr, 0,
                                reinterpret_cast<cudaStream_t>(stream));
}

int64_t rlt_kv_dedup_workspace_bytes(int32_t num_requests, int32_t table_width, int32_t planes) {
  if (num_requests < 1 || table_width < 1 || planes < 1) return RLT_E_INVALID;
  return rlt::dedup_workspace_bytes(num_requests, table_width, planes);
}

int64_t rlt_kv_packed_bytes(const RltPool* pool, int64_t total_tokens, int32_t wire_planes, int32_t layers) {
  if (pool == nullptr || total_tokens < 0 || wire_planes < 1 || layers < 1) return RLT_E_INVALID;
  const int64_t row = pool->codes.token_bytes + (pool->scales.key != nullptr ? pool->scales.token_bytes : 0);
  return total_tokens * wire_planes * 2 * layers * row;
}

int rlt_kv_pack(const RltPool* src, const RltBatch* batch, const RltOptions* options, void* packed,
                int64_t packed_bytes, rlt_stream_t stream) {
  return rlt::launch_table_copy(rlt::kPack, src, nullptr, batch, options, packed, packed_bytes,
                                reinterpret_cast<cudaStream_t>(stream));
}

int rlt_kv_scatter(const void* packed, int64_t packed_bytes, const RltPool* dst, const RltBatch* batch,
                   const RltOptions* options, rlt_stream_t stream) {
  return rlt::launch_table_copy(rlt::kScatter, nullptr, dst, batch, options, const_cast<void*>(packed),
                                packed_bytes, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
