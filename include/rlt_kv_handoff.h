/*
 * C ABI of the B200 KV-handoff library (librlt_kv_handoff.so).
 *
 * The library moves paged KV-cache bytes from a prefill pool to a decode pool
 * with hand-written sm_100a kernels. It is the data plane behind the
 * reference's transfer connector: every entry point below names the reference
 * interface it replaces (paths relative to the vllm-rlt project root).
 *
 * Conventions
 *  - Plain C types only; no framework types cross this boundary.
 *  - Every pointer inside RltPool / RltBatch is a DEVICE pointer valid on the
 *    current device (a destination pool may be a peer mapping of another GPU).
 *    The structs themselves are read on the host during the call.
 *  - Calls are stream-ordered and never synchronise. The caller owns all
 *    memory; unless stated otherwise the library allocates nothing.
 *  - Return value: RLT_OK or a negative RLT_E_* code (argument errors are
 *    detected on the host before any launch). Data-dependent errors found on
 *    the device (a block id outside the pool, a token range outside the table)
 *    are recorded in the optional status words and the offending rows are
 *    skipped; the kernels never trap.
 */
#ifndef RLT_KV_HANDOFF_H
#define RLT_KV_HANDOFF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define RLT_API __attribute__((visibility("default")))
#else
#define RLT_API
#endif

/* cudaStream_t / CUstream, spelled without the CUDA headers. */
typedef struct CUstream_st* rlt_stream_t;

enum {
  RLT_OK = 0,
  RLT_E_INVALID = -1,  /* bad argument: null pointer, non-positive size, unknown mode          */
  RLT_E_GEOMETRY = -2, /* pools are not dense, or source and destination geometry differ       */
  RLT_E_LIMIT = -3,    /* a documented size limit of the entry point is exceeded               */
  RLT_E_CUDA = -4,     /* a CUDA runtime call failed; rlt_last_cuda_error() has the code        */
  RLT_E_ALIGN = -5     /* a pointer or size breaks the alignment rule of the entry point       */
};

/* Values written to status[0] by the kernels (0 = nothing to report). */
enum {
  RLT_STATUS_OK = 0,
  RLT_STATUS_BAD_RANGE = 1,   /* token range negative or past the table: status[1] = request      */
  RLT_STATUS_BAD_BLOCK = 2,   /* block id outside pool: [1] request, [2] logical block, [3] id    */
  RLT_STATUS_BAD_PLANE = 3,   /* exit plane outside [0, planes): [1] request, [2] token, [3] value */
  RLT_STATUS_TIMEOUT = 4,     /* rlt_kv_wait gave up: [1] low 32 bits of the last value seen      */
  RLT_STATUS_STALL = 5        /* a bulk copy never landed within the wait limit: [1] CTA, [2] warp */
};
#define RLT_STATUS_WORDS 4

/* Which source plane feeds a destination plane (plane = zero-based loop depth). */
enum {
  RLT_MODE_ALL_PLANES = 0, /* plane p <- plane p; what the reference's PD path sends
                              (vllm_rlt/pd/transport.py:40, "for table in tables")             */
  RLT_MODE_DEDUP = 1,      /* plane p <- plane min(p, exit); equals ALL_PLANES on a source
                              finalized by finalize_token (vllm_rlt/core/kv_cache_manager.py:1053-1076) */
  RLT_MODE_EXIT_ONLY = 2   /* single destination plane <- the token's exit plane             */
};

/*
 * One K/V tensor pair of a pool, as bytes. Same fields as the reference's
 * _kv_region (vllm_rlt/pd/transport.py:18-26). The tensors must be dense:
 * layer_bytes == block_size * token_bytes and block_bytes == num_layers *
 * layer_bytes, which is what KVCacheManager allocates
 * (vllm_rlt/core/kv_cache_manager.py:261-271).
 */
typedef struct RltRegion {
  void* key;
  void* value;
  int64_t block_bytes;
  int64_t layer_bytes;
  int64_t token_bytes; /* bytes of one token row: kv_heads * head_dim * element size */
} RltRegion;

/*
 * A paged KV pool: the codes (bf16/f16/f32 values or e4m3 bytes) and, for an
 * FP8 pool with per-vector scales, the float32 scale tensors. scales.key ==
 * NULL means no scale tensors travel (an unquantised pool, or a fixed-scale
 * FP8 pool: vllm_rlt/pd/transport.py:132-137).
 */
typedef struct RltPool {
  RltRegion codes;
  RltRegion scales;
  int32_t num_blocks;
  int32_t block_size; /* tokens per block, 1..64 */
  int32_t num_layers;
  int32_t num_planes; /* block tables per request: max_loops (LAST_EXITED) or 1 (SHARED) */
} RltPool;

/*
 * A batch of per-request handoffs. Tables are the reference's
 * plane_block_tables (vllm_rlt/core/kv_cache_manager.py:550-557), padded to a
 * common width. Token ranges are the [start, end) that queue_chunk passes to
 * kv_segments (vllm_rlt/pd/connector.py:220-231), after its prefix skip.
 */
typedef struct RltBatch {
  int32_t num_requests;        /* 1..RLT_MAX_REQUESTS                                          */
  int32_t table_width;         /* entries per table row                                         */
  const int32_t* src_tables;   /* [num_requests, src planes, table_width]                       */
  const int32_t* dst_tables;   /* [num_requests, dst planes, table_width]                       */
  const int32_t* tok_begin;    /* [num_requests]                                                */
  const int32_t* tok_end;      /* [num_requests]; a request with end <= begin moves nothing     */
  const int32_t* exit_planes;  /* NULL, or per-token zero-based exit plane (DEDUP / EXIT_ONLY)  */
  const int64_t* exit_offsets; /* [num_requests]: index in exit_planes of the request's token 0 */
  int64_t exit_count;          /* entries in exit_planes; a request whose exit_offsets[r] is negative or
                                  whose exit_offsets[r] + tok_end[r] exceeds it is reported as
                                  RLT_STATUS_BAD_RANGE and skipped, so no kernel reads past the array */
} RltBatch;

#define RLT_MAX_REQUESTS 4096

typedef struct RltOptions {
  int32_t mode;        /* RLT_MODE_*                                                            */
  int32_t layer_begin; /* layer slice [layer_begin, layer_end) for layer-by-layer streaming    */
  int32_t layer_end;   /* 0 means num_layers                                                    */
  int32_t wire_planes; /* pack/scatter: planes on the wire; 0 = source planes (1 for EXIT_ONLY) */
  int32_t* status;     /* NULL or device/mapped int32[RLT_STATUS_WORDS], zeroed by the caller   */
  int32_t grid_limit;  /* 0 = one persistent wave (a few CTAs per SM); else cap on CTAs launched */
  int32_t variant;     /* low 4 bits pick the kernel flavour: 0 register path (default), 1 and 2 its
                          deeper-unrolled forms, 3 and 4 cp.async.bulk rings, 5 32-byte accesses, 6 the
                          register path with rlt_kv_handoff's DEDUP walking destination planes (the
                          default walks source planes: each row is read once and stored to every
                          plane it fills); bits 4-11 = unit size in 16 KiB steps and bits 12-15 = CTAs
                          per SM are tuning knobs, 0 = default                                      */
  void* workspace;     /* device scratch; needed only by pack/scatter in RLT_MODE_DEDUP          */
  int64_t workspace_bytes; /* at least rlt_kv_dedup_workspace_bytes(...) for those calls          */
  int32_t plane_begin; /* destination (or wire) plane slice [plane_begin, plane_end): lets a   */
  int32_t plane_end;   /* depth be handed off as soon as it is computed; 0 means all planes     */
  uint64_t deep_layer_mask; /* rlt_kv_handoff only: layers carried for planes >= 1 (bit l = layer l);
                          0 = all. Recurrent-depth models keep only their recurrent layers per
                          depth (recurrent_layers, vllm_rlt/core/kv_cache_manager.py:228-238);
                          plane 0 always carries the whole layer slice                          */
} RltOptions;

/* --- information ---------------------------------------------------------------------------- */

RLT_API int rlt_version(void);
RLT_API const char* rlt_error_string(int code);
/* Last cudaError_t seen by this thread inside the library (0 if none). */
RLT_API int rlt_last_cuda_error(void);
/* How many of this library's kernels the calling process has launched so far. */
RLT_API int64_t rlt_kernel_launches(void);

/* --- the handoff ---------------------------------------------------------------------------- */

/*
 * Pool-to-pool handoff driven by block tables: for every request, destination
 * plane, token in [begin, end), layer in the slice and tensor (K, V, and the
 * scale tensors when present) copy the token's row from the source block to
 * the destination block. The destination may live on a peer GPU. No staging
 * buffer is used and no other destination byte is written.
 *
 * Replaces, as one launch, the plan + write of PDStageConnector.queue_chunk /
 * _submit_chunk (vllm_rlt/pd/connector.py:220-246, :444-455): kv_segments on
 * both sides (vllm_rlt/pd/transport.py:29-63), partition_segments (:95-112) and
 * NixlConnector.submit's WRITE (:182-201).
 */
RLT_API int rlt_kv_handoff(const RltPool* src, const RltPool* dst, const RltBatch* batch,
                           const RltOptions* options, rlt_stream_t stream);

/*
 * rlt_kv_handoff in RLT_MODE_ALL_PLANES for a caller whose block tables are still in HOST memory: the call copies
 * them into a staging slot of the library (pinned host memory and device memory, 16 slots of 64 KiB per GPU,
 * allocated at the first call on that GPU), queues the host-to-device copy and the launch on `stream`, and returns.
 * The arrays may be changed or freed as soon as it has returned. A batch whose tables and ranges exceed
 * rlt_kv_host_batch_limit() bytes gets RLT_E_LIMIT and nothing is queued: stage such a batch yourself and call
 * rlt_kv_handoff. When all 16 slots belong to launches that have not finished, the call waits for the oldest
 * on the host; for that reason, and because it allocates at its first use, it is not for CUDA-graph capture.
 *
 * This is what a transfer worker calls per chunk: one request, tables of a few hundred entries, where the time to
 * stage them decides how soon after the producer's event the copy starts. It takes the place of the descriptor
 * lists NixlConnector.submit builds per chunk on the host (vllm_rlt/pd/transport.py:182-201 over kv_segments,
 * :29-63); block ids and ranges are checked on the device like in rlt_kv_handoff.
 */
typedef struct RltHostBatch {
  int32_t num_requests;      /* 1..RLT_MAX_REQUESTS                                  */
  int32_t table_width;       /* entries per table row, the same on both sides        */
  int32_t src_planes;        /* rows per request in src_tables = src->num_planes     */
  int32_t dst_planes;        /* rows per request in dst_tables = dst->num_planes     */
  const int32_t* src_tables; /* HOST [num_requests, src_planes, table_width]         */
  const int32_t* dst_tables; /* HOST [num_requests, dst_planes, table_width]         */
  const int32_t* tok_begin;  /* HOST [num_requests]                                  */
  const int32_t* tok_end;    /* HOST [num_requests]                                  */
} RltHostBatch;

RLT_API int rlt_kv_handoff_host(const RltPool* src, const RltPool* dst, const RltHostBatch* batch,
                                const RltOptions* options, rlt_stream_t stream);

/* Largest sum of table and range bytes rlt_kv_handoff_host accepts. */
RLT_API int64_t rlt_kv_host_batch_limit(void);

/*
 * Bytes of the packed wire image of a batch: total_tokens * planes * 2 *
 * layers * (codes row + scales row). Host-side arithmetic only.
 */
RLT_API int64_t rlt_kv_packed_bytes(const RltPool* pool, int64_t total_tokens, int32_t wire_planes,
                                    int32_t layers);

/*
 * Scratch bytes that rlt_kv_pack / rlt_kv_scatter need in RLT_MODE_DEDUP for a
 * batch of this shape (planes = source planes). The scratch holds the wire
 * plan: where each (request, plane, block) starts when every token carries only
 * the planes up to its exit plane. After the call (stream-ordered) its first 8
 * bytes hold, as int64, the number of (token, plane) pairs on the wire; the
 * wire image is that count times 2 * layers * (codes row + scales row) bytes.
 */
RLT_API int64_t rlt_kv_dedup_workspace_bytes(int32_t num_requests, int32_t table_width, int32_t planes);

/*
 * Gather a batch into a contiguous buffer in the reference's segment order
 * (vllm_rlt/pd/transport.py:40-63: plane, logical block, codes then scales, K
 * then V, layer, token), requests back to back. batch->dst_tables is ignored.
 * packed must be 16-byte aligned. In RLT_MODE_DEDUP the image holds the same
 * walk with the rows of planes deeper than a token's exit plane left out
 * (they are copies, vllm_rlt/core/kv_cache_manager.py:1053-1076); this needs
 * options->workspace.
 */
RLT_API int rlt_kv_pack(const RltPool* src, const RltBatch* batch, const RltOptions* options,
                        void* packed, int64_t packed_bytes, rlt_stream_t stream);

/*
 * rlt_kv_pack in RLT_MODE_DEDUP for callers that must not allocate. It has no
 * counterpart in the reference.
 *
 * Who needs it: a stage worker that hands every free byte of HBM to its KV pool
 * at start-up and then serves with allocation switched off. For such a worker a
 * later cudaMalloc of the wire-plan scratch can fail outright, or stall the whole
 * device in the middle of serving, so it cannot provide options->workspace.
 *
 * This entry point takes no workspace (options->workspace is ignored): the plan
 * lives in an array inside the library image, about 4.2 MB that every GPU
 * which loads the library holds until the process exits. It calls no
 * cudaMalloc, cudaFree or any other allocating routine. Limit: num_requests *
 * table_width * source planes <= rlt_kv_static_plan_entries() (2^20); larger
 * batches get RLT_E_LIMIT and nothing is launched. Inputs and the packed
 * output are still the caller's. options->mode must be RLT_MODE_DEDUP.
 *
 * The first call on each device looks up the array's device address (one
 * runtime query, with that device current); make that first call before
 * starting any stream capture. It is also the latest moment at which the
 * array's 4.2 MB are placed on that device: CUDA loads a library's device
 * image lazily, at the first use of one of its kernels or symbols there. A
 * worker that hands all remaining HBM to its pool must therefore make this
 * first call (or any launch of this library) BEFORE the pool takes the memory,
 * or the placement itself can fail. All calls on a device share the one array and
 * it keeps the previous call's contents; every word a call reads is written
 * by that call first, so nothing has to be cleared, but two calls that overlap
 * on the GPU (different streams, no ordering between them) race on it: order
 * them, or use rlt_kv_pack with separate workspaces.
 */
RLT_API int rlt_kv_pack_dedup_static(const RltPool* src, const RltBatch* batch, const RltOptions* options,
                                     void* packed, int64_t packed_bytes, rlt_stream_t stream);
RLT_API int64_t rlt_kv_static_plan_entries(void);

/*
 * Inverse of rlt_kv_pack: write a packed image into the destination blocks
 * named by batch->dst_tables (batch->src_tables is ignored). Writes only the
 * rows of valid tokens. In RLT_MODE_DEDUP (exit planes and workspace needed)
 * the image is a dedup image and every destination plane deeper than a
 * token's exit plane receives a copy of the exit plane's row, which is what
 * finalize_token had left in the source.
 */
RLT_API int rlt_kv_scatter(const void* packed, int64_t packed_bytes, const RltPool* dst,
                           const RltBatch* batch, const RltOptions* options, rlt_stream_t stream);

/*
 * Copy one contiguous range, typically a packed image into a buffer on the
 * decode GPU through a peer pointer. Any alignment; 16-byte aligned ranges
 * take the vector path.
 */
RLT_API int rlt_kv_push(const void* src, void* dst, int64_t nbytes, rlt_stream_t stream);

/*
 * Copy a list of (source address, destination address, byte count) triples
 * held in device memory as int64[count][3], count <= RLT_MAX_SEGMENTS. This is
 * the WRITE of one NixlConnector.submit call (vllm_rlt/pd/transport.py:182-201)
 * for descriptor lists produced by partition_segments, so an unmodified
 * PDStageConnector can drive this library.
 */
RLT_API int rlt_kv_copy_segments(const int64_t* segments, int32_t count, rlt_stream_t stream);
#define RLT_MAX_SEGMENTS 4096

/* --- exit-depth propagation ------------------------------------------------------------------ */

/*
 * For each row (request index, exit plane, token position) copy the token's K,
 * V and scale rows of the exit plane into every deeper plane of the same pool,
 * for the layers whose bit is set in layer_mask (0 = all layers; the reference
 * copies its recurrent_layers). rows is a device int32[count][3]; tables is the
 * device int32[num_requests][planes][table_width] of the pool. One launch.
 *
 * Replaces KVCacheManager.finalize_token (vllm_rlt/core/kv_cache_manager.py:1053-1076)
 * and the finalize_kernel launches of ModelRunner.finalize_many
 * (vllm_rlt/kernels/routing.py:147-179, vllm_rlt/worker/model_runner.py:1349-1395).
 * Scale tensors are copied whenever pool->scales is set, fixed-scale pools
 * included, as the reference does.
 */
RLT_API int rlt_kv_finalize(const RltPool* pool, const int32_t* tables, int32_t num_requests, int32_t table_width,
                            const int32_t* rows, int32_t count, uint64_t layer_mask, int32_t* status,
                            rlt_stream_t stream);

/* --- typed tensor transfer ------------------------------------------------------------------- */

enum { RLT_DTYPE_I32 = 0, RLT_DTYPE_I64 = 1, RLT_DTYPE_F16 = 2, RLT_DTYPE_BF16 = 3, RLT_DTYPE_F32 = 4 };

/*
 * A batch of strided 2-D copies with element conversion. descriptors is an
 * int64[count][8] table readable from the device (device memory or mapped pinned
 * host memory): source address, destination address, rows, cols, source row and
 * column stride, destination row and column stride, strides in elements.
 * max_rows / max_cols bound the largest copy of the batch. Sources may be mapped
 * host memory; destinations are on the current device. Replaces the segmented mode
 * of tensor_transfer_kernel and TensorTransfer.submit
 * (vllm_rlt/kernels/tensor_transfer.py:21-35, vllm_rlt/worker/tensors.py:321-365).
 */
RLT_API int rlt_tensor_transfer(const int64_t* descriptors, int32_t count, int32_t max_rows, int32_t max_cols,
                                int32_t src_dtype, int32_t dst_dtype, rlt_stream_t stream);

/*
 * Flat copy of count elements with conversion, optionally writing a second output
 * of its own type from the same source values (secondary may be NULL). Replaces
 * copy_tensor's kernel path (vllm_rlt/worker/tensors.py:35-87).
 */
RLT_API int rlt_tensor_copy(const void* src, void* dst, void* secondary, int64_t count, int32_t src_dtype,
                            int32_t dst_dtype, int32_t secondary_dtype, rlt_stream_t stream);

/* --- completion ----------------------------------------------------------------------------- */

/*
 * Stream-ordered release store of value to *flag (device, peer or mapped host
 * memory, 8-byte aligned). Issued after a handoff on the same stream it tells
 * the receiver that every earlier write has landed; it takes the place of the
 * notification NIXL delivers with each WRITE (vllm_rlt/pd/transport.py:186-195, :222-229).
 */
RLT_API int rlt_kv_signal(uint64_t* flag, uint64_t value, rlt_stream_t stream);

/*
 * Bounded device-side wait until *flag >= value. Gives up after timeout_ns
 * (1 .. RLT_MAX_WAIT_NS), writing RLT_STATUS_TIMEOUT to status; the kernel
 * always returns and the context stays usable. Never launch it on the GPU
 * whose own later work is what sets the flag.
 */
RLT_API int rlt_kv_wait(const uint64_t* flag, uint64_t value, int64_t timeout_ns, int32_t* status,
                        rlt_stream_t stream);
#define RLT_MAX_WAIT_NS 2000000000LL

/*
 * Stream-ordered post of a 64-byte message into a mailbox slot (device, peer or
 * registered host memory, 16-byte aligned): bytes 8..63 are written first, then
 * the 8-byte stamp at offset 0 with release semantics at system scope, so a
 * reader that sees the stamp also sees the body and every earlier write of the
 * stream. Carries the (transfer id, sequence) notification that NIXL attaches
 * to each WRITE (vllm_rlt/pd/transport.py:186, :222-229).
 */
RLT_API int rlt_kv_post(void* slot, const uint8_t body[56], uint64_t stamp, rlt_stream_t stream);

/* --- peer memory ---------------------------------------------------------------------------- */

/* Enable access from device `device` to memory of device `peer` (idempotent). */
RLT_API int rlt_peer_enable(int device, int peer);
/* 1 if `device` can map memory of `peer`, 0 if not, negative on error. */
RLT_API int rlt_peer_can_access(int device, int peer);

#define RLT_IPC_HANDLE_BYTES 64
/*
 * Export the allocation that contains ptr for another process on the same
 * host: fills handle and the byte offset of ptr inside that allocation. This
 * takes the place of the NIXL agent metadata in startup_info
 * (vllm_rlt/pd/connector.py:96-98, vllm_rlt/pd/transport.py:140-154).
 */
RLT_API int rlt_ipc_export(const void* ptr, uint8_t handle[RLT_IPC_HANDLE_BYTES], int64_t* offset);
/* Map an exported allocation into this process on the current device. */
RLT_API int rlt_ipc_open(const uint8_t handle[RLT_IPC_HANDLE_BYTES], void** base);
RLT_API int rlt_ipc_close(void* base);

/*
 * Make a range of ordinary host memory (for instance a POSIX shared-memory
 * mapping that another process polls) writable from kernels on the current
 * device; returns the device-side address. The receiver of a handoff keeps its
 * mailbox in such memory so that it can poll without any CUDA call.
 */
RLT_API int rlt_host_register(void* host, size_t bytes, void** device_ptr);
RLT_API int rlt_host_unregister(void* host);

#ifdef __cplusplus
}
#endif
#endif /* RLT_KV_HANDOFF_H */
