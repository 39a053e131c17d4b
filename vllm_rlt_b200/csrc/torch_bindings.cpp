// torch.ops.vllm_rlt.kv_* : the KV-handoff ops, registered the way the
// reference registers its one native op (csrc/torch_bindings.cpp:7-15 there):
// schema in the vllm_rlt namespace, CUDA implementation, empty Python module.
// A FRAGMENT is used so the ops can live beside the reference's own
// TORCH_LIBRARY(vllm_rlt, ...) definition in one process.
//
// Conventions kept from the reference's op (csrc/activation/silu_and_mul.cu:220-247):
// TORCH_CHECK on device, dtype and contiguity (a RuntimeError in Python), a
// device guard on the input's device, launch on the current stream of that
// device, no synchronisation, inputs never modified.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/pybind11.h>
#include <torch/library.h>

#include "ops.h"
#include "rlt_kv_handoff.h"

namespace vllm_rlt_b200 {
namespace {

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == RLT_OK, what, ": ", rlt_error_string(rc),
              rc == RLT_E_CUDA ? " (cudaError " + std::to_string(rlt_last_cuda_error()) + ")" : std::string());
}

void check_pool_tensor(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor: the KV handoff has no CPU path");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
  TORCH_CHECK(t.dim() >= 4, name, " must be [blocks, layers, block_size, ...]");
}

RltRegion region_of(const at::Tensor& key, const at::Tensor& value, const char* name) {
  check_pool_tensor(key, name);
  check_pool_tensor(value, name);
  TORCH_CHECK(key.sizes() == value.sizes() && key.scalar_type() == value.scalar_type() &&
                  key.device() == value.device(),
              name, ": key and value must agree in shape, dtype and device");
  const int64_t e = key.element_size();
  return RltRegion{key.data_ptr(), value.data_ptr(), key.stride(0) * e, key.stride(1) * e, key.stride(2) * e};
}

RltPool pool_of(const at::Tensor& key, const at::Tensor& value, const OptTensor& key_scale,
                const OptTensor& value_scale, int64_t planes) {
  RltPool pool{};
  pool.codes = region_of(key, value, "KV pool");
  TORCH_CHECK(key_scale.has_value() == value_scale.has_value(), "scale tensors come as a pair");
  if (key_scale.has_value()) {
    TORCH_CHECK(key_scale->scalar_type() == at::kFloat, "scale tensors must be float32");
    TORCH_CHECK(key_scale->device() == key.device(), "scale tensors must be on the pool's device");
    pool.scales = region_of(*key_scale, *value_scale, "KV scale pool");
  }
  pool.num_blocks = static_cast<int32_t>(key.size(0));
  pool.num_layers = static_cast<int32_t>(key.size(1));
  pool.block_size = static_cast<int32_t>(key.size(2));
  pool.num_planes = static_cast<int32_t>(planes);
  return pool;
}

const int32_t* i32(const at::Tensor& t, const at::Device& device, const char* name) {
  TORCH_CHECK(t.device() == device, name, " must be on the pool's device");
  TORCH_CHECK(t.scalar_type() == at::kInt && t.is_contiguous(), name, " must be a contiguous int32 tensor");
  return t.data_ptr<int32_t>();
}

struct BatchArgs {
  RltBatch batch{};
  int64_t src_planes = 0, dst_planes = 0;
};

BatchArgs batch_of(const at::Tensor* src_tables, const at::Tensor* dst_tables, const at::Tensor& tok_begin,
                   const at::Tensor& tok_end, const OptTensor& exit_planes, const OptTensor& exit_offsets,
                   const at::Device& device) {
  BatchArgs out;
  const at::Tensor& any = src_tables != nullptr ? *src_tables : *dst_tables;
  TORCH_CHECK(any.dim() == 3, "block tables must be [requests, planes, pages]");
  out.batch.num_requests = static_cast<int32_t>(any.size(0));
  out.batch.table_width = static_cast<int32_t>(any.size(2));
  if (src_tables != nullptr) {
    TORCH_CHECK(src_tables->dim() == 3 && src_tables->size(0) == any.size(0) && src_tables->size(2) == any.size(2),
                "source and destination tables must agree in requests and width");
    out.batch.src_tables = i32(*src_tables, device, "src_tables");
    out.src_planes = src_tables->size(1);
  }
  if (dst_tables != nullptr) {
    TORCH_CHECK(dst_tables->dim() == 3 && dst_tables->size(0) == any.size(0) && dst_tables->size(2) == any.size(2),
                "source and destination tables must agree in requests and width");
    out.batch.dst_tables = i32(*dst_tables, device, "dst_tables");
    out.dst_planes = dst_tables->size(1);
  }
  TORCH_CHECK(tok_begin.numel() == any.size(0) && tok_end.numel() == any.size(0), "one token range per request");
  out.batch.tok_begin = i32(tok_begin, device, "tok_begin");
  out.batch.tok_end = i32(tok_end, device, "tok_end");
  TORCH_CHECK(exit_planes.has_value() == exit_offsets.has_value(), "exit_planes and exit_offsets come as a pair");
  if (exit_planes.has_value()) {
    out.batch.exit_planes = i32(*exit_planes, device, "exit_planes");
    TORCH_CHECK(exit_offsets->device() == device && exit_offsets->scalar_type() == at::kLong &&
                    exit_offsets->is_contiguous() && exit_offsets->numel() == any.size(0),
                "exit_offsets must be a contiguous int64 tensor with one entry per request");
    out.batch.exit_offsets = exit_offsets->data_ptr<int64_t>();
    out.batch.exit_count = exit_planes->numel();  // lets the kernels refuse offsets that would run past the array
  }
  return out;
}

int32_t* status_ptr(const OptTensor& status, const at::Device& device) {
  if (!status.has_value()) return nullptr;
  TORCH_CHECK(status->device() == device && status->scalar_type() == at::kInt && status->is_contiguous() &&
                  status->numel() >= RLT_STATUS_WORDS,
              "status must be a contiguous int32 tensor of at least ", RLT_STATUS_WORDS, " words on the pool's device");
  return status->data_ptr<int32_t>();
}

RltOptions options_of(int64_t mode, int64_t layer_begin, int64_t layer_end, int32_t* status) {
  RltOptions o{};
  o.mode = static_cast<int32_t>(mode);
  o.layer_begin = static_cast<int32_t>(layer_begin);
  o.layer_end = static_cast<int32_t>(layer_end);
  o.status = status;
  return o;
}

rlt_stream_t current_stream(const at::Device& device) {
  return reinterpret_cast<rlt_stream_t>(at::cuda::getCurrentCUDAStream(device.index()).stream());
}

}  // namespace

void kv_handoff_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                     const OptTensor& src_value_scale, at::Tensor& dst_key, at::Tensor& dst_value,
                     const OptTensor& dst_key_scale, const OptTensor& dst_value_scale, const at::Tensor& src_tables,
                     const at::Tensor& dst_tables, const at::Tensor& tok_begin, const at::Tensor& tok_end,
                     const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin,
                     int64_t layer_end, const OptTensor& status) {
  const at::Device device = src_key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(&src_tables, &dst_tables, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool src = pool_of(src_key, src_value, src_key_scale, src_value_scale, b.src_planes);
  const RltPool dst = pool_of(dst_key, dst_value, dst_key_scale, dst_value_scale, b.dst_planes);
  const RltOptions o = options_of(mode, layer_begin, layer_end, status_ptr(status, device));
  check_rc(rlt_kv_handoff(&src, &dst, &b.batch, &o, current_stream(device)), "kv_handoff");
}

// The all-planes handoff with the block tables still in host memory (CPU int32 tensors): the library stages them
// in a slot of its own and queues copy and launch on the current stream. For chunk-sized batches.
void kv_handoff_host_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                          const OptTensor& src_value_scale, at::Tensor& dst_key, at::Tensor& dst_value,
                          const OptTensor& dst_key_scale, const OptTensor& dst_value_scale, const at::Tensor& src_tables,
                          const at::Tensor& dst_tables, const at::Tensor& tok_begin, const at::Tensor& tok_end,
                          int64_t layer_begin, int64_t layer_end, const OptTensor& status) {
  const at::Device device = src_key.device();
  const c10::cuda::CUDAGuard guard(device);
  for (const at::Tensor* t : {&src_tables, &dst_tables, &tok_begin, &tok_end}) {
    TORCH_CHECK(t->device().is_cpu() && t->scalar_type() == at::kInt && t->is_contiguous(),
                "kv_handoff_host takes its tables and ranges as contiguous CPU int32 tensors");
  }
  TORCH_CHECK(src_tables.dim() == 3 && dst_tables.dim() == 3 && src_tables.size(0) == dst_tables.size(0) &&
                  src_tables.size(2) == dst_tables.size(2),
              "block tables must be [requests, planes, pages] and agree in requests and pages");
  TORCH_CHECK(tok_begin.numel() == src_tables.size(0) && tok_end.numel() == src_tables.size(0),
              "one token range per request");
  RltHostBatch hb{};
  hb.num_requests = static_cast<int32_t>(src_tables.size(0));
  hb.table_width = static_cast<int32_t>(src_tables.size(2));
  hb.src_planes = static_cast<int32_t>(src_tables.size(1));
  hb.dst_planes = static_cast<int32_t>(dst_tables.size(1));
  hb.src_tables = src_tables.data_ptr<int32_t>();
  hb.dst_tables = dst_tables.data_ptr<int32_t>();
  hb.tok_begin = tok_begin.data_ptr<int32_t>();
  hb.tok_end = tok_end.data_ptr<int32_t>();
  const RltPool src = pool_of(src_key, src_value, src_key_scale, src_value_scale, hb.src_planes);
  const RltPool dst = pool_of(dst_key, dst_value, dst_key_scale, dst_value_scale, hb.dst_planes);
  const RltOptions o = options_of(RLT_MODE_ALL_PLANES, layer_begin, layer_end, status_ptr(status, device));
  check_rc(rlt_kv_handoff_host(&src, &dst, &hb, &o, current_stream(device)), "kv_handoff_host");
}

void kv_handoff_peer_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                          const OptTensor& src_value_scale, int64_t dst_key_ptr, int64_t dst_value_ptr,
                          int64_t dst_key_scale_ptr, int64_t dst_value_scale_ptr, int64_t dst_num_blocks,
                          int64_t dst_num_planes, const at::Tensor& src_tables, const at::Tensor& dst_tables,
                          const at::Tensor& tok_begin, const at::Tensor& tok_end, const OptTensor& exit_planes,
                          const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin, int64_t layer_end,
                          const OptTensor& status) {
  const at::Device device = src_key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(&src_tables, &dst_tables, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool src = pool_of(src_key, src_value, src_key_scale, src_value_scale, b.src_planes);
  TORCH_CHECK(dst_num_planes == b.dst_planes, "dst_tables planes must equal dst_num_planes");
  // The peer pool has the source's geometry (the handshake enforces it,
  // vllm_rlt/pd/transport.py:162-173); only its addresses and block count differ.
  RltPool dst = src;
  dst.codes.key = reinterpret_cast<void*>(dst_key_ptr);
  dst.codes.value = reinterpret_cast<void*>(dst_value_ptr);
  if (src.scales.key != nullptr) {
    dst.scales.key = reinterpret_cast<void*>(dst_key_scale_ptr);
    dst.scales.value = reinterpret_cast<void*>(dst_value_scale_ptr);
  }
  dst.num_blocks = static_cast<int32_t>(dst_num_blocks);
  dst.num_planes = static_cast<int32_t>(dst_num_planes);
  const RltOptions o = options_of(mode, layer_begin, layer_end, status_ptr(status, device));
  check_rc(rlt_kv_handoff(&src, &dst, &b.batch, &o, current_stream(device)), "kv_handoff_peer");
}

void kv_pack_cuda(const at::Tensor& key, const at::Tensor& value, const OptTensor& key_scale,
                  const OptTensor& value_scale, const at::Tensor& tables, const at::Tensor& tok_begin,
                  const at::Tensor& tok_end, const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode,
                  int64_t layer_begin, int64_t layer_end, at::Tensor& out, const OptTensor& status) {
  const at::Device device = key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(&tables, nullptr, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool src = pool_of(key, value, key_scale, value_scale, b.src_planes);
  TORCH_CHECK(out.device() == device && out.scalar_type() == at::kByte && out.is_contiguous(),
              "packed buffer must be a contiguous uint8 tensor on the pool's device");
  const RltOptions o = options_of(mode, layer_begin, layer_end, status_ptr(status, device));
  check_rc(rlt_kv_pack(&src, &b.batch, &o, out.data_ptr(), out.numel(), current_stream(device)), "kv_pack");
}

void kv_scatter_cuda(const at::Tensor& packed, const at::Tensor& tables, const at::Tensor& tok_begin,
                     const at::Tensor& tok_end, int64_t layer_begin, int64_t layer_end, at::Tensor& key,
                     at::Tensor& value, const OptTensor& key_scale, const OptTensor& value_scale,
                     const OptTensor& status) {
  const at::Device device = key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(nullptr, &tables, tok_begin, tok_end, std::nullopt, std::nullopt, device);
  const RltPool dst = pool_of(key, value, key_scale, value_scale, b.dst_planes);
  TORCH_CHECK(packed.device() == device && packed.scalar_type() == at::kByte && packed.is_contiguous(),
              "packed buffer must be a contiguous uint8 tensor on the pool's device");
  const RltOptions o = options_of(RLT_MODE_ALL_PLANES, layer_begin, layer_end, status_ptr(status, device));
  check_rc(rlt_kv_scatter(packed.data_ptr(), packed.numel(), &dst, &b.batch, &o, current_stream(device)), "kv_scatter");
}

void kv_handoff_slice_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                           const OptTensor& src_value_scale, at::Tensor& dst_key, at::Tensor& dst_value,
                           const OptTensor& dst_key_scale, const OptTensor& dst_value_scale, const at::Tensor& src_tables,
                           const at::Tensor& dst_tables, const at::Tensor& tok_begin, const at::Tensor& tok_end,
                           const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin,
                           int64_t layer_end, int64_t plane_begin, int64_t plane_end, const OptTensor& status) {
  const at::Device device = src_key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(&src_tables, &dst_tables, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool src = pool_of(src_key, src_value, src_key_scale, src_value_scale, b.src_planes);
  const RltPool dst = pool_of(dst_key, dst_value, dst_key_scale, dst_value_scale, b.dst_planes);
  RltOptions o = options_of(mode, layer_begin, layer_end, status_ptr(status, device));
  o.plane_begin = static_cast<int32_t>(plane_begin);
  o.plane_end = static_cast<int32_t>(plane_end);
  check_rc(rlt_kv_handoff(&src, &dst, &b.batch, &o, current_stream(device)), "kv_handoff_slice");
}

namespace {

void attach_workspace(RltOptions& o, at::Tensor& workspace, const at::Device& device) {
  TORCH_CHECK(workspace.device() == device && workspace.scalar_type() == at::kByte && workspace.is_contiguous(),
              "workspace must be a contiguous uint8 tensor on the pool's device");
  o.workspace = workspace.data_ptr();
  o.workspace_bytes = workspace.numel();
}

}  // namespace

void kv_pack_dedup_cuda(const at::Tensor& key, const at::Tensor& value, const OptTensor& key_scale,
                        const OptTensor& value_scale, const at::Tensor& tables, const at::Tensor& tok_begin,
                        const at::Tensor& tok_end, const at::Tensor& exit_planes, const at::Tensor& exit_offsets,
                        int64_t layer_begin, int64_t layer_end, at::Tensor& out, at::Tensor& workspace,
                        const OptTensor& status) {
  const at::Device device = key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(&tables, nullptr, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool src = pool_of(key, value, key_scale, value_scale, b.src_planes);
  TORCH_CHECK(out.device() == device && out.scalar_type() == at::kByte && out.is_contiguous(),
              "packed buffer must be a contiguous uint8 tensor on the pool's device");
  RltOptions o = options_of(RLT_MODE_DEDUP, layer_begin, layer_end, status_ptr(status, device));
  attach_workspace(o, workspace, device);
  check_rc(rlt_kv_pack(&src, &b.batch, &o, out.data_ptr(), out.numel(), current_stream(device)), "kv_pack_dedup");
}

void kv_scatter_dedup_cuda(const at::Tensor& packed, const at::Tensor& tables, const at::Tensor& tok_begin,
                           const at::Tensor& tok_end, const at::Tensor& exit_planes, const at::Tensor& exit_offsets,
                           int64_t layer_begin, int64_t layer_end, at::Tensor& key, at::Tensor& value,
                           const OptTensor& key_scale, const OptTensor& value_scale, at::Tensor& workspace,
                           const OptTensor& status) {
  const at::Device device = key.device();
  const c10::cuda::CUDAGuard guard(device);
  BatchArgs b = batch_of(nullptr, &tables, tok_begin, tok_end, exit_planes, exit_offsets, device);
  const RltPool dst = pool_of(key, value, key_scale, value_scale, b.dst_planes);
  TORCH_CHECK(packed.device() == device && packed.scalar_type() == at::kByte && packed.is_contiguous(),
              "packed buffer must be a contiguous uint8 tensor on the pool's device");
  RltOptions o = options_of(RLT_MODE_DEDUP, layer_begin, layer_end, status_ptr(status, device));
  attach_workspace(o, workspace, device);
  check_rc(rlt_kv_scatter(packed.data_ptr(), packed.numel(), &dst, &b.batch, &o, current_stream(device)), "kv_scatter_dedup");
}

void kv_finalize_cuda(at::Tensor& key, at::Tensor& value, const OptTensor& key_scale, const OptTensor& value_scale,
                      const at::Tensor& tables, const at::Tensor& rows, int64_t layer_mask, const OptTensor& status) {
  const at::Device device = key.device();
  const c10::cuda::CUDAGuard guard(device);
  TORCH_CHECK(tables.dim() == 3, "tables must be [requests, planes, pages]");
  TORCH_CHECK(rows.dim() == 2 && rows.size(1) == 3, "rows must be [n, 3]: request index, exit plane, token position");
  const RltPool pool = pool_of(key, value, key_scale, value_scale, tables.size(1));
  check_rc(rlt_kv_finalize(&pool, i32(tables, device, "tables"), static_cast<int32_t>(tables.size(0)),
                           static_cast<int32_t>(tables.size(2)), i32(rows, device, "rows"),
                           static_cast<int32_t>(rows.size(0)), static_cast<uint64_t>(layer_mask),
                           status_ptr(status, device), current_stream(device)),
           "kv_finalize");
}

void kv_push_cuda(const at::Tensor& src, int64_t dst_ptr, int64_t nbytes) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous(), "kv_push source must be a contiguous CUDA tensor");
  TORCH_CHECK(nbytes >= 0 && nbytes <= static_cast<int64_t>(src.nbytes()), "kv_push size exceeds the source tensor");
  const c10::cuda::CUDAGuard guard(src.device());
  check_rc(rlt_kv_push(src.data_ptr(), reinterpret_cast<void*>(dst_ptr), nbytes, current_stream(src.device())), "kv_push");
}

void kv_copy_segments_cuda(const at::Tensor& segments) {
  TORCH_CHECK(segments.is_cuda() && segments.is_contiguous() && segments.scalar_type() == at::kLong &&
                  segments.dim() == 2 && segments.size(1) == 3,
              "segments must be a contiguous CUDA int64 [n, 3] tensor");
  const c10::cuda::CUDAGuard guard(segments.device());
  check_rc(rlt_kv_copy_segments(segments.data_ptr<int64_t>(), static_cast<int32_t>(segments.size(0)),
                                current_stream(segments.device())),
           "kv_copy_segments");
}

void kv_signal_cuda(const at::Tensor& anchor, int64_t flag_ptr, int64_t value) {
  TORCH_CHECK(anchor.is_cuda(), "kv_signal anchor must be a CUDA tensor (it selects the device and stream)");
  const c10::cuda::CUDAGuard guard(anchor.device());
  check_rc(rlt_kv_signal(reinterpret_cast<uint64_t*>(flag_ptr), static_cast<uint64_t>(value),
                         current_stream(anchor.device())),
           "kv_signal");
}

void kv_wait_cuda(int64_t flag_ptr, int64_t value, int64_t timeout_ns, at::Tensor& status) {
  TORCH_CHECK(status.is_cuda(), "kv_wait status must be a CUDA tensor");
  const c10::cuda::CUDAGuard guard(status.device());
  check_rc(rlt_kv_wait(reinterpret_cast<const uint64_t*>(flag_ptr), static_cast<uint64_t>(value), timeout_ns,
                       status_ptr(status, status.device()), current_stream(status.device())),
           "kv_wait");
}

}  // namespace vllm_rlt_b200

TORCH_LIBRARY_FRAGMENT(vllm_rlt, ops) {
  ops.def(
      "kv_handoff(Tensor src_key, Tensor src_value, Tensor? src_key_scale, Tensor? src_value_scale, "
      "Tensor(a!) dst_key, Tensor(b!) dst_value, Tensor(c!)? dst_key_scale, Tensor(d!)? dst_value_scale, "
      "Tensor src_tables, Tensor dst_tables, Tensor tok_begin, Tensor tok_end, Tensor? exit_planes, "
      "Tensor? exit_offsets, int mode, int layer_begin, int layer_end, Tensor(e!)? status) -> ()");
  ops.def(
      "kv_handoff_host(Tensor src_key, Tensor src_value, Tensor? src_key_scale, Tensor? src_value_scale, "
      "Tensor(a!) dst_key, Tensor(b!) dst_value, Tensor(c!)? dst_key_scale, Tensor(d!)? dst_value_scale, "
      "Tensor src_tables, Tensor dst_tables, Tensor tok_begin, Tensor tok_end, int layer_begin, int layer_end, "
      "Tensor(e!)? status) -> ()");
  ops.def(
      "kv_handoff_peer(Tensor src_key, Tensor src_value, Tensor? src_key_scale, Tensor? src_value_scale, "
      "int dst_key_ptr, int dst_value_ptr, int dst_key_scale_ptr, int dst_value_scale_ptr, int dst_num_blocks, "
      "int dst_num_planes, Tensor src_tables, Tensor dst_tables, Tensor tok_begin, Tensor tok_end, "
      "Tensor? exit_planes, Tensor? exit_offsets, int mode, int layer_begin, int layer_end, "
      "Tensor(a!)? status) -> ()");
  ops.def(
      "kv_pack(Tensor key, Tensor value, Tensor? key_scale, Tensor? value_scale, Tensor tables, Tensor tok_begin, "
      "Tensor tok_end, Tensor? exit_planes, Tensor? exit_offsets, int mode, int layer_begin, int layer_end, "
      "Tensor(a!) out, Tensor(b!)? status) -> ()");
  ops.def(
      "kv_scatter(Tensor packed, Tensor tables, Tensor tok_begin, Tensor tok_end, int layer_begin, int layer_end, "
      "Tensor(a!) key, Tensor(b!) value, Tensor(c!)? key_scale, Tensor(d!)? value_scale, Tensor(e!)? status) -> ()");
  ops.def(
      "kv_handoff_slice(Tensor src_key, Tensor src_value, Tensor? src_key_scale, Tensor? src_value_scale, "
      "Tensor(a!) dst_key, Tensor(b!) dst_value, Tensor(c!)? dst_key_scale, Tensor(d!)? dst_value_scale, "
      "Tensor src_tables, Tensor dst_tables, Tensor tok_begin, Tensor tok_end, Tensor? exit_planes, "
      "Tensor? exit_offsets, int mode, int layer_begin, int layer_end, int plane_begin, int plane_end, "
      "Tensor(e!)? status) -> ()");
  ops.def(
      "kv_pack_dedup(Tensor key, Tensor value, Tensor? key_scale, Tensor? value_scale, Tensor tables, "
      "Tensor tok_begin, Tensor tok_end, Tensor exit_planes, Tensor exit_offsets, int layer_begin, int layer_end, "
      "Tensor(a!) out, Tensor(b!) workspace, Tensor(c!)? status) -> ()");
  ops.def(
      "kv_scatter_dedup(Tensor packed, Tensor tables, Tensor tok_begin, Tensor tok_end, Tensor exit_planes, "
      "Tensor exit_offsets, int layer_begin, int layer_end, Tensor(a!) key, Tensor(b!) value, Tensor(c!)? key_scale, "
      "Tensor(d!)? value_scale, Tensor(e!) workspace, Tensor(f!)? status) -> ()");
  ops.def(
      "kv_finalize(Tensor(a!) key, Tensor(b!) value, Tensor(c!)? key_scale, Tensor(d!)? value_scale, Tensor tables, "
      "Tensor rows, int layer_mask, Tensor(e!)? status) -> ()");
  ops.def("kv_push(Tensor src, int dst_ptr, int nbytes) -> ()");
  ops.def("kv_copy_segments(Tensor segments) -> ()");
  ops.def("kv_signal(Tensor anchor, int flag_ptr, int value) -> ()");
  ops.def("kv_wait(int flag_ptr, int value, int timeout_ns, Tensor(a!) status) -> ()");
}

TORCH_LIBRARY_IMPL(vllm_rlt, CUDA, ops) {
  ops.impl("kv_handoff", &vllm_rlt_b200::kv_handoff_cuda);
  ops.impl("kv_handoff_host", &vllm_rlt_b200::kv_handoff_host_cuda);
  ops.impl("kv_handoff_peer", &vllm_rlt_b200::kv_handoff_peer_cuda);
  ops.impl("kv_pack", &vllm_rlt_b200::kv_pack_cuda);
  ops.impl("kv_scatter", &vllm_rlt_b200::kv_scatter_cuda);
  ops.impl("kv_handoff_slice", &vllm_rlt_b200::kv_handoff_slice_cuda);
  ops.impl("kv_pack_dedup", &vllm_rlt_b200::kv_pack_dedup_cuda);
  ops.impl("kv_scatter_dedup", &vllm_rlt_b200::kv_scatter_dedup_cuda);
  ops.impl("kv_finalize", &vllm_rlt_b200::kv_finalize_cuda);
  ops.impl("kv_push", &vllm_rlt_b200::kv_push_cuda);
  ops.impl("kv_copy_segments", &vllm_rlt_b200::kv_copy_segments_cuda);
  ops.impl("kv_signal", &vllm_rlt_b200::kv_signal_cuda);
  ops.impl("kv_wait", &vllm_rlt_b200::kv_wait_cuda);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, module) {}
