// ATen-level declarations of the KV-handoff ops. Each is a thin shim over the
// C ABI in rlt_kv_handoff.h: check tensors, fill the plain structs, launch on
// the current stream of the tensors' device.
#pragma once

#include <ATen/ATen.h>

#include <optional>

namespace vllm_rlt_b200 {

using OptTensor = std::optional<at::Tensor>;

void kv_handoff_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                     const OptTensor& src_value_scale, at::Tensor& dst_key, at::Tensor& dst_value,
                     const OptTensor& dst_key_scale, const OptTensor& dst_value_scale, const at::Tensor& src_tables,
                     const at::Tensor& dst_tables, const at::Tensor& tok_begin, const at::Tensor& tok_end,
                     const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin,
                     int64_t layer_end, const OptTensor& status);

void kv_handoff_peer_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                          const OptTensor& src_value_scale, int64_t dst_key_ptr, int64_t dst_value_ptr,
                          int64_t dst_key_scale_ptr, int64_t dst_value_scale_ptr, int64_t dst_num_blocks,
                          int64_t dst_num_planes, const at::Tensor& src_tables, const at::Tensor& dst_tables,
                          const at::Tensor& tok_begin, const at::Tensor& tok_end, const OptTensor& exit_planes,
                          const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin, int64_t layer_end,
                          const OptTensor& status);

void kv_pack_cuda(const at::Tensor& key, const at::Tensor& value, const OptTensor& key_scale,
                  const OptTensor& value_scale, const at::Tensor& tables, const at::Tensor& tok_begin,
                  const at::Tensor& tok_end, const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode,
                  int64_t layer_begin, int64_t layer_end, at::Tensor& out, const OptTensor& status);

void kv_scatter_cuda(const at::Tensor& packed, const at::Tensor& tables, const at::Tensor& tok_begin,
                     const at::Tensor& tok_end, int64_t layer_begin, int64_t layer_end, at::Tensor& key,
                     at::Tensor& value, const OptTensor& key_scale, const OptTensor& value_scale,
                     const OptTensor& status);

void kv_handoff_slice_cuda(const at::Tensor& src_key, const at::Tensor& src_value, const OptTensor& src_key_scale,
                           const OptTensor& src_value_scale, at::Tensor& dst_key, at::Tensor& dst_value,
                           const OptTensor& dst_key_scale, const OptTensor& dst_value_scale, const at::Tensor& src_tables,
                           const at::Tensor& dst_tables, const at::Tensor& tok_begin, const at::Tensor& tok_end,
                           const OptTensor& exit_planes, const OptTensor& exit_offsets, int64_t mode, int64_t layer_begin,
                           int64_t layer_end, int64_t plane_begin, int64_t plane_end, const OptTensor& status);

void kv_pack_dedup_cuda(const at::Tensor& key, const at::Tensor& value, const OptTensor& key_scale,
                        const OptTensor& value_scale, const at::Tensor& tables, const at::Tensor& tok_begin,
                        const at::Tensor& tok_end, const at::Tensor& exit_planes, const at::Tensor& exit_offsets,
                        int64_t layer_begin, int64_t layer_end, at::Tensor& out, at::Tensor& workspace,
                        const OptTensor& status);

void kv_scatter_dedup_cuda(const at::Tensor& packed, const at::Tensor& tables, const at::Tensor& tok_begin,
                           const at::Tensor& tok_end, const at::Tensor& exit_planes, const at::Tensor& exit_offsets,
                           int64_t layer_begin, int64_t layer_end, at::Tensor& key, at::Tensor& value,
                           const OptTensor& key_scale, const OptTensor& value_scale, at::Tensor& workspace,
                           const OptTensor& status);

void kv_finalize_cuda(at::Tensor& key, at::Tensor& value, const OptTensor& key_scale, const OptTensor& value_scale,
                      const at::Tensor& tables, const at::Tensor& rows, int64_t layer_mask, const OptTensor& status);

void kv_push_cuda(const at::Tensor& src, int64_t dst_ptr, int64_t nbytes);
void kv_copy_segments_cuda(const at::Tensor& segments);
void kv_signal_cuda(const at::Tensor& anchor, int64_t flag_ptr, int64_t value);
void kv_wait_cuda(int64_t flag_ptr, int64_t value, int64_t timeout_ns, at::Tensor& status);

}  // namespace vllm_rlt_b200
