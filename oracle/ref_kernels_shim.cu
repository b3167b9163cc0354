// C entry points over the reference's own CUDA kernels -- TEST INFRASTRUCTURE ONLY.
//
// oracle/Makefile (target `ref_kernels`) compiles the reference's
// runtime/src/cuda/transformer_kernels.cu, unmodified and from where it lies, for sm_100a
// together with this file into oracle/_ref/libqllm_ref_kernels.so.  The GPU parity tests run
// those kernels on small cases of the reference's own smoke fixtures and compare the CPU
// oracle, and this library's kernels, with what they produce.  Nothing in the shipped
// library links, loads or calls this file.
//
// Every pointer is device memory; every call runs on the default stream, waits for it and
// returns 0, or -1 with the text in qr_last_error().
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "expert/runtime/cuda/flash_attention.hpp"
#include "expert/runtime/cuda/transformer_kernels.hpp"

namespace rc = expert::runtime::cuda;

// The reference's prompt path calls into its vendored FlashAttention translation unit, which is not
// part of this build (it needs CUTLASS); nothing here reaches that call.  Defined so that the
// library loads.
namespace expert::runtime::cuda {
Status flash_gqa_segment_bf16(const FlashGqaSegmentLaunch&) noexcept {
  return Status(ErrorCode::invalid_argument, "flash attention is not part of the reference-kernel shim");
}
}  // namespace expert::runtime::cuda

namespace {
thread_local std::string g_error;

int done(const expert::runtime::Status& status) {
  if (!status.ok()) {
    g_error = std::string(status.message());
    return -1;
  }
  const cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    g_error = cudaGetErrorString(e);
    return -1;
  }
  return 0;
}
}  // namespace

extern "C" {

const char* qr_last_error(void) { return g_error.c_str(); }

// nvfp4_gemv_f32_batch (transformer_kernels.cu:7970; kernels :1943, :1970)
int qr_nvfp4_gemv(const uint8_t* codes, const uint8_t* scales, float weight_scale, float input_scale, uint32_t rows,
                  uint32_t cols, const float* x, float* y, float* quantized_dequantized_x, uint32_t batch) {
  rc::Nvfp4Block16Matrix m{};
  m.weights = codes;
  m.scales = scales;
  m.weight_global_scale = weight_scale;
  m.input_global_scale = input_scale;
  m.rows = rows;
  m.columns = cols;
  return done(rc::nvfp4_gemv_f32_batch(m, x, y, quantized_dequantized_x, batch, nullptr));
}

// store_gqa_kv_paged_q4_per_head_batch (:8480; record :229-288): head_dim 256 only
int qr_store_q4h(const float* key, const float* value, const void* const* page_table, uint32_t layer,
                 uint32_t page_tokens, uint32_t first_cache_position, uint32_t rows, uint32_t kv_heads,
                 uint32_t head_dim) {
  return done(rc::store_gqa_kv_paged_q4_per_head_batch(key, value, page_table, layer, page_tokens,
                                                       first_cache_position, rows, kv_heads, head_dim, nullptr));
}

// store_gqa_kv_paged_q8_batch (record :601-625)
int qr_store_q8(const float* key, const float* value, const void* const* page_table, uint32_t layer,
                uint32_t page_tokens, uint32_t first_cache_position, uint32_t rows, uint32_t kv_heads,
                uint32_t head_dim) {
  return done(rc::store_gqa_kv_paged_q8_batch(key, value, page_table, layer, page_tokens, first_cache_position,
                                              rows, kv_heads, head_dim, nullptr));
}

// quantize_gqa_queries_q8 (:9537; kernel :4391): q_and_gate is [rows, heads, 2*head_dim]
int qr_quantize_queries_q8(const float* q_and_gate, int8_t* q8, float* scales, uint32_t rows, uint32_t q_heads,
                           uint32_t head_dim) {
  return done(rc::quantize_gqa_queries_q8(q_and_gate, q8, scales, rows, q_heads, head_dim, nullptr));
}

// gated_gqa_attention_microbatch_paged_q4_per_head_tensor_core (:9553-9651; kernels :4421-4976, :5741)
int qr_attention_q4h(const float* q_and_gate, const int8_t* q8, const float* query_scales,
                     const void* const* page_table, float* output, float* partial_maxima, float* partial_sums,
                     float* partial_outputs, uint32_t first_context_tokens, uint32_t rows, uint32_t layer,
                     uint32_t page_tokens, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                     uint32_t split_tokens, uint32_t maximum_splits, int bf16_activations) {
  rc::PagedQ4BfpGatedGqaAttentionLaunch l{};
  l.q_and_gate = q_and_gate;
  l.q8_queries = q8;
  l.query_scales = query_scales;
  l.page_table = page_table;
  l.output = output;
  l.partial_maxima = partial_maxima;
  l.partial_sums = partial_sums;
  l.partial_outputs = partial_outputs;
  l.first_context_tokens = first_context_tokens;
  l.rows = rows;
  l.full_attention_layer = layer;
  l.page_tokens = page_tokens;
  l.query_heads = q_heads;
  l.kv_heads = kv_heads;
  l.head_dim = head_dim;
  l.split_tokens = split_tokens;
  l.maximum_splits = maximum_splits;
  l.stream = nullptr;
  l.bf16_activations = bf16_activations != 0;
  return done(rc::gated_gqa_attention_microbatch_paged_q4_per_head_tensor_core(l));
}

// gated_gqa_attention_microbatch_paged_q8_tensor_core (:9852; impl :9736)
int qr_attention_q8(const float* q_and_gate, const void* const* page_table, float* output, float* partial_maxima,
                    float* partial_sums, float* partial_outputs, uint32_t first_context_tokens, uint32_t rows,
                    uint32_t layer, uint32_t page_tokens, uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                    uint32_t split_tokens, uint32_t maximum_splits, int bf16_activations) {
  rc::PagedQ8GatedGqaPrefillLaunch l{};
  l.q_and_gate = q_and_gate;
  l.page_table = page_table;
  l.output = output;
  l.partial_maxima = partial_maxima;
  l.partial_sums = partial_sums;
  l.partial_outputs = partial_outputs;
  l.first_context_tokens = first_context_tokens;
  l.rows = rows;
  l.full_attention_layer = layer;
  l.page_tokens = page_tokens;
  l.query_heads = q_heads;
  l.kv_heads = kv_heads;
  l.head_dim = head_dim;
  l.split_tokens = split_tokens;
  l.maximum_splits = maximum_splits;
  l.stream = nullptr;
  l.bf16_activations = bf16_activations != 0;
  return done(rc::gated_gqa_attention_microbatch_paged_q8_tensor_core(l));
}

// argmax_batch, topk_logits (:10737-10783; kernels :7059-7178)
int qr_argmax_batch(const float* values, uint32_t count, uint32_t batch, uint32_t* output) {
  return done(rc::argmax_batch(values, count, batch, output, nullptr));
}
size_t qr_topk_workspace_items(uint32_t count) { return rc::topk_logits_workspace_items(count); }
int qr_topk(const float* values, uint32_t count, uint32_t top_k, float* out_values, uint32_t* out_indices,
            float* workspace_values, size_t workspace_values_bytes, uint32_t* workspace_indices,
            size_t workspace_indices_bytes) {
  rc::TopKLogitsWorkspace w{};
  w.values = workspace_values;
  w.values_bytes = workspace_values_bytes;
  w.indices = workspace_indices;
  w.indices_bytes = workspace_indices_bytes;
  return done(rc::topk_logits(values, count, top_k, out_values, out_indices, w, nullptr));
}

}  // extern "C"
