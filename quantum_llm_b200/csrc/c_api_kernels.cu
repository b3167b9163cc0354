// extern "C" forms of the kernel launchers declared in include/qllm_b200.h.
#include <string>

#include "common.cuh"
#include "gemv_mma.h"
#include "kernels.h"
#include "moe.h"

using namespace qllm;

extern "C" {

int qllm_k_embedding_bf16(const uint16_t* table, const uint32_t* tokens, float* out, uint32_t rows,
                          uint32_t hidden, uint32_t vocab, void* stream) {
  if (!table || !tokens || !out || !rows || !hidden || !vocab)
    return fail(QLLM_INVALID_ARGUMENT, "invalid embedding batch");
  return launch_embedding(table, tokens, out, rows, hidden, vocab, static_cast<cudaStream_t>(stream));
}

int qllm_k_rms_norm(const float* x, const float* weight, float* out, uint32_t rows, uint32_t cols,
                    float eps, void* stream) {
  if (!x || !weight || !out || !rows || !cols) return fail(QLLM_INVALID_ARGUMENT, "invalid RMSNorm batch");
  return launch_rms_norm(x, weight, out, rows, cols, cols, cols, eps, nullptr, static_cast<cudaStream_t>(stream));
}

int qllm_k_nvfp4_fake_quant(const float* x, float* out, uint32_t rows, uint32_t cols,
                            float global_scale, void* stream) {
  if (!x || !out || !rows || !cols || cols % 16U || !(global_scale > 0.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 activation quant-dequant");
  return launch_fake_quant(x, out, rows, cols, global_scale, static_cast<cudaStream_t>(stream));
}

size_t qllm_k_nvfp4_gemv_workspace_bytes(uint32_t batch, uint32_t rows, uint32_t cols) {
  const size_t simt = act_quant_bytes(batch, cols);
  const size_t mma = gemv_mma_workspace_bytes(batch, rows, cols);
  return simt > mma ? simt : mma;
}

int qllm_k_nvfp4_gemv(const qllm_matrix* m, uint32_t first_row, uint32_t row_count, const float* x,
                      float* y, uint32_t batch, void* workspace, size_t workspace_bytes, int impl,
                      void* stream) {
  if (!m || !m->codes || !m->scales || !x || !y || !workspace || !m->rows || !m->cols ||
      m->cols % 16U || !batch || !row_count || row_count > m->rows || first_row > m->rows - row_count ||
      !(m->weight_scale > 0.0F) || !(m->input_scale > 0.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 GEMV");
  // the kernels read x as float4, the codes as uint2 and the workspace as uint4
  if ((reinterpret_cast<uintptr_t>(x) & 15U) || (reinterpret_cast<uintptr_t>(m->codes) & 7U) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15U))
    return fail(QLLM_INVALID_ARGUMENT,
                "native NVFP4 GEMV needs x and the workspace on 16-byte and the codes on 8-byte boundaries");
  if (workspace_bytes < qllm_k_nvfp4_gemv_workspace_bytes(batch, row_count, m->cols))
    return fail(QLLM_INVALID_ARGUMENT, "native NVFP4 GEMV workspace is too small");
  auto s = static_cast<cudaStream_t>(stream);
  if (impl == 0) {
    int rc = launch_act_quant_i8(x, workspace, batch, m->cols, m->input_scale, s);
    if (rc) return rc;
    return launch_gemv_simt(*m, first_row, row_count, workspace, batch, y, batch, s);
  }
  if (impl == 1) {
    // one-shot form: build the tensor map and the re-tiled scales for this call
    MmaWeights w;
    int rc = w.prepare(*m, s);
    if (rc) return rc;
    if (!w.ready) return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64)");
    rc = check_cuda(cudaMemsetAsync(workspace, 0, sizeof(uint32_t), s), "clear GEMV status word");
    if (rc) return rc;
    rc = launch_gemv_mma(w, *m, first_row, row_count, x, y, batch, workspace, workspace_bytes, s);
    if (rc) return rc;
    uint32_t status = 0;
    rc = check_cuda(cudaMemcpyAsync(&status, workspace, sizeof(status), cudaMemcpyDeviceToHost, s), "read GEMV status");
    if (rc) return rc;
    rc = check_cuda(cudaStreamSynchronize(s), "native NVFP4 tensor-core GEMV");
    if (rc) return rc;
    if (status) return fail(QLLM_INTERNAL, "tensor-core GEMV pipeline wait ran out (status " + std::to_string(status) + ")");
    return 0;
  }
  return fail(QLLM_INVALID_ARGUMENT, "unknown GEMV implementation");
}

struct qllm_prepared_matrix {
  qllm_matrix m;
  MmaWeights mma;
};

int qllm_k_matrix_prepare(const qllm_matrix* m, void* stream, qllm_prepared_matrix** out) {
  if (!m || !out || !m->codes || !m->scales || !m->rows || !m->cols || m->cols % 16U)
    return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 matrix");
  auto* p = new qllm_prepared_matrix;
  p->m = *m;
  const int rc = p->mma.prepare(*m, static_cast<cudaStream_t>(stream));
  if (rc) {
    delete p;
    return rc;
  }
  *out = p;
  return 0;
}

void qllm_k_matrix_release(qllm_prepared_matrix* p) { delete p; }

int qllm_k_nvfp4_gemv_prepared(const qllm_prepared_matrix* p, const float* x, float* y, uint32_t batch,
                               void* workspace, size_t workspace_bytes, int impl, void* stream) {
  if (!p || !x || !y || !workspace || !batch) return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 GEMV");
  if (workspace_bytes < qllm_k_nvfp4_gemv_workspace_bytes(batch, p->m.rows, p->m.cols))
    return fail(QLLM_INVALID_ARGUMENT, "native NVFP4 GEMV workspace is too small");
  auto s = static_cast<cudaStream_t>(stream);
  if (impl == 0) {
    int rc = launch_act_quant_i8(x, workspace, batch, p->m.cols, p->m.input_scale, s);
    if (rc) return rc;
    return launch_gemv_simt(p->m, 0U, p->m.rows, workspace, batch, y, batch, s);
  }
  if (impl != 1 || !p->mma.ready) return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64)");
  return launch_gemv_mma(p->mma, p->m, 0U, p->m.rows, x, y, batch, workspace, workspace_bytes, s);
}

int qllm_k_nvfp4_gemv_prepared_core(const qllm_prepared_matrix* p, uint32_t batch, void* workspace,
                                    size_t workspace_bytes, void* stream) {
  if (!p || !workspace || !batch) return fail(QLLM_INVALID_ARGUMENT, "invalid native NVFP4 GEMV");
  if (!p->mma.ready) return fail(QLLM_INVALID_ARGUMENT, "shape is outside the tensor-core GEMV (K % 64)");
  return launch_gemv_mma_core_only(p->mma, p->m, batch, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int qllm_k_nvfp4_quantize_weights(const float* w, uint32_t rows, uint32_t cols, float global_scale,
                                  uint8_t* codes, uint8_t* scales, void* stream) {
  if (!w || !codes || !scales || !rows || !cols || cols % 16U || !(global_scale > 0.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid NVFP4 weight quantisation");
  return launch_quantize_weights(w, rows, cols, global_scale, codes, scales, static_cast<cudaStream_t>(stream));
}

int qllm_k_add(float* dst, const float* src, uint64_t count, int bf16, void* stream) {
  if (!dst || !src || !count) return fail(QLLM_INVALID_ARGUMENT, "invalid add");
  return launch_add(dst, src, count, bf16 != 0, static_cast<cudaStream_t>(stream));
}

int qllm_k_silu_product(const float* gate_up, float* out, uint32_t rows, uint32_t ffn, int bf16,
                        void* stream) {
  if (!gate_up || !out || !rows || !ffn) return fail(QLLM_INVALID_ARGUMENT, "invalid SiLU product");
  return launch_silu_product(gate_up, out, rows, ffn, bf16 != 0, static_cast<cudaStream_t>(stream));
}

int qllm_k_rope_kv_store(float* qkv, uint32_t rows, uint32_t q_heads, uint32_t kv_heads,
                         uint32_t head_dim, uint32_t rotary_dim, const float* inv_freq,
                         const uint32_t* first_position, uint32_t position_offset,
                         uint32_t rotary_offset, uint8_t* const* page_table, size_t layer_offset,
                         uint32_t page_tokens, uint32_t encoding, int bf16, void* stream) {
  if (!qkv || !rows || !q_heads || !kv_heads || !inv_freq || !first_position || !page_table ||
      !page_tokens || encoding > 2U)
    return fail(QLLM_INVALID_ARGUMENT, "invalid RoPE/KV store batch");
  RopeStoreArgs a{qkv, rows, q_heads, kv_heads, head_dim, rotary_dim, inv_freq, first_position,
                  position_offset, rotary_offset, page_table, layer_offset, page_tokens, encoding,
                  bf16 != 0, true};
  return launch_rope_kv_store(a, static_cast<cudaStream_t>(stream));
}

size_t qllm_k_kv_layer_bytes(uint32_t encoding, uint32_t page_tokens, uint32_t kv_heads,
                             uint32_t head_dim) {
  return kv_layer_bytes(encoding, page_tokens, kv_heads, head_dim);
}

size_t qllm_k_attention_workspace_bytes(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                                        uint32_t max_splits) {
  return attention_workspace_bytes(rows, q_heads, head_dim, max_splits);
}

int qllm_k_attention(uint32_t encoding, const uint8_t* const* page_table, size_t layer_offset,
                     uint32_t page_tokens, const float* query, uint32_t query_row_stride,
                     uint32_t rows, const uint32_t* first_position, uint32_t position_offset,
                     uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim, uint32_t split_tokens,
                     uint32_t max_splits, int bf16, void* workspace, float* out, int impl,
                     void* stream) {
  if (!page_table || !query || !first_position || !workspace || !out || !kv_heads)
    return fail(QLLM_INVALID_ARGUMENT, "invalid attention launch");
  AttentionArgs a{};
  a.encoding = encoding;
  a.page_table = page_table;
  a.layer_offset = layer_offset;
  a.page_tokens = page_tokens;
  a.query = query;
  a.query_row_stride = query_row_stride;
  a.rows = rows;
  a.first_position = first_position;
  a.position_offset = position_offset;
  a.q_heads = q_heads;
  a.kv_heads = kv_heads;
  a.head_dim = head_dim;
  a.split_tokens = split_tokens;
  a.max_splits = max_splits;
  a.bf16 = bf16 != 0;
  a.workspace = workspace;
  a.out = out;
  a.impl = impl;
  return launch_attention(a, static_cast<cudaStream_t>(stream));
}

int qllm_k_argmax(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride,
                  uint32_t* out, void* stream) {
  if (!values || !rows || !count || !out) return fail(QLLM_INVALID_ARGUMENT, "invalid argmax");
  return launch_argmax(values, rows, count, row_stride, out, static_cast<cudaStream_t>(stream));
}

int qllm_k_moe_route(const float* logits, uint32_t rows, uint32_t experts, uint32_t top_k, float route_scale,
                     uint32_t* indices, float* scores, void* stream) {
  if (!logits || !indices || !scores || !rows || !(route_scale > 0.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid router selection");
  GemvOut values{};
  values.data = logits;  // final values, row-major [rows, experts]
  values.split = 0U;
  values.n = experts;
  values.batch = rows;
  values.weight_scale = values.input_scale = 1.0F;
  MoeArgs a{};
  a.rows = rows;
  a.experts = experts;
  a.route_width = top_k;
  a.route_scale = route_scale;
  a.indices = indices;
  a.scores = scores;
  return launch_moe_router_select(values, a, static_cast<cudaStream_t>(stream));
}

size_t qllm_k_topk_workspace_bytes(uint32_t rows, uint32_t count, uint32_t k) {
  return topk_workspace_bytes(rows, count, k);
}

int qllm_k_topk(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride, uint32_t k,
                float* out_values, uint32_t* out_tokens, void* workspace, void* stream) {
  if (!values || !rows || !count || !k || k > 64U || k > count || !out_values || !out_tokens || !workspace)
    return fail(QLLM_INVALID_ARGUMENT, "invalid top-k");
  return launch_topk(values, rows, count, row_stride, k, out_values, out_tokens, workspace,
                     static_cast<cudaStream_t>(stream));
}

size_t qllm_k_sample_token_workspace_bytes(uint32_t vocabulary) { return full_sampler_workspace_bytes(vocabulary); }

int qllm_k_sample_token(const float* logits, uint32_t vocabulary, uint64_t seed, uint32_t temperature_ppm,
                        uint32_t top_p_ppm, uint32_t top_k, uint32_t min_p_ppm, uint32_t position,
                        void* workspace, uint32_t* status, uint32_t* token, void* stream) {
  if (!logits || !vocabulary || !workspace || !status || !token || top_k > vocabulary)
    return fail(QLLM_INVALID_ARGUMENT, "invalid token sampling contract");
  const FullSampleParams q{seed, temperature_ppm, top_p_ppm, top_k, min_p_ppm, position};
  return launch_full_vocabulary_sample(q, logits, vocabulary, workspace, status, token,
                                       static_cast<cudaStream_t>(stream));
}

}  // extern "C"
