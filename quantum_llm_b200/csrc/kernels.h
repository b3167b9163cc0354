// Internal C++ launch interface of the kernel layer (one function per kernel
// family).  All pointers are device memory; every function returns 0 or a
// negative qllm_status and never synchronises.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/qllm_b200.h"

namespace qllm {

int launch_embedding(const uint16_t* table, const uint32_t* tokens, float* out, uint32_t rows,
                     uint32_t hidden, uint32_t vocab, cudaStream_t stream);
int launch_rms_norm(const float* x, const float* weight, float* out, uint32_t rows, uint32_t cols,
                    uint32_t in_stride, uint32_t out_stride, float eps,
                    const uint32_t* row_select, cudaStream_t stream);
int launch_fake_quant(const float* x, float* out, uint32_t rows, uint32_t cols, float g,
                      cudaStream_t stream);
// Quantised activations of the CUDA-core GEMV: INT8 (twice the E2M1 value) [rows, cols]
// followed by FP32 block scales [rows, cols/16].
size_t act_quant_bytes(uint32_t rows, uint32_t cols);
int launch_act_quant_i8(const float* x, void* qact, uint32_t rows, uint32_t cols, float g,
                        cudaStream_t stream);
int launch_gemv_simt(const qllm_matrix& m, uint32_t first_row, uint32_t row_count, const void* qact,
                     uint32_t qact_rows, float* y, uint32_t batch, cudaStream_t stream);
int launch_quantize_weights(const float* w, uint32_t rows, uint32_t cols, float g, uint8_t* codes,
                            uint8_t* scales, cudaStream_t stream);
int launch_add(float* dst, const float* src, uint64_t count, bool bf16, cudaStream_t stream);
int launch_silu_product(const float* gate_up, float* out, uint32_t rows, uint32_t ffn, bool bf16,
                        cudaStream_t stream);
int launch_copy_rows(float* dst, uint32_t dst_stride, const float* src, uint32_t src_stride,
                     uint32_t rows, uint32_t cols, const uint32_t* row_select, cudaStream_t stream);
int launch_argmax(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride,
                  uint32_t* out, cudaStream_t stream);
size_t topk_workspace_bytes(uint32_t rows, uint32_t count, uint32_t k);
int launch_topk(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride, uint32_t k,
                float* out_values, uint32_t* out_tokens, void* workspace, cudaStream_t stream);

// ---- attention -----------------------------------------------------------
size_t kv_layer_bytes(uint32_t encoding, uint32_t page_tokens, uint32_t kv_heads, uint32_t head_dim);
struct RopeStoreArgs {
  float* qkv;                 // [rows, (q+2kv)*head_dim]
  uint32_t rows, q_heads, kv_heads, head_dim, rotary_dim;
  const float* inv_freq;      // [rotary_dim/2]
  const uint32_t* first_position;  // device scalar
  uint32_t position_offset;   // cache position of row r = *first_position + position_offset + r
  uint32_t rotary_offset;     // rotary position = cache position + rotary_offset
  uint8_t* const* page_table;
  size_t layer_offset;
  uint32_t page_tokens, encoding;
  bool bf16;
  // sin / cos from the deterministic double-precision series (the same bits as the CPU oracle)
  // instead of the device's single-precision library functions
  bool exact;
};
int launch_rope_kv_store(const RopeStoreArgs& a, cudaStream_t stream);

struct AttentionArgs {
  uint32_t encoding;
  const uint8_t* const* page_table;
  size_t layer_offset;
  uint32_t page_tokens;
  const float* query;         // row r, head h at query + r*query_row_stride + h*head_dim
  uint32_t query_row_stride;
  uint32_t rows;
  const uint32_t* first_position;  // device scalar; row r sees *first_position + position_offset + r + 1 tokens
  uint32_t position_offset;
  uint32_t q_heads, kv_heads, head_dim;
  uint32_t split_tokens, max_splits;
  bool bf16;
  void* workspace;
  float* out;                 // [rows, q_heads*head_dim]
  int impl;                   // 0 scalar, 1 tensor cores through mma.sync, 2 tcgen05 + tensor memory (Q4H; else as 1)
  uint32_t* error;            // optional device status word (set when a pipeline wait runs out)
  bool skip_combine;          // leave the per-split partials in the workspace (merged by the caller)
  // optional (tensor-core Q4H path): queries already quantised to INT8 by the RoPE kernel,
  // [rows, q_heads, head_dim] codes and [rows, q_heads] scales; null = quantise from `query`
  const int8_t* query_q8;
  const float* query_q8_scale;
  // > 1: one launch over `tiles` consecutive row tiles of `rows` rows each (grid z): tile z holds
  // rows z*rows.. of the pass (queries, positions) and its partials follow tile z-1's in the workspace
  uint32_t tiles;
};
// Floats in the maxima (and in the sums) section of the split partials [maxima][sums][outputs] of one
// row tile: rows x splits x heads rounded up to a multiple of four, so that the outputs section,
// which the kernels read and write as float4, starts on a 16-byte boundary for every head count
// (5 query heads, one row, 65 splits gave an odd count and a misaligned section).
#if defined(__CUDACC__)
__host__ __device__
#endif
inline size_t attention_partial_items(uint32_t rows, uint32_t max_splits, uint32_t q_heads) {
  return (static_cast<size_t>(rows) * max_splits * q_heads + 3U) & ~static_cast<size_t>(3U);
}
#ifdef __CUDACC__
// Entry of every attention kernel: moves the arguments to the row tile of this block.
template <typename P>
__device__ __forceinline__ void attention_row_tile(AttentionArgs& a, P& part) {
  const uint32_t z = blockIdx.z;
  if (z == 0U) return;
  const uint32_t r0 = z * a.rows;
  const size_t shift = z * attention_partial_items(a.rows, a.max_splits, a.q_heads) * (2U + a.head_dim);
  part.maxima += shift;
  part.sums += shift;
  part.outputs += shift;
  a.query += static_cast<size_t>(r0) * a.query_row_stride;
  if (a.query_q8) {
    a.query_q8 += static_cast<size_t>(r0) * a.q_heads * a.head_dim;
    a.query_q8_scale += static_cast<size_t>(r0) * a.q_heads;
  }
  a.position_offset += r0;
}
#endif
int launch_attention_q4h_pipelined(const AttentionArgs& a, float* maxima, float* sums, float* outputs,
                                   uint32_t* error, cudaStream_t stream);
// tcgen05 (tensor memory) kernel over the Q4H cache: head_dim 128, rows * group <= 32, 128-token
// aligned pages and splits.  `scratch` (attention_q4h_tc_query_bytes) holds the INT8 queries when the
// caller passes FP32 queries only.
bool attention_q4h_tc_supported(const AttentionArgs& a);
size_t attention_q4h_tc_query_bytes(uint32_t rows, uint32_t q_heads);
int launch_attention_q4h_tc(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                            void* scratch, cudaStream_t stream);
// BF16 tensor-core kernel over the Q8 cache (head_dim 128, at most 8 kv heads).
bool attention_q8_mma_supported(const AttentionArgs& a);
int launch_attention_q8_mma(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                            cudaStream_t stream);
// F16 tensor-core kernel over the exact-F16 cache (head_dim 128).
bool attention_f16_mma_supported(const AttentionArgs& a);
int launch_attention_f16_mma(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                             cudaStream_t stream);
size_t attention_workspace_bytes(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                                 uint32_t max_splits);
int launch_attention(const AttentionArgs& a, cudaStream_t stream);
int launch_fill_synthetic_kv(uint8_t* const* page_table, size_t layer_offset, uint32_t encoding,
                             uint32_t page_tokens, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t first, uint32_t count, uint64_t seed, cudaStream_t stream);

// ---- sampler --------------------------------------------------------------
// Device-resident request/step state; layout shared with the provider.
struct DraftDistribution {
  uint32_t count;
  uint32_t pad;
  uint32_t tokens[64];
  double probabilities[64];
};
struct StepState {
  // request parameters
  unsigned long long seed;
  uint32_t temperature_ppm, top_p_ppm, top_k, min_p_ppm, context_limit, draft_depth;
  // cursor
  uint32_t position;        // position of verify_tokens[0]; also the draft cache length
  uint32_t draft_count;     // proposals available for the next verify
  uint32_t verify_tokens[8];
  // outputs of the acceptance kernel
  uint32_t accepted, next_token, rejected, new_position;
  uint32_t mtp_tokens[8];   // accepted drafts + next token, padded with next token
  uint32_t mtp_rows;        // accepted + 1
  uint32_t error;           // sticky: non-zero when a kernel met an invalid state
  uint32_t step_index;      // results ring cursor
  uint32_t pad;
  unsigned long long exact_calls, accepted_drafts, accepted_depth_calls[5];
  DraftDistribution drafts[4];
};
// One ring entry per step: the result the caller reads plus the state summary the host
// mirror needs, so that one small device-to-host copy ends a step.
struct StepRecord {
  qllm_exact_result result;
  uint32_t draft_count;  // proposals ready for the next step
  uint32_t error;        // StepState::error after the step
};
struct AcceptArgs {
  StepState* state;
  const uint32_t* argmax_tokens;  // [rows] (greedy)
  const float* top_values;        // [rows, top_k] (sampling)
  const uint32_t* top_tokens;
  StepRecord* results;            // device ring [results_capacity]
  uint32_t results_capacity;
};
int launch_accept(const AcceptArgs& a, cudaStream_t stream);
struct DraftSampleArgs {
  StepState* state;
  const uint32_t* argmax_token;   // [1] (greedy)
  const float* top_values;        // [top_k]
  const uint32_t* top_tokens;
  uint32_t pass;                  // 0 = first draft pass of a step, 1.. = chained passes
  uint32_t from_sync;             // 1: called from a synchronisation batch (position is final)
  StepRecord* results;            // ring of the acceptance kernel (may be null)
  uint32_t results_capacity;
  const uint32_t* kernel_error;   // status word of the pipelined kernels, folded into the state
};
int launch_draft_sample(const DraftSampleArgs& a, cudaStream_t stream);
int launch_first_token(StepState* state, const uint32_t* argmax_token, const float* top_values,
                       const uint32_t* top_tokens, uint32_t sample_position, uint32_t* out,
                       cudaStream_t stream);
// Scalar decode fallback (top_k == 0 or > 64): full-vocabulary ordering + the sequential
// double-precision distribution of sample_token (dense_fp4_provider.cpp:771-802) on the device.
// Presence penalty over `rows` logits rows of `stride` floats, the first `count` entries of each:
// mode 0: tokens of the emitted mask; mode 1: verify rows -- row r also sees the step's proposals
// 1..r (StepState::verify_tokens); mode 2: draft pass `pass` -- also the drafts 1..pass of the
// running rollout.  In place, like the reference's kernel.
struct PresenceArgs {
  float* logits;
  uint32_t rows;
  size_t stride;
  uint32_t count;
  const uint8_t* emitted;   // [vocabulary] bytes, non-zero = emitted
  const StepState* state;   // device; may be null for mode 0
  uint32_t mode, pass;
  float penalty;            // [-2, 2]
};
int launch_presence_penalty(const PresenceArgs& a, cudaStream_t stream);
int launch_presence_commit_step(const StepState* state, uint8_t* emitted, uint32_t vocab, cudaStream_t stream);
int launch_presence_commit_token(const uint32_t* token, uint8_t* emitted, uint32_t vocab, cudaStream_t stream);

struct FullSampleParams {
  unsigned long long seed;
  uint32_t temperature_ppm, top_p_ppm, top_k, min_p_ppm;   // top_k 0 = the whole vocabulary
  uint32_t sample_position;
};
size_t full_sampler_workspace_bytes(uint32_t vocab);
// *error = 5 when the candidates hold no finite mass (the reference throws); *out: the token.
int launch_full_vocabulary_sample(const FullSampleParams& q, const float* logits, uint32_t vocab, void* workspace,
                                  uint32_t* error, uint32_t* out, cudaStream_t stream);

}  // namespace qllm
