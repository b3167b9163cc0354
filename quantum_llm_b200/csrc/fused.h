// Launch interface of the fused row-wise kernels (kernels_fused.cu) and of the GEMV core
// calls that exchange quantised operands and split-K partials with them.
#pragma once

#include "gemv_mma.h"
#include "kernels.h"
#include "quant.cuh"

namespace qllm {

inline QuantSink no_sink() {
  QuantSink s{};
  s.kind = -1;
  return s;
}

struct NormQuantArgs {
  const float* x;            // input rows
  uint32_t x_stride;
  uint32_t cols;
  bool has_delta;            // x' = act(x + delta)
  GemvOut delta;
  bool bf16;
  float* store;              // optional: x' written here (the residual stream)
  uint32_t store_stride;
  const float* weight;       // norm weight; null = residual update only
  float eps;
  float* normalized;         // optional FP32 copy of the normalised rows
  uint32_t normalized_stride;
  bool round_normalized;     // round the normalised rows to BF16 before they are stored and quantised
  QuantSink sink;            // kind < 0: no quantised output
  uint32_t sink_block_offset;  // first 16-value block inside the operand row (concatenated inputs)
  const uint32_t* row_select;  // optional device index of the single input row
};
int launch_residual_norm_quant(const NormQuantArgs& a, uint32_t rows, cudaStream_t stream);

int launch_silu_quant(const GemvOut& gate_up, uint32_t ffn, bool bf16, const QuantSink& sink, float* inter,
                      cudaStream_t stream);

struct CombineArgs {
  const float* maxima;
  const float* sums;
  const float* outputs;
  const uint32_t* first_position;
  uint32_t position_offset;
  uint32_t q_heads, head_dim, split_tokens, max_splits;
  bool bf16;
  float* out;                // optional FP32 attention output [rows, q_heads*head_dim]
  QuantSink sink;
  uint32_t sink_row_offset;  // operand row of this launch's row 0 (a chunk merged in row tiles)
  uint32_t tiles;            // > 1: grid z = row tile; `rows` rows each, partials one tile after the other
  bool exact;                // exp from the deterministic series shared with the CPU oracle
};
int launch_combine_quant(const CombineArgs& c, uint32_t rows, cudaStream_t stream);

int launch_gemv_finalize(const GemvOut& o, float* y, cudaStream_t stream);

// RoPE + K/V store reading the fused qkv GEMV result; the rotated queries go to q_out
// [rows, q_heads*head_dim].
struct RopeStoreFusedArgs {
  GemvOut qkv;
  float* q_out;
  RopeStoreArgs base;        // qkv pointer unused
  // optional: INT8 copy of the rotated queries for the Q4H attention (scale = max(absmax/127,
  // 2^-24) per head, code = rn(q/scale)): [rows, q_heads, head_dim] and [rows, q_heads]
  int8_t* q8_out;
  float* q8_scale;
};
int launch_rope_kv_store_fused(const RopeStoreFusedArgs& a, cudaStream_t stream);

// ---- GEMV cores -------------------------------------------------------------------------
// Operand buffers: where a producer kernel writes the quantised activations of a GEMV.
size_t quant_buffer_bytes(uint32_t max_rows, uint32_t max_cols);
QuantSink make_sink(int gemv_impl, void* quant_buffer, uint32_t rows, uint32_t cols, float g);
size_t gemv_partial_floats(uint32_t batch, uint32_t rows, uint32_t cols);
// y = W . operand: CUDA-core kernel writes final values into `final_out`; the tensor-core
// kernel writes split-K partials into `partials`.  `out` describes the result for consumers.
// With `exchange` (tensor-core kernel only) the partials go to every rank's inbox instead.
int launch_gemv_core(int gemv_impl, const MmaWeights& w, const qllm_matrix& m, uint32_t first_row,
                     uint32_t row_count, uint32_t batch, void* quant_buffer, float* partials,
                     float* final_out, uint32_t* error, GemvOut* out, cudaStream_t stream,
                     const GemvExchange* exchange = nullptr, const struct RopeTail* rope_tail = nullptr);
// `rope_tail` (tensor-core kernel, decode steps): the projection is the fused q/k/v one and every
// head is rotated, quantised and stored by the CTA that finishes it (rope_tail.cuh); the caller
// then launches no separate RoPE / KV-store kernel.
bool gemv_rope_tail_supported(int gemv_impl, const MmaWeights& w, const qllm_matrix& m, uint32_t batch, uint32_t head_dim,
                              uint32_t rotary_dim);

}  // namespace qllm
