// Fused row-wise kernels between the GEMVs of a decode step.  Each one consumes a GEMV
// result (final values or split-K partials), applies the reference's element-wise step with
// its BF16 rounding points, and writes the NEXT GEMV's quantised NVFP4 operand directly, so a
// transformer block is ten launches instead of eighteen:
//   residual add + RMSNorm + quantise      (add_kernel, rms_batch_kernel, nvfp4_quant_dequant_kernel;
//                                           runtime/src/cuda/transformer_kernels.cu:2522, 2487, 1943)
//   SiLU(gate)*up + quantise               (silu_product_kernel 2774)
//   split combine + quantise               (combine kernel 5741)
#include "common.cuh"
#include "fused.h"

namespace qllm {

// ---------------------------------------------------- residual + norm + quantise
// One CTA per row.  x' = act(x + delta) (delta optional), optionally stored back; then
// n = x' * rsqrt(mean x'^2 + eps) * w, optionally stored; then the NVFP4 operand of n.
__global__ void __launch_bounds__(512)
residual_norm_quant_kernel(NormQuantArgs a) {
  extern __shared__ float rowbuf[];
  __shared__ double partial[16];
  const uint32_t out_row = blockIdx.x;
  const uint32_t in_row = a.row_select ? *a.row_select : out_row;
  // x == null: the row is the GEMV result alone (0 + delta is exact)
  const float* x = a.x ? a.x + static_cast<size_t>(in_row) * a.x_stride : nullptr;
  double sq = 0.0;
  for (uint32_t i = threadIdx.x; i < a.cols; i += blockDim.x) {
    float v = x ? x[i] : 0.0F;
    if (a.has_delta) v = actv(v + gemv_value(a.delta, in_row, i), a.bf16);
    if (a.store) a.store[static_cast<size_t>(out_row) * a.store_stride + i] = v;
    rowbuf[i] = v;
    sq += static_cast<double>(v) * static_cast<double>(v);
  }
  sq = warp_sum_f64(sq);
  if ((threadIdx.x & 31U) == 0U) partial[threadIdx.x >> 5U] = sq;
  __syncthreads();
  if (threadIdx.x < 32U) {
    double v = threadIdx.x < (blockDim.x >> 5U) ? partial[threadIdx.x] : 0.0;
    v = warp_sum_f64(v);
    if (threadIdx.x == 0U) partial[0] = v;
  }
  __syncthreads();
  if (!a.weight) return;  // residual update only
  const float inverse = 1.0F / sqrtf(static_cast<float>(partial[0]) / static_cast<float>(a.cols) + a.eps);
  for (uint32_t b = threadIdx.x; b < a.cols / 16U; b += blockDim.x) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = rowbuf[b * 16U + i] * inverse * a.weight[b * 16U + i];
    if (a.normalized) {
      float4* o = reinterpret_cast<float4*>(a.normalized + static_cast<size_t>(out_row) * a.normalized_stride + b * 16U);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    }
    if (a.sink.kind >= 0) quant_store_block16(a.sink, out_row, a.sink_block_offset + b, v);
  }
}

int launch_residual_norm_quant(const NormQuantArgs& a, uint32_t rows, cudaStream_t stream) {
  if (!rows || !a.cols || a.cols % 16U || a.cols > 12288U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported row length for the fused norm");
  residual_norm_quant_kernel<<<rows, 512, a.cols * sizeof(float), stream>>>(a);
  count_launch();
  return check_launch("residual_norm_quant");
}

// ------------------------------------------------------------ SiLU product + quantise
// One thread per (row, 16 outputs): inter = act(act(silu(g)) * u), quantised for the down GEMV.
__global__ void silu_quant_kernel(GemvOut gate_up, uint32_t ffn, bool bf16, QuantSink sink, float* inter) {
  const uint32_t blocks = ffn / 16U;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  if (item >= gate_up.batch * blocks) return;
  const uint32_t row = item / blocks, b = item % blocks;
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float g = gemv_value(gate_up, row, b * 16U + i);
    const float u = gemv_value(gate_up, row, ffn + b * 16U + i);
    const float s = actv(g / (1.0F + expf(-g)), bf16);
    v[i] = actv(s * u, bf16);
  }
  if (inter) {
#pragma unroll
    for (int i = 0; i < 16; ++i) inter[static_cast<size_t>(row) * ffn + b * 16U + i] = v[i];
  }
  quant_store_block16(sink, row, b, v);
}

int launch_silu_quant(const GemvOut& gate_up, uint32_t ffn, bool bf16, const QuantSink& sink, float* inter,
                      cudaStream_t stream) {
  const uint32_t items = gate_up.batch * (ffn / 16U);
  silu_quant_kernel<<<(items + 127U) / 128U, 128, 0, stream>>>(gate_up, ffn, bf16, sink, inter);
  count_launch();
  return check_launch("silu_quant");
}

// ------------------------------------------------------------- split combine + quantise
// grid (q_heads, rows), block head_dim.  Merges the context splits by log-sum-exp (sums in
// double: independent of the visiting order) and writes the o-projection operand.
__global__ void combine_quant_kernel(CombineArgs c) {
  __shared__ float weights[512];
  __shared__ float values[256];
  __shared__ float gmax_s, gsum_s;
  const uint32_t head = blockIdx.x, row = blockIdx.y, d = threadIdx.x, hd = c.head_dim;
  const uint32_t ctx = *c.first_position + c.position_offset + 1U + row;
  const uint32_t active = (ctx + c.split_tokens - 1U) / c.split_tokens;
  const size_t base = static_cast<size_t>(row) * c.max_splits * c.q_heads + head;
  // warp 0: maximum over the splits, then the split weights and their sum
  if (d < 32U) {
    float m = kNegInf;
    for (uint32_t s = d; s < active; s += 32U) m = fmaxf(m, c.maxima[base + static_cast<size_t>(s) * c.q_heads]);
    m = warp_max(m);
    double sum = 0.0;
    for (uint32_t s = d; s < active; s += 32U) {
      const size_t p = base + static_cast<size_t>(s) * c.q_heads;
      const float w = expf(c.maxima[p] - m);
      weights[s] = w;
      sum += static_cast<double>(c.sums[p] * w);
    }
    sum = warp_sum_f64(sum);
    if (d == 0U) { gmax_s = m; gsum_s = static_cast<float>(sum); }
  }
  __syncthreads();
  double result = 0.0;
  for (uint32_t s = 0; s < active; ++s) {
    const size_t p = base + static_cast<size_t>(s) * c.q_heads;
    result += static_cast<double>(c.outputs[p * hd + d] * weights[s]);
  }
  const float out = actv(static_cast<float>(result) / gsum_s, c.bf16);
  if (c.out) c.out[(static_cast<size_t>(row) * c.q_heads + head) * hd + d] = out;
  if (c.sink.kind < 0) return;
  values[d] = out;
  __syncthreads();
  if ((d & 15U) == 0U) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = values[d + i];
    quant_store_block16(c.sink, row, (head * hd + d) / 16U, v);
  }
}

int launch_combine_quant(const CombineArgs& c, uint32_t rows, cudaStream_t stream) {
  if (c.max_splits > 512U || c.head_dim > 256U || c.head_dim % 32U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported split count or head_dim for the combine");
  combine_quant_kernel<<<dim3(c.q_heads, rows), c.head_dim, 0, stream>>>(c);
  count_launch();
  return check_launch("combine_quant");
}

// --------------------------------------------------------- materialise a GEMV result
__global__ void gemv_finalize_kernel(GemvOut o, float* y) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const uint64_t count = static_cast<uint64_t>(o.batch) * o.n;
  if (i >= count) return;
  y[i] = gemv_value(o, static_cast<uint32_t>(i / o.n), static_cast<uint32_t>(i % o.n));
}

int launch_gemv_finalize(const GemvOut& o, float* y, cudaStream_t stream) {
  if (o.split == 0U && o.data == y) return 0;
  const uint64_t count = static_cast<uint64_t>(o.batch) * o.n;
  gemv_finalize_kernel<<<static_cast<unsigned>((count + 255U) / 256U), 256, 0, stream>>>(o, y);
  count_launch();
  return check_launch("gemv_finalize");
}

}  // namespace qllm
