// Fused row-wise kernels between the GEMVs of a decode step.  Each one consumes a GEMV
// result (final values or split-K partials), applies the reference's element-wise step with
// its BF16 rounding points, and writes the NEXT GEMV's quantised NVFP4 operand directly, so a
// transformer block is ten launches instead of eighteen:
//   residual add + RMSNorm + quantise      (add_kernel, rms_batch_kernel, nvfp4_quant_dequant_kernel;
//                                           runtime/src/cuda/transformer_kernels.cu:2522, 2487, 1943)
//   SiLU(gate)*up + quantise               (silu_product_kernel 2774)
//   split combine + quantise               (combine kernel 5741)
// All of them move 16 bytes per thread and let four neighbouring lanes share one 16-value
// quantisation block.
#include "common.cuh"
#include "fused.h"

namespace qllm {

// ---------------------------------------------------- residual + norm + quantise
// One CTA (512 threads) per row, the row lives in registers as float4s.
// x' = act(x + delta) (delta optional), optionally stored back; then
// n = x' * rsqrt(mean x'^2 + eps) * w, optionally stored; then the NVFP4 operand of n.
constexpr uint32_t kNormThreads = 512;
constexpr uint32_t kNormVecs = 6;  // up to 512*6*4 = 12288 columns

__global__ void __launch_bounds__(kNormThreads)
residual_norm_quant_kernel(NormQuantArgs a) {
  __shared__ double partial[16];
  const uint32_t out_row = blockIdx.x;
  const uint32_t in_row = a.row_select ? *a.row_select : out_row;
  const uint32_t n4 = a.cols / 4U;
  // x == null: the row is the GEMV result alone (0 + delta is exact)
  const float4* x4 = a.x ? reinterpret_cast<const float4*>(a.x + static_cast<size_t>(in_row) * a.x_stride) : nullptr;
  float4 v[kNormVecs];
  double sq = 0.0;
#pragma unroll
  for (uint32_t k = 0; k < kNormVecs; ++k) {
    const uint32_t f = threadIdx.x + k * kNormThreads;
    v[k] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (f < n4) {
      if (x4) v[k] = x4[f];
      if (a.has_delta) {
        const float4 d = gemv_value4(a.delta, in_row, 4U * f);
        v[k] = make_float4(actv(v[k].x + d.x, a.bf16), actv(v[k].y + d.y, a.bf16), actv(v[k].z + d.z, a.bf16),
                           actv(v[k].w + d.w, a.bf16));
      }
      if (a.store) reinterpret_cast<float4*>(a.store + static_cast<size_t>(out_row) * a.store_stride)[f] = v[k];
      sq += static_cast<double>(v[k].x) * v[k].x + static_cast<double>(v[k].y) * v[k].y +
            static_cast<double>(v[k].z) * v[k].z + static_cast<double>(v[k].w) * v[k].w;
    }
  }
  if (!a.weight) return;  // residual update only
  sq = warp_sum_f64(sq);
  if ((threadIdx.x & 31U) == 0U) partial[threadIdx.x >> 5U] = sq;
  __syncthreads();
  if (threadIdx.x < 32U) {
    double t = threadIdx.x < (kNormThreads >> 5U) ? partial[threadIdx.x] : 0.0;
    t = warp_sum_f64(t);
    if (threadIdx.x == 0U) partial[0] = t;
  }
  __syncthreads();
  const float inverse = 1.0F / sqrtf(static_cast<float>(partial[0]) / static_cast<float>(a.cols) + a.eps);
  const float4* w4 = reinterpret_cast<const float4*>(a.weight);
#pragma unroll
  for (uint32_t k = 0; k < kNormVecs; ++k) {
    const uint32_t f = threadIdx.x + k * kNormThreads;
    if (k * kNormThreads >= n4) break;  // uniform: no lane of the CTA has work left
    const bool valid = f < n4;
    float4 n = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (valid) {
      const float4 w = w4[f];
      n = make_float4(v[k].x * inverse * w.x, v[k].y * inverse * w.y, v[k].z * inverse * w.z, v[k].w * inverse * w.w);
      if (a.normalized)
        reinterpret_cast<float4*>(a.normalized + static_cast<size_t>(out_row) * a.normalized_stride)[f] = n;
    }
    if (a.sink.kind >= 0) quant_store_quad(a.sink, out_row, a.sink_block_offset + f / 4U, n, valid);
  }
}

int launch_residual_norm_quant(const NormQuantArgs& a, uint32_t rows, cudaStream_t stream) {
  if (!rows || !a.cols || a.cols % 16U || a.cols > kNormThreads * kNormVecs * 4U || a.x_stride % 4U ||
      a.store_stride % 4U || a.normalized_stride % 4U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported row length for the fused norm");
  residual_norm_quant_kernel<<<rows, kNormThreads, 0, stream>>>(a);
  count_launch();
  return check_launch("residual_norm_quant");
}

// ------------------------------------------------------------ SiLU product + quantise
// One thread per 4 outputs: inter = act(act(silu(g)) * u), quantised for the down GEMV.
__global__ void __launch_bounds__(256)
silu_quant_kernel(GemvOut gate_up, uint32_t ffn, bool bf16, QuantSink sink, float* inter) {
  const uint32_t n4 = ffn / 4U;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = item < gate_up.batch * n4;
  const uint32_t row = valid ? item / n4 : 0U, f = valid ? item % n4 : 0U;
  float4 v = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  if (valid) {
    const float4 g = gemv_value4(gate_up, row, 4U * f);
    const float4 u = gemv_value4(gate_up, row, ffn + 4U * f);
    v.x = actv(actv(g.x / (1.0F + expf(-g.x)), bf16) * u.x, bf16);
    v.y = actv(actv(g.y / (1.0F + expf(-g.y)), bf16) * u.y, bf16);
    v.z = actv(actv(g.z / (1.0F + expf(-g.z)), bf16) * u.z, bf16);
    v.w = actv(actv(g.w / (1.0F + expf(-g.w)), bf16) * u.w, bf16);
    if (inter) reinterpret_cast<float4*>(inter + static_cast<size_t>(row) * ffn)[f] = v;
  }
  quant_store_quad(sink, row, f / 4U, v, valid);
}

int launch_silu_quant(const GemvOut& gate_up, uint32_t ffn, bool bf16, const QuantSink& sink, float* inter,
                      cudaStream_t stream) {
  if (ffn % 16U) return fail(QLLM_INVALID_ARGUMENT, "FFN width must be a multiple of 16");
  const uint32_t items = gate_up.batch * (ffn / 4U);
  silu_quant_kernel<<<(items + 255U) / 256U, 256, 0, stream>>>(gate_up, ffn, bf16, sink, inter);
  count_launch();
  return check_launch("silu_quant");
}

// ------------------------------------------------------------- split combine + quantise
// One warp per (row, query head), four heads per CTA; a lane owns 4 (head_dim 128) or
// 8 (head_dim 256) output dims.  Merges the context splits by log-sum-exp (sums in double:
// independent of the visiting order) and writes the o-projection operand.
constexpr uint32_t kCombineSplits = 512;

__global__ void __launch_bounds__(128)
combine_quant_kernel(CombineArgs c) {
  __shared__ float weights[4][kCombineSplits];
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t head = blockIdx.x * 4U + warp, row = blockIdx.y, hd = c.head_dim;
  if (head >= c.q_heads) return;  // whole warp
  const uint32_t ctx = *c.first_position + c.position_offset + 1U + row;
  const uint32_t active = (ctx + c.split_tokens - 1U) / c.split_tokens;
  const size_t base = static_cast<size_t>(row) * c.max_splits * c.q_heads + head;
  float m = kNegInf;
  for (uint32_t s = lane; s < active; s += 32U) m = fmaxf(m, c.maxima[base + static_cast<size_t>(s) * c.q_heads]);
  m = warp_max(m);
  double sum = 0.0;
  for (uint32_t s = lane; s < active; s += 32U) {
    const size_t p = base + static_cast<size_t>(s) * c.q_heads;
    const float w = expf(c.maxima[p] - m);
    weights[warp][s] = w;
    sum += static_cast<double>(c.sums[p] * w);
  }
  const float gsum = static_cast<float>(warp_sum_f64(sum));
  __syncwarp();
  for (uint32_t f = lane; f < ((hd / 4U + 31U) & ~31U); f += 32U) {  // warp-uniform trip count
    const bool valid = f < hd / 4U;
    float4 out = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (valid) {
      double r0 = 0.0, r1 = 0.0, r2 = 0.0, r3 = 0.0;
#pragma unroll 4
      for (uint32_t s = 0; s < active; ++s) {
        const size_t p = base + static_cast<size_t>(s) * c.q_heads;
        const float4 o = reinterpret_cast<const float4*>(c.outputs + p * hd)[f];
        const float w = weights[warp][s];
        r0 += static_cast<double>(o.x * w);
        r1 += static_cast<double>(o.y * w);
        r2 += static_cast<double>(o.z * w);
        r3 += static_cast<double>(o.w * w);
      }
      out = make_float4(actv(static_cast<float>(r0) / gsum, c.bf16), actv(static_cast<float>(r1) / gsum, c.bf16),
                        actv(static_cast<float>(r2) / gsum, c.bf16), actv(static_cast<float>(r3) / gsum, c.bf16));
      if (c.out) reinterpret_cast<float4*>(c.out + (static_cast<size_t>(row) * c.q_heads + head) * hd)[f] = out;
    }
    if (c.sink.kind >= 0) quant_store_quad(c.sink, row, (head * hd + 4U * f) / 16U, out, valid);
  }
}

int launch_combine_quant(const CombineArgs& c, uint32_t rows, cudaStream_t stream) {
  if (c.max_splits > kCombineSplits || c.head_dim > 256U || c.head_dim % 16U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported split count or head_dim for the combine");
  combine_quant_kernel<<<dim3((c.q_heads + 3U) / 4U, rows), 128, 0, stream>>>(c);
  count_launch();
  return check_launch("combine_quant");
}

// --------------------------------------------------------- materialise a GEMV result
__global__ void gemv_finalize_kernel(GemvOut o, float* y) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const uint64_t count = static_cast<uint64_t>(o.batch) * o.n / 4U;
  if (i >= count) return;
  const uint32_t per_row = o.n / 4U;
  reinterpret_cast<float4*>(y)[i] =
      gemv_value4(o, static_cast<uint32_t>(i / per_row), 4U * static_cast<uint32_t>(i % per_row));
}

int launch_gemv_finalize(const GemvOut& o, float* y, cudaStream_t stream) {
  if (o.split == 0U && o.data == y) return 0;
  if (o.n % 4U) return fail(QLLM_INVALID_ARGUMENT, "GEMV output width must be a multiple of 4");
  const uint64_t count = static_cast<uint64_t>(o.batch) * o.n / 4U;
  gemv_finalize_kernel<<<static_cast<unsigned>((count + 255U) / 256U), 256, 0, stream>>>(o, y);
  count_launch();
  return check_launch("gemv_finalize");
}

}  // namespace qllm
