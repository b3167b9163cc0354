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
#include "launch.cuh"

#include <cooperative_groups.h>

namespace qllm {

// ---------------------------------------------------- residual + norm + quantise
// A cluster of four CTAs per row (the kernel sits on the critical path between two GEMVs and
// is bound by its own latency, so the row is spread over four SMs); each CTA keeps its quarter
// of the row in registers as float4s and the sums of squares meet in distributed shared memory.
// x' = act(x + delta) (delta optional), optionally stored back; then
// n = x' * rsqrt(mean x'^2 + eps) * w, optionally stored; then the NVFP4 operand of n.
constexpr uint32_t kNormThreads = 320;
constexpr uint32_t kNormVecs = 3;     // up to 4 * 320 * 3 * 4 = 15360 columns
constexpr uint32_t kNormCluster = 4;

// kExchange: delta is a tensor-parallel exchange result (its own instantiation, so that the
// single-GPU kernel carries none of the polling code).
template <bool kExchange>
__global__ void __launch_bounds__(kNormThreads)
residual_norm_quant_kernel(NormQuantArgs a) {
  namespace cg = cooperative_groups;
  __shared__ double partial[kNormThreads / 32U];
  __shared__ double cta_sum;
  pdl_trigger();
  cg::cluster_group cluster = cg::this_cluster();
  const uint32_t rank = cluster.block_rank();
  const uint32_t out_row = blockIdx.x / kNormCluster;
  const uint32_t n4 = a.cols / 4U;
  const uint32_t chunk = ((n4 + kNormCluster - 1U) / kNormCluster + 3U) & ~3U;  // whole 16-value blocks
  const uint32_t begin = rank * chunk, end = min(n4, begin + chunk);
  // the norm weights do not depend on the kernel before this one
  float4 w[kNormVecs];
#pragma unroll
  for (uint32_t k = 0; k < kNormVecs; ++k) {
    const uint32_t f = begin + threadIdx.x + k * kNormThreads;
    w[k] = (a.weight && f < end) ? reinterpret_cast<const float4*>(a.weight)[f] : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  }
  pdl_wait();
  const uint32_t in_row = a.row_select ? *a.row_select : out_row;
  // x == null: the row is the GEMV result alone (0 + delta is exact)
  const float4* x4 = a.x ? reinterpret_cast<const float4*>(a.x + static_cast<size_t>(in_row) * a.x_stride) : nullptr;
  float4 v[kNormVecs];
  double sq = 0.0;
#pragma unroll
  for (uint32_t k = 0; k < kNormVecs; ++k) {
    const uint32_t f = begin + threadIdx.x + k * kNormThreads;
    v[k] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (f < end) {
      if (x4) v[k] = x4[f];
      if (a.has_delta) {
        const float4 d = kExchange ? gemv_exchange_value4(a.delta, in_row, 4U * f)
                                   : gemv_value4(a.delta, in_row, 4U * f);
        v[k] = make_float4(actv(v[k].x + d.x, a.bf16), actv(v[k].y + d.y, a.bf16), actv(v[k].z + d.z, a.bf16),
                           actv(v[k].w + d.w, a.bf16));
      }
      if (a.store) reinterpret_cast<float4*>(a.store + static_cast<size_t>(out_row) * a.store_stride)[f] = v[k];
      sq += static_cast<double>(v[k].x) * v[k].x + static_cast<double>(v[k].y) * v[k].y +
            static_cast<double>(v[k].z) * v[k].z + static_cast<double>(v[k].w) * v[k].w;
    }
  }
  if (!a.weight) return;  // residual update only (uniform over the grid)
  sq = warp_sum_f64(sq);
  if ((threadIdx.x & 31U) == 0U) partial[threadIdx.x >> 5U] = sq;
  __syncthreads();
  if (threadIdx.x == 0U) {
    double t = 0.0;
    for (uint32_t i = 0; i < kNormThreads / 32U; ++i) t += partial[i];
    cta_sum = t;
  }
  cluster.sync();
  double total = 0.0;
  for (uint32_t r = 0; r < kNormCluster; ++r) total += *cluster.map_shared_rank(&cta_sum, r);
  const float inverse = 1.0F / sqrtf(static_cast<float>(total) / static_cast<float>(a.cols) + a.eps);
#pragma unroll
  for (uint32_t k = 0; k < kNormVecs; ++k) {
    const uint32_t f = begin + threadIdx.x + k * kNormThreads;
    if (begin + k * kNormThreads >= end) break;  // uniform: no lane of the CTA has work left
    const bool valid = f < end;
    float4 n = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (valid) {
      n = make_float4(v[k].x * inverse * w[k].x, v[k].y * inverse * w[k].y, v[k].z * inverse * w[k].z,
                      v[k].w * inverse * w[k].w);
      if (a.round_normalized) n = make_float4(bf16r(n.x), bf16r(n.y), bf16r(n.z), bf16r(n.w));
      if (a.normalized)
        reinterpret_cast<float4*>(a.normalized + static_cast<size_t>(out_row) * a.normalized_stride)[f] = n;
    }
    if (a.sink.kind >= 0) quant_store_quad(a.sink, out_row, a.sink_block_offset + f / 4U, n, valid);
  }
  cluster.sync();  // no CTA leaves while a neighbour may still read its sum
}

int launch_residual_norm_quant(const NormQuantArgs& a, uint32_t rows, cudaStream_t stream) {
  if (!rows || !a.cols || a.cols % 16U || a.cols > kNormCluster * kNormThreads * kNormVecs * 4U || a.x_stride % 4U ||
      a.store_stride % 4U || a.normalized_stride % 4U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported row length for the fused norm");
  count_launch();
  if (a.has_delta && a.delta.exchange != nullptr)
    return check_cuda(launch_pdl_cluster(residual_norm_quant_kernel<true>, dim3(rows * kNormCluster),
                                         dim3(kNormThreads), kNormCluster, 0, stream, a),
                      "residual_norm_quant");
  return check_cuda(launch_pdl_cluster(residual_norm_quant_kernel<false>, dim3(rows * kNormCluster), dim3(kNormThreads),
                                       kNormCluster, 0, stream, a),
                    "residual_norm_quant");
}

// ------------------------------------------------------------ SiLU product + quantise
// One thread per 4 outputs: inter = act(act(silu(g)) * u), quantised for the down GEMV.
template <bool kExact>  // exp from the deterministic series shared with the CPU oracle (the parity path)
__global__ void __launch_bounds__(256)
silu_quant_kernel(GemvOut gate_up, uint32_t ffn, bool bf16, QuantSink sink, float* inter) {
  pdl_trigger();
  pdl_wait();
  const uint32_t n4 = ffn / 4U;
  const uint32_t item = blockIdx.x * blockDim.x + threadIdx.x;
  const bool valid = item < gate_up.batch * n4;
  constexpr bool exact = kExact;
  const uint32_t row = valid ? item / n4 : 0U, f = valid ? item % n4 : 0U;
  float4 v = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  if (valid) {
    const float4 g = gemv_value4(gate_up, row, 4U * f);
    const float4 u = gemv_value4(gate_up, row, ffn + 4U * f);
    v.x = actv(actv(g.x / (1.0F + (exact ? det_expf(-g.x) : expf(-g.x))), bf16) * u.x, bf16);
    v.y = actv(actv(g.y / (1.0F + (exact ? det_expf(-g.y) : expf(-g.y))), bf16) * u.y, bf16);
    v.z = actv(actv(g.z / (1.0F + (exact ? det_expf(-g.z) : expf(-g.z))), bf16) * u.z, bf16);
    v.w = actv(actv(g.w / (1.0F + (exact ? det_expf(-g.w) : expf(-g.w))), bf16) * u.w, bf16);
    if (inter) reinterpret_cast<float4*>(inter + static_cast<size_t>(row) * ffn)[f] = v;
  }
  quant_store_quad(sink, row, f / 4U, v, valid);
}

int launch_silu_quant(const GemvOut& gate_up, uint32_t ffn, bool bf16, const QuantSink& sink, float* inter,
                      cudaStream_t stream) {
  if (ffn % 16U) return fail(QLLM_INVALID_ARGUMENT, "FFN width must be a multiple of 16");
  const uint32_t items = gate_up.batch * (ffn / 4U);
  count_launch();
  // the exact path (CUDA-core operand) takes exp from the deterministic series shared with the oracle
  if (sink.kind == 0)
    return check_cuda(launch_pdl(silu_quant_kernel<true>, dim3((items + 255U) / 256U), dim3(256), 0, stream, gate_up, ffn,
                                 bf16, sink, inter), "silu_quant");
  return check_cuda(launch_pdl(silu_quant_kernel<false>, dim3((items + 255U) / 256U), dim3(256), 0, stream, gate_up, ffn,
                               bf16, sink, inter), "silu_quant");
}

// ------------------------------------------------------------- split combine + quantise
// One warp per (row, query head), four heads per CTA; a lane owns 4 (head_dim 128) or
// 8 (head_dim 256) output dims.  Merges the context splits by log-sum-exp (sums in double:
// independent of the visiting order) and writes the o-projection operand.
constexpr uint32_t kCombineSplits = 512;

// two CTAs per SM (128 registers): rows x heads CTAs of a verify pass then fit one wave
// kExact: exp from the deterministic series shared with the CPU oracle (the parity path); its own
// instantiation, because the benchmarked form sits exactly at its register limit
template <bool kTiled, bool kExact>  // kTiled: grid z = row tile of a wide pass
__global__ void __launch_bounds__(256, 2)
combine_quant_kernel(CombineArgs c) {
  // CTA = (row, query head), 8 warps: warp w merges the splits s = w (mod 8); a lane owns
  // 4 (head_dim 128) or 8 (head_dim 256) output dims.
  // Every load is issued before anything is reduced, so the kernel costs one memory round
  // trip and one barrier: each warp finds the global maximum itself (the maxima of all
  // splits are a few hundred floats) while the partial outputs of its own splits are in flight.
  __shared__ double partial[8][4][64];
  __shared__ double sums[8];
  pdl_trigger();
  pdl_wait();
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t head = blockIdx.x, row = blockIdx.y, hd = c.head_dim;
  // grid z = row tile of a wide pass: gridDim.y rows each, partials one tile after the other
  const uint32_t tile_row0 = kTiled ? blockIdx.z * gridDim.y : 0U;
  if constexpr (kTiled) {
    const size_t tile_shift = blockIdx.z * attention_partial_items(gridDim.y, c.max_splits, c.q_heads) * (2U + hd);
    c.maxima += tile_shift;
    c.sums += tile_shift;
    c.outputs += tile_shift;
  }
  const uint32_t ctx = *c.first_position + c.position_offset + 1U + tile_row0 + row;
  const uint32_t active = (ctx + c.split_tokens - 1U) / c.split_tokens;
  const size_t base = static_cast<size_t>(row) * c.max_splits * c.q_heads + head;
  const uint32_t vecs = hd / 4U;  // float4s per head: 16, 32 or 64
  constexpr uint32_t kBatch = 8;  // splits of this warp held in registers at a time
  float mine[kCombineSplits / 32U];  // maxima of the splits lane, lane+32, ...
  float m = kNegInf;
#pragma unroll
  for (uint32_t i = 0; i < kCombineSplits / 32U; ++i) {
    const uint32_t s = lane + 32U * i;
    mine[i] = s < active ? c.maxima[base + static_cast<size_t>(s) * c.q_heads] : kNegInf;
  }
  // The splits are merged in eight classes s = cls (mod 8), one partial sum per class, whatever
  // the number of warps: eight warps take one class each; the row-tiled form (thousands of CTAs
  // with one or two splits each at prompt lengths) runs two warps that take four classes each,
  // so that more CTAs fit an SM.  Same additions in the same order either way.
  constexpr uint32_t kWarps = kTiled ? 2U : 8U;
  bool have_max = false;
  uint32_t cls = warp;
  do {
  double r[2][4] = {{0.0, 0.0, 0.0, 0.0}, {0.0, 0.0, 0.0, 0.0}};
  double sum = 0.0;
  for (uint32_t s0 = cls; s0 < active; s0 += 8U * kBatch) {
    float4 o[kBatch][2];
    float ssum[kBatch], smax[kBatch];
#pragma unroll
    for (uint32_t b = 0; b < kBatch; ++b) {
      const uint32_t s = s0 + 8U * b;
      const size_t p = base + static_cast<size_t>(min(s, active - 1U)) * c.q_heads;
      const float4* src = reinterpret_cast<const float4*>(c.outputs + p * hd);
      o[b][0] = lane < vecs ? src[lane] : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
      o[b][1] = lane + 32U < vecs ? src[lane + 32U] : make_float4(0.0F, 0.0F, 0.0F, 0.0F);
      ssum[b] = c.sums[p];
      smax[b] = c.maxima[p];
    }
    if (!have_max) {
#pragma unroll
      for (uint32_t i = 0; i < kCombineSplits / 32U; ++i) m = fmaxf(m, mine[i]);
      m = warp_max(m);
      have_max = true;
    }
#pragma unroll
    for (uint32_t b = 0; b < kBatch; ++b) {
      if (s0 + 8U * b >= active) break;
      const float w = kExact ? det_expf(smax[b] - m) : expf(smax[b] - m);
      sum += static_cast<double>(ssum[b] * w);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        r[h][0] += static_cast<double>(o[b][h].x * w);
        r[h][1] += static_cast<double>(o[b][h].y * w);
        r[h][2] += static_cast<double>(o[b][h].z * w);
        r[h][3] += static_cast<double>(o[b][h].w * w);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t f = lane + 32U * h;
    if (f < vecs) {
      partial[cls][0][f] = r[h][0]; partial[cls][1][f] = r[h][1];
      partial[cls][2][f] = r[h][2]; partial[cls][3][f] = r[h][3];
    }
  }
  if (lane == 0U) sums[cls] = sum;
  cls += kWarps;
  } while (kTiled && cls < 8U);
  __syncthreads();
  if (warp >= (vecs + 31U) / 32U) return;  // warps 0 (and 1 for head_dim 256) finish
  const uint32_t f = warp * 32U + lane;
  const bool valid = f < vecs;
  float4 out = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  if (valid) {
    double r[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
      for (int w = 0; w < 8; ++w) r[e] += partial[w][e][f];
    double total = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) total += sums[w];
    const float gsum = static_cast<float>(total);
    out = make_float4(actv(static_cast<float>(r[0]) / gsum, c.bf16), actv(static_cast<float>(r[1]) / gsum, c.bf16),
                      actv(static_cast<float>(r[2]) / gsum, c.bf16), actv(static_cast<float>(r[3]) / gsum, c.bf16));
    if (c.out) reinterpret_cast<float4*>(c.out + (static_cast<size_t>(tile_row0 + row) * c.q_heads + head) * hd)[f] = out;
  }
  if (c.sink.kind >= 0)
    quant_store_quad(c.sink, tile_row0 + row + c.sink_row_offset, (head * hd + 4U * f) / 16U, out, valid);
}

int launch_combine_quant(const CombineArgs& c, uint32_t rows, cudaStream_t stream) {
  if (c.max_splits > kCombineSplits || c.head_dim > 256U || c.head_dim % 16U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported split count or head_dim for the combine");
  count_launch();
  if (c.tiles > 1U)
    return check_cuda(c.exact ? launch_pdl(combine_quant_kernel<true, true>, dim3(c.q_heads, rows, c.tiles), dim3(64), 0, stream, c)
                              : launch_pdl(combine_quant_kernel<true, false>, dim3(c.q_heads, rows, c.tiles), dim3(64), 0, stream, c),
                      "combine_quant");
  return check_cuda(c.exact ? launch_pdl(combine_quant_kernel<false, true>, dim3(c.q_heads, rows), dim3(256), 0, stream, c)
                            : launch_pdl(combine_quant_kernel<false, false>, dim3(c.q_heads, rows), dim3(256), 0, stream, c),
                    "combine_quant");
}

// --------------------------------------------------------- materialise a GEMV result
__global__ void gemv_finalize_kernel(GemvOut o, float* y) {
  pdl_trigger();
  pdl_wait();
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
  count_launch();
  return check_cuda(launch_pdl(gemv_finalize_kernel, dim3(static_cast<unsigned>((count + 255U) / 256U)), dim3(256), 0,
                               stream, o, y), "gemv_finalize");
}

}  // namespace qllm
