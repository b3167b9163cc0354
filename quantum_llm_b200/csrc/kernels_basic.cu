// Small per-row kernels of the decode step: embedding gather, RMSNorm, NVFP4
// activation fake-quantisation, the CUDA-core NVFP4 GEMV, residual add, SwiGLU
// product, argmax and exact top-k.  Arithmetic follows the reference launchers
// named in include/qllm_b200.h; layouts and launch shapes are this library's own.
#include "common.cuh"
#include "fp4_dot.cuh"
#include "kernels.h"

namespace qllm {

// ------------------------------------------------------------------ embedding
__global__ void embedding_bf16_kernel(const uint16_t* __restrict__ table,
                                      const uint32_t* __restrict__ tokens, float* __restrict__ out,
                                      uint32_t hidden, uint32_t vocab) {
  const uint32_t row = blockIdx.y;
  const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
  if (col >= hidden) return;
  uint32_t token = tokens[row];
  if (token >= vocab) token = vocab - 1U;  // host validates; keep the gather in bounds
  out[static_cast<size_t>(row) * hidden + col] =
      __uint_as_float(static_cast<uint32_t>(table[static_cast<size_t>(token) * hidden + col]) << 16U);
}

int launch_embedding(const uint16_t* table, const uint32_t* tokens, float* out, uint32_t rows,
                     uint32_t hidden, uint32_t vocab, cudaStream_t stream) {
  const dim3 grid((hidden + 255U) / 256U, rows);
  embedding_bf16_kernel<<<grid, 256, 0, stream>>>(table, tokens, out, hidden, vocab);
  count_launch();
  return check_launch("embedding");
}

// -------------------------------------------------------------------- RMSNorm
// One CTA per row. `row_select`, when set, names the single input row to read
// (the accepted row of a verify batch); output row is blockIdx.x.
__global__ void rms_norm_kernel(const float* __restrict__ x, const float* __restrict__ weight,
                                float* __restrict__ out, uint32_t cols, uint32_t in_stride,
                                uint32_t out_stride, float eps,
                                const uint32_t* __restrict__ row_select) {
  __shared__ double partial[32];
  const uint32_t in_row = row_select ? *row_select : blockIdx.x;
  const float* in = x + static_cast<size_t>(in_row) * in_stride;
  float* o = out + static_cast<size_t>(blockIdx.x) * out_stride;
  double sq = 0.0;
  // squares and their sum in double: the sum is then independent of the reduction order
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) {
    const double v = static_cast<double>(in[i]);
    sq += v * v;
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
  const float inverse =
      1.0F / sqrtf(static_cast<float>(partial[0]) / static_cast<float>(cols) + eps);
  for (uint32_t i = threadIdx.x; i < cols; i += blockDim.x) o[i] = in[i] * inverse * weight[i];
}

int launch_rms_norm(const float* x, const float* weight, float* out, uint32_t rows, uint32_t cols,
                    uint32_t in_stride, uint32_t out_stride, float eps,
                    const uint32_t* row_select, cudaStream_t stream) {
  rms_norm_kernel<<<rows, 256, 0, stream>>>(x, weight, out, cols, in_stride, out_stride, eps,
                                            row_select);
  count_launch();
  return check_launch("rms_norm");
}

// ----------------------------------------------------- NVFP4 fake quantisation
// One thread per 16-value block.
__global__ void nvfp4_fake_quant_kernel(const float* __restrict__ x, float* __restrict__ out,
                                        uint64_t blocks, float g) {
  const uint64_t b = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const float4* in4 = reinterpret_cast<const float4*>(x + b * 16U);
  float v[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = in4[i];
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float local = e4m3_value(e4m3_code(fminf(448.0F, g * amax / 6.0F)));
  float4* out4 = reinterpret_cast<float4*>(out + b * 16U);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float scaled = local == 0.0F ? 0.0F : fminf(6.0F, fmaxf(-6.0F, v[i] * g / local));
    v[i] = e2m1_value(e2m1_code(scaled)) * local / g;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out4[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
}

int launch_fake_quant(const float* x, float* out, uint32_t rows, uint32_t cols, float g,
                      cudaStream_t stream) {
  const uint64_t blocks = static_cast<uint64_t>(rows) * (cols / 16U);
  nvfp4_fake_quant_kernel<<<static_cast<unsigned>((blocks + 127U) / 128U), 128, 0, stream>>>(
      x, out, blocks, g);
  count_launch();
  return check_launch("nvfp4_fake_quant");
}

// --------------------------------------------- NVFP4 activation quantisation
// One thread per 16-value block.  Output for the CUDA-core GEMV: twice the E2M1
// value as INT8 (0, +-1, +-2, +-3, +-4, +-6, +-8, +-12) and the decoded E4M3 block
// scale as FP32.  The fake-quantised activation is value8/2 * scale / g.
__global__ void nvfp4_act_quant_i8_kernel(const float* __restrict__ x, int8_t* __restrict__ xi8,
                                          float* __restrict__ xscale, uint64_t blocks, float g) {
  const uint64_t b = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const float4* in4 = reinterpret_cast<const float4*>(x + b * 16U);
  float v[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = in4[i];
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float local = e4m3_value(e4m3_code(fminf(448.0F, g * amax / 6.0F)));
  uint32_t packed[4] = {0U, 0U, 0U, 0U};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float scaled = local == 0.0F ? 0.0F : fminf(6.0F, fmaxf(-6.0F, v[i] * g / local));
    const unsigned code = e2m1_code(scaled);
    const unsigned m = code & 7U;
    int twice = m < 5U ? static_cast<int>(m) : static_cast<int>(2U * m - 4U) + (m == 7U ? 2 : 0);
    // m: 0 1 2 3 4 5 6 7 -> 0 1 2 3 4 6 8 12
    if (code & 8U) twice = -twice;
    packed[i / 4] |= (static_cast<uint32_t>(twice) & 0xffU) << (8 * (i % 4));
  }
  reinterpret_cast<uint4*>(xi8)[b] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  xscale[b] = local;
}

size_t act_quant_bytes(uint32_t rows, uint32_t cols) {
  // INT8 values followed by the FP32 block scales (16-byte aligned)
  const size_t values = (static_cast<size_t>(rows) * cols + 15U) & ~static_cast<size_t>(15U);
  return values + static_cast<size_t>(rows) * (cols / 16U) * sizeof(float);
}

int launch_act_quant_i8(const float* x, void* qact, uint32_t rows, uint32_t cols, float g,
                        cudaStream_t stream) {
  const uint64_t blocks = static_cast<uint64_t>(rows) * (cols / 16U);
  const size_t values = (static_cast<size_t>(rows) * cols + 15U) & ~static_cast<size_t>(15U);
  int8_t* xi8 = static_cast<int8_t*>(qact);
  float* xscale = reinterpret_cast<float*>(static_cast<uint8_t*>(qact) + values);
  nvfp4_act_quant_i8_kernel<<<static_cast<unsigned>((blocks + 127U) / 128U), 128, 0, stream>>>(
      x, xi8, xscale, blocks, g);
  count_launch();
  return check_launch("nvfp4_act_quant");
}

// ------------------------------------------------------ CUDA-core NVFP4 GEMV
// W4A4 product with exact block arithmetic: per 16-value block the integer dot of
// (2*weight code value) and (2*activation code value) by four DP4A, times the exact
// FP32 product of the two E4M3 block scales; block terms are summed in double, so the
// result does not depend on the summation order, and rounded once:
//   y = bf16(float(S) * weight_scale / input_scale),  S = sum (dot/4) * sw * sx.
// A warp owns two weight rows and walks the row in 16-value blocks, one block per
// lane per step: 8 code bytes + 1 scale byte per row, the activations of the block
// (16 INT8 + 1 FP32 per batch row) are loaded once for both weight rows.
// (prmt / expand_fp4x8: fp4_dot.cuh)
template <int B>
__global__ void __launch_bounds__(256)
nvfp4_gemv_dp4a_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                       float weight_scale, float input_scale, const int8_t* __restrict__ xi8,
                       const float* __restrict__ xscale, float* __restrict__ y, uint32_t first_row,
                       uint32_t row_count, uint32_t cols, uint32_t y_stride) {
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t local_row = (blockIdx.x * 8U + warp) * 2U;
  if (local_row >= row_count) return;
  const bool two = local_row + 1U < row_count;
  const uint32_t blocks = cols / 16U;
  const size_t row0 = static_cast<size_t>(first_row) + local_row;
  const size_t row1 = two ? row0 + 1U : row0;
  const uint2* w0 = reinterpret_cast<const uint2*>(codes + row0 * (cols / 2U));
  const uint2* w1 = reinterpret_cast<const uint2*>(codes + row1 * (cols / 2U));
  const uint8_t* s0 = scales + row0 * blocks;
  const uint8_t* s1 = scales + row1 * blocks;
  double acc0[B], acc1[B];
#pragma unroll
  for (int b = 0; b < B; ++b) { acc0[b] = 0.0; acc1[b] = 0.0; }
  for (uint32_t blk = lane; blk < blocks; blk += 32U) {
    const uint2 c0 = __ldg(w0 + blk), c1 = __ldg(w1 + blk);
    const float sw0 = e4m3_value(__ldg(s0 + blk)), sw1 = e4m3_value(__ldg(s1 + blk));
    uint32_t a0[4], a1[4];
    expand_fp4x8(c0.x, a0[0], a0[1]);
    expand_fp4x8(c0.y, a0[2], a0[3]);
    expand_fp4x8(c1.x, a1[0], a1[1]);
    expand_fp4x8(c1.y, a1[2], a1[3]);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(xi8 + static_cast<size_t>(b) * cols) + blk);
      const float sx = __ldg(xscale + static_cast<size_t>(b) * blocks + blk);
      int d0 = __dp4a(static_cast<int>(a0[0]), static_cast<int>(xv.x), 0);
      d0 = __dp4a(static_cast<int>(a0[1]), static_cast<int>(xv.y), d0);
      d0 = __dp4a(static_cast<int>(a0[2]), static_cast<int>(xv.z), d0);
      d0 = __dp4a(static_cast<int>(a0[3]), static_cast<int>(xv.w), d0);
      int d1 = __dp4a(static_cast<int>(a1[0]), static_cast<int>(xv.x), 0);
      d1 = __dp4a(static_cast<int>(a1[1]), static_cast<int>(xv.y), d1);
      d1 = __dp4a(static_cast<int>(a1[2]), static_cast<int>(xv.z), d1);
      d1 = __dp4a(static_cast<int>(a1[3]), static_cast<int>(xv.w), d1);
      // exact: |d| < 2^12, scale product has 8 significant bits
      acc0[b] += static_cast<double>(static_cast<float>(d0) * (sw0 * sx) * 0.25F);
      acc1[b] += static_cast<double>(static_cast<float>(d1) * (sw1 * sx) * 0.25F);
    }
  }
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const double t0 = warp_sum_f64(acc0[b]), t1 = warp_sum_f64(acc1[b]);
    if (lane == 0U) {
      y[static_cast<size_t>(b) * y_stride + local_row] =
          bf16r(static_cast<float>(t0) * weight_scale / input_scale);
      if (two)
        y[static_cast<size_t>(b) * y_stride + local_row + 1U] =
            bf16r(static_cast<float>(t1) * weight_scale / input_scale);
    }
  }
}

int launch_gemv_simt(const qllm_matrix& m, uint32_t first_row, uint32_t row_count, const void* qact,
                     uint32_t qact_rows, float* y, uint32_t batch, cudaStream_t stream) {
  const unsigned grid = (row_count + 15U) / 16U;
  const size_t values = (static_cast<size_t>(qact_rows) * m.cols + 15U) & ~static_cast<size_t>(15U);
  const int8_t* xi8 = static_cast<const int8_t*>(qact);
  const float* xscale = reinterpret_cast<const float*>(static_cast<const uint8_t*>(qact) + values);
  for (uint32_t first = 0; first < batch; first += 8U) {
    const uint32_t tile = batch - first < 8U ? batch - first : 8U;
    const int8_t* xin = xi8 + static_cast<size_t>(first) * m.cols;
    const float* sin = xscale + static_cast<size_t>(first) * (m.cols / 16U);
    float* yo = y + static_cast<size_t>(first) * row_count;
#define QLLM_GEMV_CASE(N)                                                                     \
  case N:                                                                                     \
    nvfp4_gemv_dp4a_kernel<N><<<grid, 256, 0, stream>>>(m.codes, m.scales, m.weight_scale,    \
                                                         m.input_scale, xin, sin, yo,         \
                                                         first_row, row_count, m.cols,        \
                                                         row_count);                          \
    break;
    switch (tile) {
      QLLM_GEMV_CASE(1) QLLM_GEMV_CASE(2) QLLM_GEMV_CASE(3) QLLM_GEMV_CASE(4)
      QLLM_GEMV_CASE(5) QLLM_GEMV_CASE(6) QLLM_GEMV_CASE(7) QLLM_GEMV_CASE(8)
    }
#undef QLLM_GEMV_CASE
    count_launch();
  }
  return check_launch("nvfp4_gemv");
}

// ------------------------------------------------- device weight quantiser
__global__ void nvfp4_quantize_weights_kernel(const float* __restrict__ w, uint64_t blocks,
                                              float g, uint8_t* __restrict__ codes,
                                              uint8_t* __restrict__ scales) {
  const uint64_t b = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (b >= blocks) return;
  const float4* in4 = reinterpret_cast<const float4*>(w + b * 16U);
  float v[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = in4[i];
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const unsigned sc = e4m3_code(fminf(448.0F, g * amax / 6.0F));
  const float local = e4m3_value(sc);
  scales[b] = static_cast<uint8_t>(sc);
  uint32_t packed[2] = {0U, 0U};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    unsigned code = 0U;
    if (local != 0.0F) code = e2m1_code(fminf(6.0F, fmaxf(-6.0F, v[i] * g / local)));
    packed[i / 8] |= code << (4 * (i % 8));
  }
  reinterpret_cast<uint2*>(codes)[b] = make_uint2(packed[0], packed[1]);
}

int launch_quantize_weights(const float* w, uint32_t rows, uint32_t cols, float g, uint8_t* codes,
                            uint8_t* scales, cudaStream_t stream) {
  const uint64_t blocks = static_cast<uint64_t>(rows) * (cols / 16U);
  nvfp4_quantize_weights_kernel<<<static_cast<unsigned>((blocks + 255U) / 256U), 256, 0, stream>>>(
      w, blocks, g, codes, scales);
  count_launch();
  return check_launch("nvfp4_quantize_weights");
}

// ------------------------------------------------------------ elementwise
__global__ void add_kernel(float* __restrict__ dst, const float* __restrict__ src, uint64_t count,
                           bool bf16) {
  const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) dst[i] = actv(dst[i] + src[i], bf16);
}
int launch_add(float* dst, const float* src, uint64_t count, bool bf16, cudaStream_t stream) {
  add_kernel<<<static_cast<unsigned>((count + 255U) / 256U), 256, 0, stream>>>(dst, src, count, bf16);
  count_launch();
  return check_launch("add");
}

__global__ void silu_product_kernel(const float* __restrict__ gate_up, float* __restrict__ out,
                                    uint32_t ffn, bool bf16) {
  const uint32_t row = blockIdx.y;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ffn) return;
  const float g = gate_up[static_cast<size_t>(row) * 2U * ffn + i];
  const float u = gate_up[static_cast<size_t>(row) * 2U * ffn + ffn + i];
  const float a = actv(g / (1.0F + det_expf(-g)), bf16);
  out[static_cast<size_t>(row) * ffn + i] = actv(a * u, bf16);
}
int launch_silu_product(const float* gate_up, float* out, uint32_t rows, uint32_t ffn, bool bf16,
                        cudaStream_t stream) {
  const dim3 grid((ffn + 255U) / 256U, rows);
  silu_product_kernel<<<grid, 256, 0, stream>>>(gate_up, out, ffn, bf16);
  count_launch();
  return check_launch("silu_product");
}

__global__ void copy_rows_kernel(float* __restrict__ dst, uint32_t dst_stride,
                                 const float* __restrict__ src, uint32_t src_stride, uint32_t cols,
                                 const uint32_t* __restrict__ row_select) {
  const uint32_t row = blockIdx.y;
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= cols) return;
  const uint32_t in_row = row_select ? *row_select : row;
  dst[static_cast<size_t>(row) * dst_stride + i] = src[static_cast<size_t>(in_row) * src_stride + i];
}
int launch_copy_rows(float* dst, uint32_t dst_stride, const float* src, uint32_t src_stride,
                     uint32_t rows, uint32_t cols, const uint32_t* row_select, cudaStream_t stream) {
  const dim3 grid((cols + 255U) / 256U, rows);
  copy_rows_kernel<<<grid, 256, 0, stream>>>(dst, dst_stride, src, src_stride, cols, row_select);
  count_launch();
  return check_launch("copy_rows");
}

// ---------------------------------------------------------- argmax / top-k
// Order used everywhere: larger value first, equal values -> lower index first.
__device__ __forceinline__ bool better(float av, uint32_t ai, float bv, uint32_t bi) {
  return av > bv || (av == bv && ai < bi);
}

__device__ __forceinline__ void block_best(float& v, uint32_t& i, float* sv, uint32_t* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffU, v, o);
    const uint32_t oi = __shfl_xor_sync(0xffffffffU, i, o);
    if (better(ov, oi, v, i)) { v = ov; i = oi; }
  }
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  __syncthreads();
  if (lane == 0U) { sv[warp] = v; si[warp] = i; }
  __syncthreads();
  if (warp == 0U) {
    const uint32_t warps = blockDim.x >> 5U;
    v = lane < warps ? sv[lane] : kNegInf;
    i = lane < warps ? si[lane] : 0xffffffffU;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffU, v, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffU, i, o);
      if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    if (lane == 0U) { sv[0] = v; si[0] = i; }
  }
  __syncthreads();
  v = sv[0];
  i = si[0];
}

__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ values, uint32_t count, uint32_t row_stride,
              uint32_t* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  const float* v = values + static_cast<size_t>(blockIdx.x) * row_stride;
  float best = kNegInf;
  uint32_t index = 0xffffffffU;
  if ((reinterpret_cast<uintptr_t>(v) & 15U) == 0U) {
    // 16-byte loads, four in flight per thread
    const float4* v4 = reinterpret_cast<const float4*>(v);
    const uint32_t n4 = count / 4U;
#pragma unroll 4
    for (uint32_t i = threadIdx.x; i < n4; i += blockDim.x) {
      const float4 x = __ldg(v4 + i);
      const uint32_t b = 4U * i;
      if (better(x.x, b, best, index)) { best = x.x; index = b; }
      if (better(x.y, b + 1U, best, index)) { best = x.y; index = b + 1U; }
      if (better(x.z, b + 2U, best, index)) { best = x.z; index = b + 2U; }
      if (better(x.w, b + 3U, best, index)) { best = x.w; index = b + 3U; }
    }
    for (uint32_t i = 4U * n4 + threadIdx.x; i < count; i += blockDim.x) {
      const float x = v[i];
      if (better(x, i, best, index)) { best = x; index = i; }
    }
  } else {
    for (uint32_t i = threadIdx.x; i < count; i += blockDim.x) {
      const float x = v[i];
      if (better(x, i, best, index)) { best = x; index = i; }
    }
  }
  block_best(best, index, sv, si);
  if (threadIdx.x == 0U) out[blockIdx.x] = index;
}
int launch_argmax(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride,
                  uint32_t* out, cudaStream_t stream) {
  argmax_kernel<<<rows, 1024, 0, stream>>>(values, count, row_stride, out);
  count_launch();
  return check_launch("argmax");
}

// Exact top-k (k <= 64): every CTA ranks the k best of its 4096-value chunk by k
// successive block-wide selections; a second kernel ranks the chunk winners.
constexpr uint32_t kTopkChunk = 4096;

__global__ void __launch_bounds__(256)
topk_chunk_kernel(const float* __restrict__ values, uint32_t count, uint32_t row_stride, uint32_t k,
                  float* __restrict__ part_values, uint32_t* __restrict__ part_tokens,
                  uint32_t chunks) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  __shared__ float chunk[kTopkChunk];
  const uint32_t row = blockIdx.y, c = blockIdx.x;
  const float* v = values + static_cast<size_t>(row) * row_stride;
  const uint32_t first = c * kTopkChunk;
  const uint32_t n = min(kTopkChunk, count - first);
  for (uint32_t i = threadIdx.x; i < kTopkChunk; i += blockDim.x) {
    const float x = i < n ? v[first + i] : kNegInf;
    chunk[i] = isnan(x) ? kNegInf : x;  // NaN never ranks
  }
  __syncthreads();
  for (uint32_t rank = 0; rank < k; ++rank) {
    float best = kNegInf;
    uint32_t index = 0xffffffffU;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x)
      if (better(chunk[i], first + i, best, index)) { best = chunk[i]; index = first + i; }
    block_best(best, index, sv, si);
    if (threadIdx.x == 0U) {
      const size_t o = (static_cast<size_t>(row) * chunks + c) * k + rank;
      part_values[o] = best;
      part_tokens[o] = index;
      // taken entries drop below every real value and lose every index tie
      if (index != 0xffffffffU) chunk[index - first] = -INFINITY;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256)
topk_merge_kernel(float* __restrict__ part_values, const uint32_t* __restrict__ part_tokens,
                  uint32_t items, uint32_t k, float* __restrict__ out_values,
                  uint32_t* __restrict__ out_tokens) {
  __shared__ float sv[32];
  __shared__ uint32_t si[32];
  const uint32_t row = blockIdx.x;
  float* pv = part_values + static_cast<size_t>(row) * items;
  const uint32_t* pt = part_tokens + static_cast<size_t>(row) * items;
  for (uint32_t rank = 0; rank < k; ++rank) {
    float best = kNegInf;
    uint32_t index = 0xffffffffU, slot = 0xffffffffU;
    for (uint32_t i = threadIdx.x; i < items; i += blockDim.x) {
      const uint32_t t = pt[i];
      if (t != 0xffffffffU && pv[i] != -INFINITY && better(pv[i], t, best, index)) {
        best = pv[i]; index = t; slot = i;
      }
    }
    // the winner's slot travels with its token id (token ids are unique per row)
    float bv = best;
    uint32_t bi = index;
    block_best(bv, bi, sv, si);
    if (bi != 0xffffffffU && bi == index && slot != 0xffffffffU) pv[slot] = -INFINITY;
    if (threadIdx.x == 0U) {
      out_values[static_cast<size_t>(row) * k + rank] = bv;
      out_tokens[static_cast<size_t>(row) * k + rank] = bi;
    }
    __syncthreads();
  }
}

size_t topk_workspace_bytes(uint32_t rows, uint32_t count, uint32_t k) {
  const size_t chunks = (count + kTopkChunk - 1U) / kTopkChunk;
  return static_cast<size_t>(rows) * chunks * k * (sizeof(float) + sizeof(uint32_t));
}

int launch_topk(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride, uint32_t k,
                float* out_values, uint32_t* out_tokens, void* workspace, cudaStream_t stream) {
  const uint32_t chunks = (count + kTopkChunk - 1U) / kTopkChunk;
  float* pv = static_cast<float*>(workspace);
  uint32_t* pt = reinterpret_cast<uint32_t*>(pv + static_cast<size_t>(rows) * chunks * k);
  topk_chunk_kernel<<<dim3(chunks, rows), 256, 0, stream>>>(values, count, row_stride, k, pv, pt,
                                                           chunks);
  topk_merge_kernel<<<rows, 256, 0, stream>>>(pv, pt, chunks * k, k, out_values, out_tokens);
  count_launch(2);
  return check_launch("topk");
}

}  // namespace qllm
