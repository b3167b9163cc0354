// Device-side NVFP4 activation quantisation shared by the fused producer kernels, and the
// descriptor of a GEMV result that its consumers read (final values or split-K partials).
#pragma once

#include "common.cuh"

namespace qllm {

// Where quantised activations go: the operand format of the CUDA-core GEMV (INT8 values +
// FP32 block scales) or of the tensor-core GEMV (packed E2M1 codes + E4M3 scale atoms).
struct QuantSink {
  int kind;          // 0 = CUDA-core operand, 1 = tensor-core operand
  int8_t* xi8;       // [rows, cols]
  float* xscale;     // [rows, cols/16]
  uint8_t* codes;    // [rows_padded, cols/2]
  uint8_t* atoms;    // [cols/64][512]: (row%32)*16 + (row/32)*4 + block%4
  uint32_t cols;     // row length of the operand (K of the GEMV that consumes it)
  float g;           // activation global scale of that GEMV
};

// Quantises 16 consecutive values (block `block` of row `row`) and stores them.
__device__ __forceinline__ void quant_store_block16(const QuantSink& q, uint32_t row, uint32_t block,
                                                    const float (&v)[16]) {
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const unsigned sc = e4m3_code(fminf(448.0F, q.g * amax / 6.0F));
  const float local = e4m3_value(sc);
  if (q.kind == 0) {
    uint32_t packed[4] = {0U, 0U, 0U, 0U};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float scaled = local == 0.0F ? 0.0F : fminf(6.0F, fmaxf(-6.0F, v[i] * q.g / local));
      const unsigned code = e2m1_code(scaled);
      const unsigned m = code & 7U;
      int twice = m < 5U ? static_cast<int>(m) : static_cast<int>(2U * m - 4U) + (m == 7U ? 2 : 0);
      if (code & 8U) twice = -twice;
      packed[i / 4] |= (static_cast<uint32_t>(twice) & 0xffU) << (8 * (i % 4));
    }
    const size_t blocks = q.cols / 16U;
    reinterpret_cast<uint4*>(q.xi8 + static_cast<size_t>(row) * q.cols)[block] =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
    q.xscale[static_cast<size_t>(row) * blocks + block] = local;
  } else {
    uint32_t packed[2] = {0U, 0U};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      unsigned code = 0U;
      if (local != 0.0F) code = e2m1_code(fminf(6.0F, fmaxf(-6.0F, v[i] * q.g / local)));
      packed[i / 8] |= code << (4 * (i % 8));
    }
    reinterpret_cast<uint2*>(q.codes + static_cast<size_t>(row) * (q.cols / 2U))[block] =
        make_uint2(packed[0], packed[1]);
    const uint32_t tile = row / 128U, r = row % 128U;
    q.atoms[(static_cast<size_t>(tile) * (q.cols / 64U) + block / 4U) * 512U + (r % 32U) * 16U + (r / 32U) * 4U +
            block % 4U] = static_cast<uint8_t>(sc);
  }
}

// Warp-cooperative form: four consecutive lanes hold one 16-value block as a float4 each
// (lane & 3 = position inside the block).  All 32 lanes must call it; lanes with
// valid == false take part in the shuffles only.
__device__ __forceinline__ void quant_store_quad(const QuantSink& q, uint32_t row, uint32_t block, float4 v,
                                                 bool valid) {
  const uint32_t quad_lane = threadIdx.x & 3U;
  float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffU, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffU, amax, 2));
  if (!valid) return;
  const unsigned sc = e4m3_code(fminf(448.0F, q.g * amax / 6.0F));
  const float local = e4m3_value(sc);
  const float in[4] = {v.x, v.y, v.z, v.w};
  unsigned code[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    code[i] = local == 0.0F ? 0U : e2m1_code(fminf(6.0F, fmaxf(-6.0F, in[i] * q.g / local)));
  if (q.kind == 0) {
    uint32_t packed = 0U;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned m = code[i] & 7U;
      int twice = m < 5U ? static_cast<int>(m) : static_cast<int>(2U * m - 4U) + (m == 7U ? 2 : 0);
      if (code[i] & 8U) twice = -twice;
      packed |= (static_cast<uint32_t>(twice) & 0xffU) << (8 * i);
    }
    reinterpret_cast<uint32_t*>(q.xi8 + static_cast<size_t>(row) * q.cols)[block * 4U + quad_lane] = packed;
    if (quad_lane == 0U) q.xscale[static_cast<size_t>(row) * (q.cols / 16U) + block] = local;
  } else {
    const uint16_t packed = static_cast<uint16_t>(code[0] | (code[1] << 4U) | (code[2] << 8U) | (code[3] << 12U));
    reinterpret_cast<uint16_t*>(q.codes + static_cast<size_t>(row) * (q.cols / 2U))[block * 4U + quad_lane] = packed;
    if (quad_lane == 0U) {
      const uint32_t tile = row / 128U, r = row % 128U;
      q.atoms[(static_cast<size_t>(tile) * (q.cols / 64U) + block / 4U) * 512U + (r % 32U) * 16U + (r / 32U) * 4U +
              block % 4U] = static_cast<uint8_t>(sc);
    }
  }
}

// Result of a GEMV as its consumers see it: either final BF16-rounded values [batch, n], or
// `split` raw FP32 partial sums [split][batch][n] that still need the output scale.
struct GemvOut {
  const float* data;
  uint32_t split;   // 0: data holds final values
  uint32_t n;       // outputs per activation row
  uint32_t batch;
  float weight_scale, input_scale;
  // Tensor-parallel exchange (null: none).  `data` is then a slot of this rank's inbox that
  // holds every rank's partials ([rank][split][batch][n], `split` counting all of them) as
  // 8-byte pairs {FP32 bits, sequence number of the exchange}: a value is valid once its own
  // sequence word equals exchange[1].  The pair is written by one 8-byte store, so no
  // flag, fence or separate signal is involved (gemv_exchange_value4 below).
  // exchange[0]: error word; exchange[1]: exchanges this rank has produced = the number to wait
  // for; exchange[2]: ticket counter of the running producer launch.
  uint32_t* exchange;
};

constexpr uint32_t kExchangePolls = 1U << 21U;  // about a second of polling: the peer counts as lost

__device__ __forceinline__ float gemv_value(const GemvOut& o, uint32_t row, uint32_t col) {
  const size_t i = static_cast<size_t>(row) * o.n + col;
  if (o.split == 0U) return o.data[i];
  float sum = 0.0F;
  const size_t stride = static_cast<size_t>(o.batch) * o.n;
  for (uint32_t s = 0; s < o.split; ++s) sum += o.data[s * stride + i];
  return bf16r(sum * o.weight_scale / o.input_scale);
}

// Four consecutive outputs (col % 4 == 0, n % 4 == 0): 16-byte loads of every split.
__device__ __forceinline__ float4 gemv_value4(const GemvOut& o, uint32_t row, uint32_t col) {
  const size_t i = (static_cast<size_t>(row) * o.n + col) / 4U;
  const float4* data = reinterpret_cast<const float4*>(o.data);
  if (o.split == 0U) return data[i];
  const size_t stride = static_cast<size_t>(o.batch) * o.n / 4U;
  float4 sum = data[i];
  for (uint32_t s = 1; s < o.split; ++s) {
    const float4 t = data[s * stride + i];
    sum.x += t.x; sum.y += t.y; sum.z += t.z; sum.w += t.w;
  }
  return make_float4(bf16r(sum.x * o.weight_scale / o.input_scale), bf16r(sum.y * o.weight_scale / o.input_scale),
                     bf16r(sum.z * o.weight_scale / o.input_scale), bf16r(sum.w * o.weight_scale / o.input_scale));
}

// The same four outputs of an exchanged result (o.exchange set): every partial is an 8-byte pair
// {value, sequence}.  The loads of eight partials go out together (one memory round trip when
// everything has arrived); a batch is read again until all of its sequence words match.  The
// wait is bounded: after the limit the error word is set and whatever is there is used; once
// the error word is set nobody waits any more.  Partials are added in storage order (rank,
// split), the same on every rank.
__device__ __forceinline__ float4 gemv_exchange_value4(const GemvOut& o, uint32_t row, uint32_t col) {
  const uint32_t sequence = *reinterpret_cast<const volatile uint32_t*>(o.exchange + 1);
  const uint4* slot = reinterpret_cast<const uint4*>(o.data);  // two pairs per 16 bytes
  const size_t stride = static_cast<size_t>(o.batch) * o.n / 2U, first = (static_cast<size_t>(row) * o.n + col) / 2U;
  float4 sum = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
  constexpr uint32_t kBatch = 8;
  for (uint32_t s0 = 0; s0 < o.split; s0 += kBatch) {
    uint4 lo[kBatch], hi[kBatch];
    for (uint32_t poll = 0;; ++poll) {
      bool complete = true;
#pragma unroll
      for (uint32_t k = 0; k < kBatch; ++k) {
        if (s0 + k >= o.split) break;
        const uint4* p = slot + (s0 + k) * stride + first;
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(lo[k].x), "=r"(lo[k].y), "=r"(lo[k].z), "=r"(lo[k].w) : "l"(p) : "memory");
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(hi[k].x), "=r"(hi[k].y), "=r"(hi[k].z), "=r"(hi[k].w) : "l"(p + 1) : "memory");
      }
#pragma unroll
      for (uint32_t k = 0; k < kBatch; ++k) {
        if (s0 + k >= o.split) break;
        complete = complete && lo[k].y == sequence && lo[k].w == sequence && hi[k].y == sequence && hi[k].w == sequence;
      }
      if (complete) break;
      if (poll >= kExchangePolls ||
          ((poll & 1023U) == 1023U && *reinterpret_cast<volatile uint32_t*>(o.exchange) != 0U)) {
        atomicCAS(o.exchange, 0U, 200U);  // results from here on are invalid; nothing hangs
        break;
      }
    }
#pragma unroll
    for (uint32_t k = 0; k < kBatch; ++k) {
      if (s0 + k >= o.split) break;
      sum.x += __uint_as_float(lo[k].x); sum.y += __uint_as_float(lo[k].z);
      sum.z += __uint_as_float(hi[k].x); sum.w += __uint_as_float(hi[k].z);
    }
  }
  return make_float4(bf16r(sum.x * o.weight_scale / o.input_scale), bf16r(sum.y * o.weight_scale / o.input_scale),
                     bf16r(sum.z * o.weight_scale / o.input_scale), bf16r(sum.w * o.weight_scale / o.input_scale));
}

}  // namespace qllm
