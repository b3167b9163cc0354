// RoPE + INT8 query quantisation + K/V record store for ONE head (head_dim 128) of up to eight
// rows, as the finishing step of the fused q/k/v projection: the CTA that adds up a head's split-K
// partial sums rotates and stores that head itself, instead of a separate kernel after the GEMV.
// Same arithmetic and the same bytes as rope_kv_store_warp128_kernel (kernels_attention.cu), whose
// reference is runtime/src/cuda/transformer_kernels.cu:229-288, 601-625, 3551-3643.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace qllm {

struct RopeTail {
  RopeStoreArgs a;        // qkv pointer unused
  float* q_out;           // [rows, q_heads*128] rotated queries
  int8_t* q8_out;         // optional INT8 queries [rows, q_heads, 128]
  float* q8_scale;        // [rows, q_heads]
  uint32_t* tickets;      // one counter per 128-row tile of the projection, zero between launches
};

// One warp, one (head, row): `in` = the lane's four consecutive dims (4*lane ..) of the projected
// row (already BF16-rounded by the GEMV's output rule).  head < q_heads: query; < q_heads+kv_heads:
// key; else value.
__device__ __forceinline__ void rope_tail_head_row(const RopeTail& t, uint32_t head, uint32_t row, const float (&in)[4],
                                                   uint32_t lane) {
  const RopeStoreArgs& a = t.a;
  constexpr uint32_t hd = 128;
  const uint32_t cache_position = *a.first_position + a.position_offset + row;
  const uint32_t rotary_position = cache_position + a.rotary_offset;
  const uint32_t d0 = 4U * lane, half = a.rotary_dim / 2U;
  const bool is_value = head >= a.q_heads + a.kv_heads;
  float result[4];
  if (!is_value) {
    const float src[4] = {actv(in[0], a.bf16), actv(in[1], a.bf16), actv(in[2], a.bf16), actv(in[3], a.bf16)};
    const bool rotated = d0 < a.rotary_dim;      // rotary_dim % 8 == 0: a lane is inside or outside
    const bool low = d0 < half;
    const uint32_t partner = rotated ? (low ? lane + half / 4U : lane - half / 4U) : lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other_raw = __shfl_sync(0xffffffffU, src[i], partner);
      result[i] = src[i];
      if (rotated) {
        const uint32_t pair = (d0 + i) % half;
        const float angle = static_cast<float>(rotary_position) * a.inv_freq[pair];
        const float other = low ? -other_raw : other_raw;
        float sine, cosine;
        if (a.exact) det_sincosf(angle, &sine, &cosine);
        else { sine = sinf(angle); cosine = cosf(angle); }
        result[i] = src[i] * actv(cosine, a.bf16) + other * actv(sine, a.bf16);
      }
      result[i] = actv(result[i], a.bf16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) result[i] = in[i];
  }
  if (head < a.q_heads) {
    const size_t item_q = static_cast<size_t>(row) * a.q_heads + head;
    *reinterpret_cast<float4*>(t.q_out + item_q * hd + d0) = make_float4(result[0], result[1], result[2], result[3]);
    if (t.q8_out) {
      const float qmax = warp_max(fmaxf(fmaxf(fabsf(result[0]), fabsf(result[1])), fmaxf(fabsf(result[2]), fabsf(result[3]))));
      const float qsc = fmaxf(qmax / 127.0F, 0x1p-24F);
      uint32_t packed = 0U;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        packed |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(result[i] / qsc)))) & 0xffU) << (8 * i);
      *reinterpret_cast<uint32_t*>(t.q8_out + item_q * hd + d0) = packed;
      if (lane == 0U) t.q8_scale[item_q] = qsc;
    }
    return;
  }
  // K or V record of kv head `kvh`
  const uint32_t kvh = is_value ? head - a.q_heads - a.kv_heads : head - a.q_heads;
  const uint32_t pt = a.page_tokens;
  uint8_t* layer = a.page_table[cache_position / pt] + a.layer_offset;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  const uint32_t slot = cache_position % pt;
  if (a.encoding == QLLM_KV_F16) {
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    __half* dst = reinterpret_cast<__half*>(layer + (is_value ? records * hd * 2U : 0U)) + rec * hd + d0;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[i] = __float2half_rn(result[i]);
    return;
  }
  const float vmax = warp_max(fmaxf(fmaxf(fabsf(result[0]), fabsf(result[1])), fmaxf(fabsf(result[2]), fabsf(result[3]))));
  if (a.encoding == QLLM_KV_Q4H) {
    const __half sh = __float2half_rn(fmaxf(vmax / 7.0F, 0x1p-24F));
    const float sc = __half2float(sh);
    uint8_t* codes = layer + (is_value ? records * (hd / 2U) + records * 2U : 0U);
    uint8_t* scales = codes + records * (hd / 2U);
    const size_t rec = static_cast<size_t>(kvh) * pt + slot;
    if (lane == 0U) reinterpret_cast<__half*>(scales)[rec] = sh;
    uint32_t b = 0U;  // two bytes: dims (d0, d0+1) and (d0+2, d0+3)
#pragma unroll
    for (int i = 0; i < 4; ++i) b |= (static_cast<uint32_t>(max(-7, min(7, __float2int_rn(result[i] / sc)))) & 15U) << (4 * i);
    reinterpret_cast<uint16_t*>(codes + rec * (hd / 2U))[lane] = static_cast<uint16_t>(b);
  } else {  // Q8: records are 2-byte aligned
    const __half sh = __float2half_rn(fmaxf(vmax / 127.0F, 0x1p-24F));
    const float sc = __half2float(sh);
    const size_t rb = hd + 2U;
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    uint8_t* r8 = layer + (is_value ? records * rb : 0U) + rec * rb;
    if (lane == 0U) *reinterpret_cast<__half*>(r8 + hd) = sh;
    uint32_t b = 0U;
#pragma unroll
    for (int i = 0; i < 4; ++i) b |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(result[i] / sc)))) & 0xffU) << (8 * i);
    reinterpret_cast<uint16_t*>(r8)[2U * lane] = static_cast<uint16_t>(b & 0xffffU);
    reinterpret_cast<uint16_t*>(r8)[2U * lane + 1U] = static_cast<uint16_t>(b >> 16U);
  }
}

}  // namespace qllm
