// Exact NVFP4 x NVFP4 block arithmetic on the CUDA cores, shared by the CUDA-core GEMV and the
// routed-expert kernels: E2M1 codes expanded to INT8 (twice the value), activations quantised
// to the same INT8 form, one dp4a chain per 16-value block, block terms summed in double.
#pragma once

#include "common.cuh"

namespace qllm {

// prmt.b32 in its default mode: selector nibble bits 2:0 pick a byte of {a, b}; bit 3
// replaces the byte by eight copies of its sign bit.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ void expand_fp4x8(uint32_t w, uint32_t& lo4, uint32_t& hi4) {
  // bytes of twice the E2M1 value of nibbles 0..3 (lo4) and 4..7 (hi4), element order kept
  constexpr uint32_t kPos0 = 0x03020100U, kPos1 = 0x0c080604U;  // 0 1 2 3 | 4 6 8 12
  constexpr uint32_t kNeg0 = 0xfdfeff00U, kNeg1 = 0xf4f8fafcU;  // 0 -1 -2 -3 | -4 -6 -8 -12
  const uint32_t wl = w << 4U;
  const uint32_t s_lo = w & 0x7777U, s_hi = (w >> 16U) & 0x7777U;
  const uint32_t pos_lo = prmt(kPos0, kPos1, s_lo), neg_lo = prmt(kNeg0, kNeg1, s_lo);
  const uint32_t pos_hi = prmt(kPos0, kPos1, s_hi), neg_hi = prmt(kNeg0, kNeg1, s_hi);
  // byte masks from the sign bit of each nibble (sign-replicating permute)
  const uint32_t m_lo = prmt(wl, w, 0xd9c8U), m_hi = prmt(wl, w, 0xfbeaU);
  lo4 = (pos_lo & ~m_lo) | (neg_lo & m_lo);
  hi4 = (pos_hi & ~m_hi) | (neg_hi & m_hi);
}

// Integer dot product of one 16-value block: weight codes (8 bytes) against INT8 activations
// (twice the E2M1 value each), i.e. four times the product of the decoded values.
__device__ __forceinline__ int block16_dot(uint2 codes, uint4 x) {
  uint32_t a[4];
  expand_fp4x8(codes.x, a[0], a[1]);
  expand_fp4x8(codes.y, a[2], a[3]);
  int d = __dp4a(static_cast<int>(a[0]), static_cast<int>(x.x), 0);
  d = __dp4a(static_cast<int>(a[1]), static_cast<int>(x.y), d);
  d = __dp4a(static_cast<int>(a[2]), static_cast<int>(x.z), d);
  return __dp4a(static_cast<int>(a[3]), static_cast<int>(x.w), d);
}

// Activation quantiser of one block (the reference's nvfp4_quant_dequant_kernel,
// runtime/src/cuda/transformer_kernels.cu:1943-1967, with the values kept as codes): `local` is
// the decoded E4M3 block scale, packed[] the 16 values as INT8 = twice the E2M1 value.
__device__ __forceinline__ void quantize_block16_i8(const float (&v)[16], float g, uint4& packed, float& local) {
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  local = e4m3_value(e4m3_code(fminf(448.0F, g * amax / 6.0F)));
  uint32_t p[4] = {0U, 0U, 0U, 0U};
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float scaled = local == 0.0F ? 0.0F : fminf(6.0F, fmaxf(-6.0F, v[i] * g / local));
    const unsigned code = e2m1_code(scaled);
    const unsigned m = code & 7U;
    int twice = m < 5U ? static_cast<int>(m) : static_cast<int>(2U * m - 4U) + (m == 7U ? 2 : 0);
    if (code & 8U) twice = -twice;
    p[i / 4] |= (static_cast<uint32_t>(twice) & 0xffU) << (8 * (i % 4));
  }
  packed = make_uint4(p[0], p[1], p[2], p[3]);
}

}  // namespace qllm
