// Shared device helpers and the internal (C++) launch interface of the kernel layer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/qllm_b200.h"

namespace qllm {

constexpr float kNegInf = -3.402823466e+38F;
constexpr unsigned kWarp = 32;

// Last error text of the calling thread (read through qllm_last_error()).
void set_error(const std::string& message);
int fail(int status, const std::string& message);
int check_cuda(cudaError_t error, const char* what);
int check_launch(const char* what);
void count_launch(unsigned launches = 1);
unsigned long long launches_counted();

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ float actv(float v, bool bf16) { return bf16 ? bf16r(v) : v; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffU, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffU, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, o));
  return v;
}

// E2M1 value of a 4-bit code.
__device__ __forceinline__ float e2m1_value(unsigned code) {
  // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6: exponent/mantissa arithmetic, no table
  const unsigned m = code & 7U;
  float v = m < 2U ? 0.5F * static_cast<float>(m)
                   : __uint_as_float(((126U + (m >> 1U)) << 23U) | ((m & 1U) << 22U));
  return (code & 8U) ? -v : v;
}
// Nearest E2M1 code, ties to the even code.
__device__ __forceinline__ unsigned e2m1_code(float value) {
  const float m = fabsf(value);
  unsigned index = 0;
  if (m > 5.0F) index = 7;
  else if (m >= 3.5F) index = 6;
  else if (m > 2.5F) index = 5;
  else if (m >= 1.75F) index = 4;
  else if (m > 1.25F) index = 3;
  else if (m >= 0.75F) index = 2;
  else if (m > 0.25F) index = 1;
  return index | (value < 0.0F ? 8U : 0U);
}
__device__ __forceinline__ float e4m3_value(unsigned code) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(code), __NV_E4M3);
  return __half2float(__half(h));
}
__device__ __forceinline__ unsigned e4m3_code(float value) {
  return static_cast<unsigned>(__nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3));
}

}  // namespace qllm
