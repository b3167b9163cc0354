// Shared device helpers and the internal (C++) launch interface of the kernel layer.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <cstring>
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

// Transcendentals that give the same bits on the host and on the device: only IEEE double
// additions, multiplications and divisions in a fixed order (no fused multiply-add on either side),
// a round-to-nearest-integer and an exponent built from bits.  The library functions (expf, cosf)
// differ in the last place between vendors, and a last-place difference that crosses a BF16
// rounding boundary changes every later step of a W4A4 decoder.
__host__ __device__ __forceinline__ double det_exp_core(double x) {  // |x| < 700
  const double k = rint(x * 1.4426950408889634);
  const double r = (x - k * 6.93147180369123816490e-01) - k * 1.90821492927058770002e-10;
  // Taylor series of exp(r), |r| <= 0.35, to r^14 / 14!
  double p = 1.0 / 87178291200.0;
  p = p * r + 1.0 / 6227020800.0;
  p = p * r + 1.0 / 479001600.0;
  p = p * r + 1.0 / 39916800.0;
  p = p * r + 1.0 / 3628800.0;
  p = p * r + 1.0 / 362880.0;
  p = p * r + 1.0 / 40320.0;
  p = p * r + 1.0 / 5040.0;
  p = p * r + 1.0 / 720.0;
  p = p * r + 1.0 / 120.0;
  p = p * r + 1.0 / 24.0;
  p = p * r + 1.0 / 6.0;
  p = p * r + 0.5;
  p = p * r + 1.0;
  p = p * r + 1.0;
  const long long e = static_cast<long long>(k) + 1023LL;  // 2^k as a double, built from its bits
  const unsigned long long bits = static_cast<unsigned long long>(e) << 52U;
  double scale;
  memcpy(&scale, &bits, sizeof(scale));
  return p * scale;
}
__host__ __device__ __forceinline__ float det_expf(float x) {
  if (!(x > -104.0F)) return 0.0F;       // below the smallest float (and NaN)
  if (x > 88.0F) x = 88.0F;
  return static_cast<float>(det_exp_core(static_cast<double>(x)));
}
// sin and cos of a float angle (|angle| < 2^20): three-part reduction by pi/2, Taylor series on
// [-pi/4, pi/4] to r^17 and r^16.
__host__ __device__ __forceinline__ void det_sincosf(float angle, float* sine, float* cosine) {
  const double x = static_cast<double>(angle);
  const double k = rint(x * 0.63661977236758134308);
  const double r = ((x - k * 1.57079632673412561417e+00) - k * 6.07710050630396597660e-11) -
                   k * 2.02226624879595063154e-21;
  const double z = r * r;
  double s = -1.0 / 355687428096000.0;   // r^17 / 17!
  s = s * z + 1.0 / 1307674368000.0;
  s = s * z - 1.0 / 6227020800.0;
  s = s * z + 1.0 / 39916800.0;
  s = s * z - 1.0 / 362880.0;
  s = s * z + 1.0 / 5040.0;
  s = s * z - 1.0 / 120.0;
  s = s * z + 1.0 / 6.0;
  s = r - r * z * s;
  double c = 1.0 / 20922789888000.0;     // r^16 / 16!
  c = c * z - 1.0 / 87178291200.0;
  c = c * z + 1.0 / 479001600.0;
  c = c * z - 1.0 / 3628800.0;
  c = c * z + 1.0 / 40320.0;
  c = c * z - 1.0 / 720.0;
  c = c * z + 1.0 / 24.0;
  c = c * z - 0.5;
  c = c * z + 1.0;
  const long long q = static_cast<long long>(k) & 3LL;
  const double sv = (q == 0) ? s : (q == 1) ? c : (q == 2) ? -s : -c;
  const double cv = (q == 0) ? c : (q == 1) ? -s : (q == 2) ? -c : s;
  *sine = static_cast<float>(sv);
  *cosine = static_cast<float>(cv);
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
