// CPU oracle for the MTP-4 speculative decode step -- TEST INFRASTRUCTURE ONLY.
// See qllm_oracle.h for the list of reference files restated here.  Nothing in
// the shipped library may call into this file.
#include "qllm_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include <omp.h>

namespace {

thread_local std::string g_error;

constexpr float kNegInf = -3.402823466e+38F;  // transformer_kernels.cu:41

// ------------------------------------------------------------------ formats
float bf16_round(float value) {
  // round-to-nearest-even on the upper 16 bits (__float2bfloat16_rn)
  uint32_t bits;
  std::memcpy(&bits, &value, 4);
  if ((bits & 0x7fffffffU) > 0x7f800000U) return value;  // NaN
  bits += 0x7fffU + ((bits >> 16U) & 1U);
  bits &= 0xffff0000U;
  float out;
  std::memcpy(&out, &bits, 4);
  return out;
}
inline float act(float value, bool bf16) { return bf16 ? bf16_round(value) : value; }

uint16_t f16_bits(float value) {
  const _Float16 h = static_cast<_Float16>(value);  // RN-even
  uint16_t bits;
  std::memcpy(&bits, &h, 2);
  return bits;
}
float f16_value(uint16_t bits) {
  _Float16 h;
  std::memcpy(&h, &bits, 2);
  return static_cast<float>(h);
}
inline float f16_round(float v) { return f16_value(f16_bits(v)); }

// Transcendentals that give the same bits on the host and on the device: only IEEE double
// additions, multiplications and divisions in a fixed order (no fused multiply-add on either side),
// a round-to-nearest-integer and an exponent built from bits.  The library functions (expf, cosf)
// differ in the last place between vendors, and a last-place difference that crosses a BF16
// rounding boundary changes every later step of a W4A4 decoder.
inline double det_exp_core(double x) {  // |x| < 700
  const double k = std::rint(x * 1.4426950408889634);
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
  std::memcpy(&scale, &bits, sizeof(scale));
  return p * scale;
}
inline float det_expf(float x) {
  if (!(x > -104.0F)) return 0.0F;       // below the smallest float (and NaN)
  if (x > 88.0F) x = 88.0F;
  return static_cast<float>(det_exp_core(static_cast<double>(x)));
}
// sin and cos of a float angle (|angle| < 2^20): three-part reduction by pi/2, Taylor series on
// [-pi/4, pi/4] to r^17 and r^16.
inline void det_sincosf(float angle, float* sine, float* cosine) {
  const double x = static_cast<double>(angle);
  const double k = std::rint(x * 0.63661977236758134308);
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


// transformer_kernels.cu:1931-1936
float e2m1_decode(uint8_t code) {
  static const float levels[8] = {0.0F, 0.5F, 1.0F, 1.5F, 2.0F, 3.0F, 4.0F, 6.0F};
  const float v = levels[code & 7U];
  return (code & 8U) ? -v : v;
}
// transformer_kernels.cu:1917-1929 (nearest level, ties to the even code)
uint8_t e2m1_encode(float value) {
  const float m = std::fabs(value);
  uint8_t index = 0;
  if (m > 5.0F) index = 7;
  else if (m >= 3.5F) index = 6;
  else if (m > 2.5F) index = 5;
  else if (m >= 1.75F) index = 4;
  else if (m > 1.25F) index = 3;
  else if (m >= 0.75F) index = 2;
  else if (m > 0.25F) index = 1;
  return static_cast<uint8_t>(index | (value < 0.0F ? 8U : 0U));
}
// E4M3FN: bias 7, no infinities, 0x7f/0xff NaN, subnormals m * 2^-9.
float e4m3_decode(uint8_t code) {
  const uint32_t exponent = (code >> 3U) & 15U;
  const uint32_t mantissa = code & 7U;
  float v;
  if (exponent == 15U && mantissa == 7U) return NAN;
  if (exponent == 0U) v = std::ldexp(static_cast<float>(mantissa), -9);
  else v = std::ldexp(1.0F + static_cast<float>(mantissa) / 8.0F, static_cast<int>(exponent) - 7);
  return (code & 0x80U) ? -v : v;
}
// __nv_fp8_e4m3(float): round-to-nearest-even, saturate to +-448.
uint8_t e4m3_encode(float value) {
  if (std::isnan(value)) return 0x7fU;
  const uint8_t sign = std::signbit(value) ? 0x80U : 0U;
  const float a = std::fabs(value);
  if (a > 448.0F) return sign | 0x7eU;
  if (a == 0.0F) return sign;
  int e;
  std::frexp(a, &e);
  int exponent = e - 1;  // a = 1.f * 2^exponent
  if (exponent < -6) {
    const float q = std::nearbyint(std::ldexp(a, 9));  // multiples of 2^-9
    return sign | static_cast<uint8_t>(q);  // q == 8 is the code of 2^-6
  }
  float mantissa = std::nearbyint((std::ldexp(a, -exponent) - 1.0F) * 8.0F);
  if (mantissa == 8.0F) { mantissa = 0.0F; ++exponent; }
  if (exponent > 8 || (exponent == 8 && mantissa > 6.0F)) return sign | 0x7eU;
  return sign | static_cast<uint8_t>(((exponent + 7) << 3) | static_cast<int>(mantissa));
}

// ------------------------------------------------------------------- NVFP4
// Harness-owned weight quantiser: the reference's activation quantiser formula
// (transformer_kernels.cu:1943-1968) applied to weight rows.
void nvfp4_quantize_weights(const float* w, uint32_t rows, uint32_t cols, float g,
                            uint8_t* codes, uint8_t* scales) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < static_cast<int64_t>(rows); ++r) {
    for (uint32_t b = 0; b < cols / 16U; ++b) {
      const float* x = w + static_cast<size_t>(r) * cols + b * 16U;
      float amax = 0.0F;
      for (int i = 0; i < 16; ++i) amax = std::fmax(amax, std::fabs(x[i]));
      const uint8_t sc = e4m3_encode(std::fmin(448.0F, g * amax / 6.0F));
      const float local = e4m3_decode(sc);
      scales[static_cast<size_t>(r) * (cols / 16U) + b] = sc;
      for (int i = 0; i < 16; i += 2) {
        uint8_t lo = 0, hi = 0;
        if (local != 0.0F) {
          lo = e2m1_encode(std::fmin(6.0F, std::fmax(-6.0F, x[i] * g / local)));
          hi = e2m1_encode(std::fmin(6.0F, std::fmax(-6.0F, x[i + 1] * g / local)));
        }
        codes[static_cast<size_t>(r) * (cols / 2U) + b * 8U + i / 2] =
            static_cast<uint8_t>(lo | (hi << 4U));
      }
    }
  }
}

inline float nvfp4_weight(const qo_matrix& m, uint32_t row, uint32_t col) {
  const uint8_t packed = m.codes[static_cast<size_t>(row) * (m.cols / 2U) + col / 2U];
  const uint8_t code = (col & 1U) ? (packed >> 4U) : (packed & 15U);
  return e2m1_decode(code) *
         e4m3_decode(m.scales[static_cast<size_t>(row) * (m.cols / 16U) + col / 16U]) *
         m.weight_scale;
}

// transformer_kernels.cu:1943-1968
void nvfp4_fake_quant(const float* x, uint32_t rows, uint32_t cols, float g, float* out) {
  for (uint32_t r = 0; r < rows; ++r)
    for (uint32_t b = 0; b < cols / 16U; ++b) {
      const float* in = x + static_cast<size_t>(r) * cols + b * 16U;
      float* o = out + static_cast<size_t>(r) * cols + b * 16U;
      float amax = 0.0F;
      for (int i = 0; i < 16; ++i) amax = std::fmax(amax, std::fabs(in[i]));
      const float local = e4m3_decode(e4m3_encode(std::fmin(448.0F, g * amax / 6.0F)));
      for (int i = 0; i < 16; ++i) {
        const float scaled =
            local == 0.0F ? 0.0F : std::fmin(6.0F, std::fmax(-6.0F, in[i] * g / local));
        o[i] = e2m1_decode(e2m1_encode(scaled)) * local / g;
      }
    }
}

// Activation side of the W4A4 product: per 16 values the E4M3 block scale and the
// E2M1 codes of transformer_kernels.cu:1943-1968 (the fake-quantised value is
// code * scale / g).
void nvfp4_quantize_activations(const float* x, uint32_t rows, uint32_t cols, float g,
                                uint8_t* codes, uint8_t* scales) {
  for (uint32_t r = 0; r < rows; ++r)
    for (uint32_t b = 0; b < cols / 16U; ++b) {
      const float* in = x + static_cast<size_t>(r) * cols + b * 16U;
      float amax = 0.0F;
      for (int i = 0; i < 16; ++i) amax = std::fmax(amax, std::fabs(in[i]));
      const uint8_t sc = e4m3_encode(std::fmin(448.0F, g * amax / 6.0F));
      const float local = e4m3_decode(sc);
      scales[static_cast<size_t>(r) * (cols / 16U) + b] = sc;
      for (int i = 0; i < 16; ++i) {
        const float scaled =
            local == 0.0F ? 0.0F : std::fmin(6.0F, std::fmax(-6.0F, in[i] * g / local));
        codes[static_cast<size_t>(r) * cols + b * 16U + i] = e2m1_encode(scaled);
      }
    }
}

// transformer_kernels.cu:1970-2002 + launcher 7970-8001: W4A4 product of the
// fake-quantised activations with the decoded weights, BF16-rounded output.
// The reference accumulates in FP32 in an order that is not part of its contract;
// here the sum is formed (to double precision) exactly and rounded once:
//   S = sum_blocks (sum_i cw_i * cx_i) * sw * sx          (every block term is exact)
//   y = bf16(float(S) * weight_scale / input_scale)
void nvfp4_gemv(const qo_matrix& m, uint32_t first_row, uint32_t row_count,
                const float* x, uint32_t batch, float* y) {
  const uint32_t blocks = m.cols / 16U;
  std::vector<uint8_t> xc(static_cast<size_t>(batch) * m.cols), xs(static_cast<size_t>(batch) * blocks);
  nvfp4_quantize_activations(x, batch, m.cols, m.input_scale, xc.data(), xs.data());
  // twice the E2M1 value as an integer
  static const int twice[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};
  std::vector<int8_t> xi(xc.size());
  for (size_t i = 0; i < xc.size(); ++i) xi[i] = static_cast<int8_t>(twice[xc[i]]);
  std::vector<float> xsf(xs.size());
  for (size_t i = 0; i < xs.size(); ++i) xsf[i] = e4m3_decode(xs[i]);
#pragma omp parallel for schedule(static)
  for (int64_t rr = 0; rr < static_cast<int64_t>(row_count); ++rr) {
    const uint32_t row = first_row + static_cast<uint32_t>(rr);
    const uint8_t* codes = m.codes + static_cast<size_t>(row) * (m.cols / 2U);
    const uint8_t* scales = m.scales + static_cast<size_t>(row) * blocks;
    std::vector<double> acc(batch, 0.0);
    int wi[16];
    for (uint32_t b = 0; b < blocks; ++b) {
      const float sw = e4m3_decode(scales[b]);
      for (int i = 0; i < 8; ++i) {
        const uint8_t p = codes[b * 8U + i];
        wi[2 * i] = twice[p & 15U];
        wi[2 * i + 1] = twice[p >> 4U];
      }
      for (uint32_t q = 0; q < batch; ++q) {
        const int8_t* xr = xi.data() + static_cast<size_t>(q) * m.cols + b * 16U;
        int isum = 0;
        for (int i = 0; i < 16; ++i) isum += wi[i] * xr[i];
        const float term = static_cast<float>(isum) * (sw * xsf[static_cast<size_t>(q) * blocks + b]) * 0.25F;
        acc[q] += static_cast<double>(term);
      }
    }
    for (uint32_t q = 0; q < batch; ++q)
      y[static_cast<size_t>(q) * row_count + rr] =
          bf16_round(static_cast<float>(acc[q]) * m.weight_scale / m.input_scale);
  }
}

// ------------------------------------------------------------ layer pieces
// transformer_kernels.cu:2487-2503
void rmsnorm(const float* x, const float* w, float* out, uint32_t rows, uint32_t cols, float eps) {
  for (uint32_t r = 0; r < rows; ++r) {
    const float* in = x + static_cast<size_t>(r) * cols;
    float* o = out + static_cast<size_t>(r) * cols;
    double sq = 0.0;
    for (uint32_t i = 0; i < cols; ++i) sq += static_cast<double>(in[i]) * in[i];
    const float inverse =
        1.0F / std::sqrt(static_cast<float>(sq) / static_cast<float>(cols) + eps);
    for (uint32_t i = 0; i < cols; ++i) o[i] = in[i] * inverse * w[i];
  }
}

// Rotate-half RoPE (transformer_kernels.cu:3590-3606, plain GQA without the
// per-head norm): cos/sin and the result are rounded when act_bf16 is set.
void rope(float* heads, uint32_t rows, uint32_t head_count, uint32_t head_dim,
          uint32_t rotary_dim, float theta, const uint32_t* positions, bool bf16) {
  const uint32_t half = rotary_dim / 2U;
  std::vector<float> inv(half), src(head_dim);
  for (uint32_t p = 0; p < half; ++p)
    inv[p] = std::pow(theta, -2.0F * static_cast<float>(p) / static_cast<float>(rotary_dim));
  for (uint32_t r = 0; r < rows; ++r)
    for (uint32_t h = 0; h < head_count; ++h) {
      float* v = heads + (static_cast<size_t>(r) * head_count + h) * head_dim;
      for (uint32_t d = 0; d < head_dim; ++d) src[d] = act(v[d], bf16);
      for (uint32_t d = 0; d < head_dim; ++d) {
        float result = src[d];
        if (d < rotary_dim) {
          const uint32_t pair = d % half;
          const float angle = static_cast<float>(positions[r]) * inv[pair];
          const float other = d < half ? -src[d + half] : src[d - half];
          float sine, cosine;
          det_sincosf(angle, &sine, &cosine);
          result = src[d] * act(cosine, bf16) + other * act(sine, bf16);
        }
        v[d] = act(result, bf16);
      }
    }
}

size_t kv_layer_bytes(uint32_t enc, uint32_t pt, uint32_t kv, uint32_t hd) {
  const size_t records = static_cast<size_t>(pt) * kv;
  switch (enc) {
    case QO_KV_F16: return records * hd * 2U * 2U;
    case QO_KV_Q4H: return records * (hd / 2U + 2U) * 2U;
    case QO_KV_Q8: return records * (hd + 2U) * 2U;
  }
  return 0;
}

inline int clamp_rn(float v, int lo, int hi) {
  // __float2int_rn then clamp
  const float r = std::nearbyint(v);
  if (!(r >= static_cast<float>(lo))) return lo;  // also NaN -> lo (not reached by valid data)
  if (r > static_cast<float>(hi)) return hi;
  return static_cast<int>(r);
}

// One K/V record store per (row, kv head): transformer_kernels.cu:229-288 (Q4H),
// 601-625 (Q8), 4208-4230 (exact F16, token-major).
void kv_store(uint32_t enc, uint8_t* const* pages, size_t layer_offset, uint32_t pt,
              uint32_t kv, uint32_t hd, const float* key, const float* value, uint32_t rows,
              uint32_t row_stride, uint32_t first_pos) {
  const size_t records = static_cast<size_t>(pt) * kv;
  for (uint32_t r = 0; r < rows; ++r) {
    const uint32_t pos = first_pos + r;
    uint8_t* layer = pages[pos / pt] + layer_offset;
    for (uint32_t h = 0; h < kv; ++h) {
      const float* k = key + static_cast<size_t>(r) * row_stride + h * hd;
      const float* v = value + static_cast<size_t>(r) * row_stride + h * hd;
      float kmax = 0.0F, vmax = 0.0F;
      for (uint32_t d = 0; d < hd; ++d) {
        kmax = std::fmax(kmax, std::fabs(k[d]));
        vmax = std::fmax(vmax, std::fabs(v[d]));
      }
      if (enc == QO_KV_Q4H) {
        const uint16_t ksb = f16_bits(std::fmax(kmax / 7.0F, 0x1p-24F));
        const uint16_t vsb = f16_bits(std::fmax(vmax / 7.0F, 0x1p-24F));
        const float ks = f16_value(ksb), vs = f16_value(vsb);
        uint8_t* kc = layer;
        uint8_t* ksc = kc + records * (hd / 2U);
        uint8_t* vc = ksc + records * 2U;
        uint8_t* vsc = vc + records * (hd / 2U);
        const size_t rec = static_cast<size_t>(h) * pt + pos % pt;
        std::memcpy(ksc + rec * 2U, &ksb, 2);
        std::memcpy(vsc + rec * 2U, &vsb, 2);
        for (uint32_t d = 0; d < hd / 2U; ++d) {
          const int kl = clamp_rn(k[2 * d] / ks, -7, 7), kh = clamp_rn(k[2 * d + 1] / ks, -7, 7);
          const int vl = clamp_rn(v[2 * d] / vs, -7, 7), vh = clamp_rn(v[2 * d + 1] / vs, -7, 7);
          kc[rec * (hd / 2U) + d] = static_cast<uint8_t>((kl & 15) | ((kh & 15) << 4));
          vc[rec * (hd / 2U) + d] = static_cast<uint8_t>((vl & 15) | ((vh & 15) << 4));
        }
      } else if (enc == QO_KV_Q8) {
        const uint16_t ksb = f16_bits(std::fmax(kmax / 127.0F, 0x1p-24F));
        const uint16_t vsb = f16_bits(std::fmax(vmax / 127.0F, 0x1p-24F));
        const float ks = f16_value(ksb), vs = f16_value(vsb);
        const size_t rb = hd + 2U;
        const size_t rec = static_cast<size_t>(pos % pt) * kv + h;
        uint8_t* kr = layer + rec * rb;
        uint8_t* vr = layer + records * rb + rec * rb;
        std::memcpy(kr + hd, &ksb, 2);
        std::memcpy(vr + hd, &vsb, 2);
        for (uint32_t d = 0; d < hd; ++d) {
          kr[d] = static_cast<uint8_t>(static_cast<int8_t>(clamp_rn(k[d] / ks, -127, 127)));
          vr[d] = static_cast<uint8_t>(static_cast<int8_t>(clamp_rn(v[d] / vs, -127, 127)));
        }
      } else {
        const size_t rec = static_cast<size_t>(pos % pt) * kv + h;
        uint8_t* kr = layer + rec * hd * 2U;
        uint8_t* vr = layer + records * hd * 2U + rec * hd * 2U;
        for (uint32_t d = 0; d < hd; ++d) {
          const uint16_t kb = f16_bits(k[d]), vb = f16_bits(v[d]);
          std::memcpy(kr + 2U * d, &kb, 2);
          std::memcpy(vr + 2U * d, &vb, 2);
        }
      }
    }
  }
}

inline int nibble_s4(uint8_t byte, bool high) {
  const int n = high ? (byte >> 4) : (byte & 15);
  return n >= 8 ? n - 16 : n;
}

// Causal GQA attention of `rows` query rows against the paged cache, split
// along the context and merged by log-sum-exp (transformer_kernels.cu:5741-5798).
// The three encodings keep the reference's own approximations:
//   Q4H: INT8 queries, integer QK^T, P*v-scale re-quantised to INT8 per 32 keys
//   Q8 : BF16 queries / keys / values / probabilities, 16-key tiles
//   F16: F16 queries / keys / values, probabilities rounded to F16 per split
void attention(uint32_t enc, const uint8_t* const* pages, size_t layer_offset, uint32_t pt,
               const float* query, uint32_t q_stride, uint32_t rows, uint32_t first_ctx,
               uint32_t qh, uint32_t kvh, uint32_t hd, uint32_t split_tokens, bool bf16,
               float* out) {
  const uint32_t group = qh / kvh;
  const size_t records = static_cast<size_t>(pt) * kvh;
  const uint32_t total = first_ctx + rows - 1U;  // tokens visible to the last row
  const uint32_t splits = (total + split_tokens - 1U) / split_tokens;
  const float inv_sqrt = 1.0F / std::sqrt(static_cast<float>(hd));
  const uint32_t tile = 32U;  // the reference tiles by 32 (Q4H), 16 (Q8) or the split (F16)
  const int64_t items = static_cast<int64_t>(rows) * qh;
#pragma omp parallel for schedule(dynamic)
  for (int64_t item = 0; item < items; ++item) {
    const uint32_t row = static_cast<uint32_t>(item / qh);
    const uint32_t head = static_cast<uint32_t>(item % qh);
    const uint32_t kv = head / group;
    const float* q = query + static_cast<size_t>(row) * q_stride + static_cast<size_t>(head) * hd;
    const uint32_t ctx = first_ctx + row;
    std::vector<float> qf(hd);
    std::vector<int> qi(hd);
    float qscale = 0.0F;
    if (enc == QO_KV_Q4H) {
      float m = 0.0F;
      for (uint32_t d = 0; d < hd; ++d) m = std::fmax(m, std::fabs(q[d]));
      qscale = std::fmax(m / 127.0F, 0x1p-24F);
      for (uint32_t d = 0; d < hd; ++d) qi[d] = clamp_rn(q[d] / qscale, -127, 127);
    } else if (enc == QO_KV_Q8) {
      for (uint32_t d = 0; d < hd; ++d) qf[d] = bf16_round(q[d]);
    } else {
      for (uint32_t d = 0; d < hd; ++d) qf[d] = f16_round(q[d]);
    }
    std::vector<float> pmax(splits, kNegInf), psum(splits, 0.0F);
    std::vector<float> pout(static_cast<size_t>(splits) * hd, 0.0F);
    std::vector<float> score(tile), prob(tile), vsc(tile), acc(hd);
    std::vector<int> pq(tile);
    for (uint32_t s = 0; s < splits; ++s) {
      const uint32_t first = s * split_tokens;
      const uint32_t last = std::min(total, first + split_tokens);
      float m = kNegInf, sum = 0.0F;
      std::fill(acc.begin(), acc.end(), 0.0F);
      for (uint32_t t0 = first; t0 < last; t0 += tile) {
        const uint32_t n = std::min(tile, last - t0);
        float tmax = kNegInf;
        for (uint32_t j = 0; j < n; ++j) {
          const uint32_t tok = t0 + j;
          score[j] = kNegInf;
          vsc[j] = 0.0F;
          const uint8_t* layer = pages[tok / pt] + layer_offset;
          if (enc == QO_KV_Q4H) {
            const size_t rec = static_cast<size_t>(kv) * pt + tok % pt;
            uint16_t sb;
            std::memcpy(&sb, layer + records * (hd / 2U) * 2U + records * 2U + rec * 2U, 2);
            vsc[j] = f16_value(sb);
            if (tok < ctx) {
              const uint8_t* kc = layer + rec * (hd / 2U);
              std::memcpy(&sb, layer + records * (hd / 2U) + rec * 2U, 2);
              int dot = 0;
              for (uint32_t d = 0; d < hd / 2U; ++d)
                dot += qi[2 * d] * nibble_s4(kc[d], false) + qi[2 * d + 1] * nibble_s4(kc[d], true);
              score[j] = static_cast<float>(dot) * qscale * f16_value(sb) * inv_sqrt;
            }
          } else if (tok < ctx) {
            const size_t rec = static_cast<size_t>(tok % pt) * kvh + kv;
            double dot = 0.0;  // products of BF16/F16 values are exact; sum once
            if (enc == QO_KV_Q8) {
              const uint8_t* kr = layer + rec * (hd + 2U);
              uint16_t sb;
              std::memcpy(&sb, kr + hd, 2);
              const float ks = f16_value(sb);
              for (uint32_t d = 0; d < hd; ++d)
                dot += static_cast<double>(qf[d] * bf16_round(static_cast<float>(static_cast<int8_t>(kr[d])) * ks));
            } else {
              const uint8_t* kr = layer + rec * hd * 2U;
              for (uint32_t d = 0; d < hd; ++d) {
                uint16_t kb;
                std::memcpy(&kb, kr + 2U * d, 2);
                dot += static_cast<double>(qf[d] * f16_value(kb));
              }
            }
            score[j] = static_cast<float>(dot) * inv_sqrt;
          }
          tmax = std::fmax(tmax, score[j]);
        }
        const float next = std::fmax(m, tmax);
        const float prev = m == kNegInf ? 0.0F : det_expf(m - next);
        double tsum_d = 0.0;
        for (uint32_t j = 0; j < n; ++j) {
          float p = (t0 + j < ctx) ? det_expf(score[j] - next) : 0.0F;
          if (enc == QO_KV_Q8) p = bf16_round(p);
          else if (enc == QO_KV_F16) p = f16_round(p);
          prob[j] = p;
          tsum_d += static_cast<double>(p);
        }
        const float tsum = static_cast<float>(tsum_d);
        for (uint32_t d = 0; d < hd; ++d) acc[d] *= prev;
        if (enc == QO_KV_Q4H) {
          float wmax = 0.0F;
          for (uint32_t j = 0; j < n; ++j) wmax = std::fmax(wmax, prob[j] * vsc[j]);
          const float pscale = std::fmax(wmax / 127.0F, 0x1p-24F);
          for (uint32_t j = 0; j < n; ++j) pq[j] = clamp_rn(prob[j] * vsc[j] / pscale, 0, 127);
          for (uint32_t d = 0; d < hd; ++d) {
            int dot = 0;
            for (uint32_t j = 0; j < n; ++j) {
              if (pq[j] == 0) continue;
              const uint32_t tok = t0 + j;
              const uint8_t* layer = pages[tok / pt] + layer_offset;
              const size_t rec = static_cast<size_t>(kv) * pt + tok % pt;
              const uint8_t* vc = layer + records * (hd / 2U) + records * 2U + rec * (hd / 2U);
              dot += pq[j] * nibble_s4(vc[d / 2U], d & 1U);
            }
            // one fused multiply-add, as the reference's `results * prev + acc * scale` compiles to
            acc[d] = std::fma(static_cast<float>(dot), pscale, acc[d]);
          }
        } else {
          std::vector<double> tdot(hd, 0.0);
          for (uint32_t j = 0; j < n; ++j) {
            if (prob[j] == 0.0F) continue;
            const uint32_t tok = t0 + j;
            const uint8_t* layer = pages[tok / pt] + layer_offset;
            const size_t rec = static_cast<size_t>(tok % pt) * kvh + kv;
            if (enc == QO_KV_Q8) {
              const uint8_t* vr = layer + records * (hd + 2U) + rec * (hd + 2U);
              uint16_t sb;
              std::memcpy(&sb, vr + hd, 2);
              const float vs = f16_value(sb);
              for (uint32_t d = 0; d < hd; ++d)
                tdot[d] += static_cast<double>(prob[j] * bf16_round(static_cast<float>(static_cast<int8_t>(vr[d])) * vs));
            } else {
              const uint8_t* vr = layer + records * hd * 2U + rec * hd * 2U;
              for (uint32_t d = 0; d < hd; ++d) {
                uint16_t vb;
                std::memcpy(&vb, vr + 2U * d, 2);
                tdot[d] += static_cast<double>(prob[j] * f16_value(vb));
              }
            }
          }
          for (uint32_t d = 0; d < hd; ++d) acc[d] += static_cast<float>(tdot[d]);
        }
        sum = sum * prev + tsum;
        m = next;
      }
      pmax[s] = m;
      psum[s] = sum;
      std::copy(acc.begin(), acc.end(), pout.begin() + static_cast<size_t>(s) * hd);
    }
    const uint32_t active = (ctx + split_tokens - 1U) / split_tokens;
    float gmax = kNegInf;
    for (uint32_t s = 0; s < active; ++s) gmax = std::fmax(gmax, pmax[s]);
    // split terms are FP32 products; their sums are formed in double so that the merge does
    // not depend on the order in which splits are visited
    double gsum_d = 0.0;
    for (uint32_t s = 0; s < active; ++s) gsum_d += static_cast<double>(psum[s] * det_expf(pmax[s] - gmax));
    const float gsum = static_cast<float>(gsum_d);
    float* o = out + (static_cast<size_t>(row) * qh + head) * hd;
    for (uint32_t d = 0; d < hd; ++d) {
      double result = 0.0;
      for (uint32_t s = 0; s < active; ++s)
        result += static_cast<double>(pout[static_cast<size_t>(s) * hd + d] * det_expf(pmax[s] - gmax));
      o[d] = act(static_cast<float>(result) / gsum, bf16);
    }
  }
}

// transformer_kernels.cu:7059-7094: strictly greater wins, ties -> lower index
uint32_t argmax(const float* v, uint32_t count) {
  float best = kNegInf;
  uint32_t index = 0xffffffffU;
  for (uint32_t i = 0; i < count; ++i)
    if (v[i] > best || (v[i] == best && i < index)) { best = v[i]; index = i; }
  return index;
}
// transformer_kernels.cu:7096-7178: k sequential rank passes, NaN excluded
void topk(const float* v, uint32_t count, uint32_t k, float* ov, uint32_t* ot) {
  std::vector<uint32_t> order;
  order.reserve(count);
  for (uint32_t i = 0; i < count; ++i)
    if (!std::isnan(v[i])) order.push_back(i);
  const uint32_t kk = std::min<uint32_t>(k, static_cast<uint32_t>(order.size()));
  std::partial_sort(order.begin(), order.begin() + kk, order.end(),
                    [&](uint32_t a, uint32_t b) { return v[a] == v[b] ? a < b : v[a] > v[b]; });
  for (uint32_t i = 0; i < k; ++i) {
    ov[i] = i < kk ? v[order[i]] : kNegInf;
    ot[i] = i < kk ? order[i] : 0xffffffffU;
  }
}

// ------------------------------------------------------------------ sampler
struct Dist {
  std::vector<uint32_t> tokens;
  std::vector<double> probs;
  double probability(uint32_t t) const {
    for (size_t i = 0; i < tokens.size(); ++i)
      if (tokens[i] == t) return probs[i];
    return 0.0;
  }
};

uint64_t splitmix64(uint64_t v) {
  v += 0x9e3779b97f4a7c15ULL;
  v = (v ^ (v >> 30U)) * 0xbf58476d1ce4e5b9ULL;
  v = (v ^ (v >> 27U)) * 0x94d049bb133111ebULL;
  return v ^ (v >> 31U);
}
// speculative_sampling.cpp:172-182
double counter_uniform(uint64_t seed, uint32_t position, uint32_t stream, uint32_t index) {
  uint64_t c = seed;
  c ^= static_cast<uint64_t>(position) * 0xd2b74407b1ce6e93ULL;
  c ^= static_cast<uint64_t>(stream) * 0xca5a826395121157ULL;
  c ^= static_cast<uint64_t>(index) * 0x9e3779b185ebca87ULL;
  return static_cast<double>(splitmix64(c) >> 11U) * (1.0 / 9007199254740992.0);
}

// speculative_sampling.cpp:52-111
Dist make_distribution(const float* logits, const uint32_t* tokens, uint32_t count,
                       uint32_t temperature_ppm, uint32_t top_p_ppm, uint32_t min_p_ppm) {
  if (!count || temperature_ppm == 0U || temperature_ppm > 2000000U || top_p_ppm == 0U ||
      top_p_ppm > 1000000U || min_p_ppm > 1000000U || !std::isfinite(logits[0]))
    throw std::invalid_argument("invalid sorted sampling candidates");
  for (uint32_t i = 1; i < count; ++i)
    if ((!std::isnan(logits[i]) && logits[i] > logits[i - 1]) ||
        (logits[i] == logits[i - 1] && tokens[i] < tokens[i - 1]))
      throw std::invalid_argument("sampling candidates are not ordered");
  const double inv_t = 1000000.0 / static_cast<double>(temperature_ppm);
  const double maximum = logits[0];
  const double min_rel = static_cast<double>(min_p_ppm) / 1000000.0;
  std::vector<double> w;
  std::vector<uint32_t> t;
  double total = 0.0;
  for (uint32_t i = 0; i < count; ++i) {
    const double l = logits[i];
    const double weight = std::isfinite(l) ? std::exp((l - maximum) * inv_t) : 0.0;
    if (weight < min_rel) continue;
    t.push_back(tokens[i]);
    w.push_back(weight);
    total += weight;
  }
  if (w.empty() || !std::isfinite(total) || !(total > 0.0))
    throw std::invalid_argument("sampling distribution has no retained mass");
  const double top_p = static_cast<double>(top_p_ppm) / 1000000.0;
  double cumulative = 0.0;
  size_t nucleus = w.size();
  for (size_t i = 0; i < w.size(); ++i) {
    cumulative += w[i] / total;
    if (cumulative >= top_p) { nucleus = i + 1; break; }
  }
  w.resize(nucleus);
  t.resize(nucleus);
  total = 0.0;
  for (double x : w) total += x;
  Dist d;
  for (size_t i = 0; i < nucleus; ++i) {
    d.tokens.push_back(t[i]);
    d.probs.push_back(w[i] / total);
  }
  return d;
}

// speculative_sampling.cpp:113-124
uint32_t sample_distribution(const Dist& d, double u) {
  double cumulative = 0.0;
  for (size_t i = 0; i < d.tokens.size(); ++i) {
    cumulative += d.probs[i];
    if (u < cumulative) return d.tokens[i];
  }
  return d.tokens.back();
}

// speculative_sampling.cpp:126-170; residual iterated in ascending token id
bool rejection_sample(uint32_t proposal, const Dist& target, const Dist& draft, double u_accept,
                      double u_correct, uint32_t* token) {
  const double tp = target.probability(proposal);
  const double dp = draft.probability(proposal);
  if (!(dp > 0.0)) throw std::invalid_argument("proposal has zero draft probability");
  if (u_accept < std::min(1.0, tp / dp)) { *token = proposal; return true; }
  std::map<uint32_t, double> residual;
  for (size_t i = 0; i < target.tokens.size(); ++i) residual[target.tokens[i]] = target.probs[i];
  for (size_t i = 0; i < draft.tokens.size(); ++i)
    residual[draft.tokens[i]] = std::max(0.0, residual[draft.tokens[i]] - draft.probs[i]);
  double total = 0.0;
  for (const auto& kv : residual) total += kv.second;
  if (!std::isfinite(total) || !(total > 0.0))
    throw std::runtime_error("rejected proposal has no correction mass");
  const double threshold = u_correct * total;
  double cumulative = 0.0;
  uint32_t last_positive = 0;
  for (const auto& kv : residual) {
    if (kv.second > 0.0) last_positive = kv.first;
    cumulative += kv.second;
    if (threshold < cumulative) { *token = kv.first; return false; }
  }
  *token = last_positive;
  return false;
}

// Router selection of the NVFP4 routed-expert branch (router_select_batch_kernel +
// scale_router_scores_kernel, runtime/src/cuda/transformer_kernels.cu:2947-3016, and the BF16
// rounding of logits and scores in run_router, dense_fp4_provider.cpp:8153-8164): top-K by
// repeated arg-max over the BF16-rounded logits (ties to the lower expert id), softmax over
// the selected values, times the routed scaling factor, rounded to BF16.
void moe_route(const float* logits, uint32_t experts, uint32_t top_k, float route_scale, uint32_t* chosen,
               float* score) {
  float value[8];
  for (uint32_t slot = 0; slot < top_k; ++slot) {
    float best = -INFINITY;
    uint32_t best_index = 0xffffffffU;
    for (uint32_t i = 0; i < experts; ++i) {
      bool used = false;
      for (uint32_t p = 0; p < slot; ++p) used |= chosen[p] == i;
      const float v = bf16_round(logits[i]);
      if (!used && (v > best || (v == best && i < best_index))) { best = v; best_index = i; }
    }
    chosen[slot] = best_index;
    value[slot] = best;
  }
  // exp evaluated in double and rounded once, so that a device and a host evaluation agree
  float top = -INFINITY, sum = 0.0F;
  for (uint32_t slot = 0; slot < top_k; ++slot) top = std::max(top, value[slot]);
  for (uint32_t slot = 0; slot < top_k; ++slot) {
    score[slot] = static_cast<float>(std::exp(static_cast<double>(value[slot] - top)));
    sum += score[slot];
  }
  for (uint32_t slot = 0; slot < top_k; ++slot) {
    score[slot] /= sum;
    if (route_scale != 1.0F) score[slot] *= route_scale;
    score[slot] = bf16_round(score[slot]);
  }
}

}  // namespace

// --------------------------------------------------------------- whole step
struct qo_session {
  qo_config cfg{};
  qo_weights w{};
  uint32_t rows_cap = 8;
  size_t page_bytes = 0;
  std::vector<size_t> layer_off;  // [layers + 1]; last = draft layer
  std::vector<std::vector<uint8_t>> page_store;
  std::vector<uint8_t*> pages;
  std::vector<float> hidden, residual, normalized, qkv, attn, gate_up, inter, logits;
  std::vector<float> mtp_last_hidden, mtp_logits, retained;
  uint32_t last_rows = 0;
  uint32_t mtp_length = 0;
  uint32_t synchronized_token = 0;
  bool draft_valid = false;
  std::vector<uint32_t> draft_tokens;
  std::vector<Dist> draft_dists;
  // sampling presence (dense_fp4_provider.cpp:5168-5171): tokens this request has emitted, and the
  // working copy a verify pass / a rollout advances with its own proposals
  std::vector<uint8_t> emitted, proposal_presence;

  // (biased - 2 000 000) / 1 000 000, dense_fp4_provider.cpp:8336-8341
  static float presence_penalty(const qo_request& rq) {
    if (rq.presence_penalty_biased_ppm > 4000000U) throw std::runtime_error("sampling presence penalty is invalid");
    return static_cast<float>((static_cast<double>(rq.presence_penalty_biased_ppm) - 2000000.0) / 1000000.0);
  }
  // presence_penalty_kernel, runtime/src/cuda/transformer_kernels.cu:7180-7186 (in place)
  static void apply_presence(float* row_logits, uint32_t count, const uint8_t* presence, float penalty) {
    for (uint32_t i = 0; i < count; ++i)
      if (presence[i] != 0U) row_logits[i] -= penalty;
  }

  void ensure_rows(uint32_t rows) {
    const auto& c = cfg;
    hidden.resize(static_cast<size_t>(rows) * c.hidden);
    residual.resize(hidden.size());
    normalized.resize(static_cast<size_t>(rows) * 2U * c.hidden);
    qkv.resize(static_cast<size_t>(rows) * (c.q_heads + 2U * c.kv_heads) * c.head_dim);
    attn.resize(static_cast<size_t>(rows) * c.q_heads * c.head_dim);
    gate_up.resize(static_cast<size_t>(rows) * 2U * c.ffn);
    inter.resize(static_cast<size_t>(rows) * c.ffn);
  }

  void embed(const uint32_t* tokens, uint32_t rows, float* out) const {
    for (uint32_t r = 0; r < rows; ++r)
      for (uint32_t i = 0; i < cfg.hidden; ++i) {
        const uint32_t bits =
            static_cast<uint32_t>(w.embedding[static_cast<size_t>(tokens[r]) * cfg.hidden + i]) << 16U;
        std::memcpy(out + static_cast<size_t>(r) * cfg.hidden + i, &bits, 4);
      }
  }

  // Routed mixture of experts in place of the dense FFN, NVFP4 branch of run_router +
  // run_routed_moe (dense_fp4_provider.cpp:8128-8166, 8207-8248) with the routed-expert
  // arithmetic of moe_kernels.cu:171-264, 430-510, 633-690, 759-790 and the router selection of
  // transformer_kernels.cu:2947-3006; no shared expert.  `normalized` holds the post-attention
  // RMSNorm rows, `residual` the residual stream; the result replaces `hidden`.
  void moe_ffn(const qo_block& b, uint32_t rows) {
    const auto& c = cfg;
    const uint32_t H = c.hidden, E = c.experts, K = c.route_width, W = c.expert_ffn;
    for (size_t i = 0; i < static_cast<size_t>(rows) * H; ++i) normalized[i] = bf16_round(normalized[i]);
    std::vector<float> logits_r(static_cast<size_t>(rows) * E);
    nvfp4_gemv(b.router, 0, E, normalized.data(), rows, logits_r.data());
    std::vector<float> gate(W), up(W), mid(W), out(H), total(H);
    for (uint32_t r = 0; r < rows; ++r) {
      const float* lg = logits_r.data() + static_cast<size_t>(r) * E;
      uint32_t chosen[8];
      float score[8];
      moe_route(lg, E, K, c.route_scale, chosen, score);
      std::fill(total.begin(), total.end(), 0.0F);
      const float* x = normalized.data() + static_cast<size_t>(r) * H;
      for (uint32_t slot = 0; slot < K; ++slot) {
        const uint32_t e = chosen[slot];
        if (e >= E) throw std::runtime_error("router selected no expert");
        // each projection fake-quantises its input with its own activation scale and rounds
        // its dot products to BF16 (nvfp4_dot + bf16 in gate_up_silu_selection_batch)
        nvfp4_gemv(b.expert_gate[e], 0, W, x, 1, gate.data());
        nvfp4_gemv(b.expert_up[e], 0, W, x, 1, up.data());
        for (uint32_t i = 0; i < W; ++i)
          mid[i] = bf16_round((gate[i] / (1.0F + det_expf(-gate[i]))) * up[i]);
        nvfp4_gemv(b.expert_down[e], 0, H, mid.data(), 1, out.data());
        for (uint32_t i = 0; i < H; ++i) total[i] += score[slot] * out[i];  // ordered over the slots
      }
      for (uint32_t i = 0; i < H; ++i) {
        const float moe = bf16_round(total[i]);
        hidden[static_cast<size_t>(r) * H + i] = bf16_round(residual[static_cast<size_t>(r) * H + i] + moe);
      }
    }
  }

  // attention sub-block (run_full_attention + residual add) then FFN (run_ffn)
  void block(const qo_block& b, uint32_t rows, uint32_t enc, size_t layer_offset,
             uint32_t first_cache_position, const uint32_t* rotary_positions) {
    const auto& c = cfg;
    const bool bf = c.activation_bf16 != 0U;
    const uint32_t qw = c.q_heads * c.head_dim, kw = c.kv_heads * c.head_dim;
    const uint32_t width = qw + 2U * kw;
    residual = hidden;
    rmsnorm(hidden.data(), b.input_norm, normalized.data(), rows, c.hidden, c.eps);
    nvfp4_gemv(b.qkv, 0, b.qkv.rows, normalized.data(), rows, qkv.data());
    // q heads and k heads are adjacent in each row: rotate them in one call
    std::vector<float> qk(static_cast<size_t>(rows) * (qw + kw));
    for (uint32_t r = 0; r < rows; ++r)
      std::memcpy(qk.data() + static_cast<size_t>(r) * (qw + kw),
                  qkv.data() + static_cast<size_t>(r) * width, sizeof(float) * (qw + kw));
    rope(qk.data(), rows, c.q_heads + c.kv_heads, c.head_dim, c.rotary_dim, c.rope_theta,
         rotary_positions, bf);
    for (uint32_t r = 0; r < rows; ++r)
      std::memcpy(qkv.data() + static_cast<size_t>(r) * width,
                  qk.data() + static_cast<size_t>(r) * (qw + kw), sizeof(float) * (qw + kw));
    kv_store(enc, pages.data(), layer_offset, c.page_tokens, c.kv_heads, c.head_dim,
             qkv.data() + qw, qkv.data() + qw + kw, rows, width, first_cache_position);
    attention(enc, pages.data(), layer_offset, c.page_tokens, qkv.data(), width, rows,
              first_cache_position + 1U, c.q_heads, c.kv_heads, c.head_dim, c.split_tokens, bf,
              attn.data());
    nvfp4_gemv(b.o, 0, b.o.rows, attn.data(), rows, hidden.data());
    for (size_t i = 0; i < static_cast<size_t>(rows) * c.hidden; ++i)
      hidden[i] = act(hidden[i] + residual[i], bf);
    // FFN
    residual = hidden;
    rmsnorm(hidden.data(), b.post_norm, normalized.data(), rows, c.hidden, c.eps);
    if (c.experts) {
      moe_ffn(b, rows);
      return;
    }
    nvfp4_gemv(b.gate_up, 0, b.gate_up.rows, normalized.data(), rows, gate_up.data());
    for (uint32_t r = 0; r < rows; ++r)
      for (uint32_t i = 0; i < c.ffn; ++i) {
        const float g = gate_up[static_cast<size_t>(r) * 2U * c.ffn + i];
        const float u = gate_up[static_cast<size_t>(r) * 2U * c.ffn + c.ffn + i];
        const float a = act(g / (1.0F + det_expf(-g)), bf);
        inter[static_cast<size_t>(r) * c.ffn + i] = act(a * u, bf);
      }
    nvfp4_gemv(b.down, 0, b.down.rows, inter.data(), rows, hidden.data());
    for (size_t i = 0; i < static_cast<size_t>(rows) * c.hidden; ++i)
      hidden[i] = act(hidden[i] + residual[i], bf);
  }

  // dense_fp4_provider.cpp:8529-8635
  void run_target(const uint32_t* tokens, const uint32_t* positions, uint32_t rows,
                  bool with_head) {
    ensure_rows(rows);
    hidden.resize(static_cast<size_t>(rows) * cfg.hidden);
    embed(tokens, rows, hidden.data());
    for (uint32_t l = 0; l < cfg.layers; ++l)
      block(w.layers[l], rows, cfg.kv_encoding, layer_off[l], positions[0], positions);
    last_rows = rows;
    if (with_head) {
      logits.resize(static_cast<size_t>(rows) * cfg.vocab);
      rmsnorm(hidden.data(), w.final_norm, normalized.data(), rows, cfg.hidden, cfg.eps);
      nvfp4_gemv(w.head, 0, cfg.vocab, normalized.data(), rows, logits.data());
    }
  }

  // dense_fp4_provider.cpp:8331-8391
  Dist distribution(float* row_logits, uint32_t vocabulary, const qo_request& rq,
                    const uint8_t* presence = nullptr) const {
    const float penalty = presence_penalty(rq);
    if (penalty != 0.0F) {
      if (!presence) throw std::runtime_error("sampling presence state is absent");
      apply_presence(row_logits, vocabulary, presence, penalty);
    }
    if (rq.temperature_ppm == 0U) return Dist{{argmax(row_logits, vocabulary)}, {1.0}};
    if (rq.top_k == 0U || rq.top_k > 64U || rq.top_k > vocabulary)
      throw std::runtime_error("sampled exact decode requires bounded nonzero top-k");
    std::vector<float> tv(rq.top_k);
    std::vector<uint32_t> tt(rq.top_k);
    topk(row_logits, vocabulary, rq.top_k, tv.data(), tt.data());
    return make_distribution(tv.data(), tt.data(), rq.top_k, rq.temperature_ppm, rq.top_p_ppm,
                             rq.min_p_ppm);
  }

  // dense_fp4_provider.cpp:8681-8807
  bool run_mtp(const uint32_t* tokens, const float* previous_hidden, const uint32_t* rotary,
               uint32_t rows, bool produce, const qo_request* rq, uint32_t sample_position,
               uint32_t stream, uint32_t* token, Dist* dist) {
    const auto& c = cfg;
    if (!rows || mtp_length + rows > c.max_context) throw std::runtime_error("invalid MTP microbatch");
    for (uint32_t r = 0; r < rows; ++r)
      if (tokens[r] >= c.vocab || rotary[r] != mtp_length + r + 1U)
        throw std::runtime_error("MTP token/position stream is not contiguous");
    std::vector<float> prev(previous_hidden, previous_hidden + static_cast<size_t>(rows) * c.hidden);
    ensure_rows(rows);
    hidden.resize(static_cast<size_t>(rows) * c.hidden);
    std::vector<float> emb(static_cast<size_t>(rows) * c.hidden), fused(static_cast<size_t>(rows) * 2U * c.hidden);
    std::vector<float> en(emb.size()), hn(emb.size());
    embed(tokens, rows, emb.data());
    rmsnorm(emb.data(), w.mtp_embedding_norm, en.data(), rows, c.hidden, c.eps);
    rmsnorm(prev.data(), w.mtp_hidden_norm, hn.data(), rows, c.hidden, c.eps);
    for (uint32_t r = 0; r < rows; ++r) {
      std::memcpy(fused.data() + static_cast<size_t>(r) * 2U * c.hidden,
                  en.data() + static_cast<size_t>(r) * c.hidden, sizeof(float) * c.hidden);
      std::memcpy(fused.data() + static_cast<size_t>(r) * 2U * c.hidden + c.hidden,
                  hn.data() + static_cast<size_t>(r) * c.hidden, sizeof(float) * c.hidden);
    }
    nvfp4_gemv(w.mtp_fusion, 0, c.hidden, fused.data(), rows, hidden.data());
    block(w.mtp_block, rows, c.mtp_kv_encoding, layer_off[c.layers], mtp_length, rotary);
    mtp_length += rows;
    if (!produce) return false;
    const float* final_hidden = hidden.data() + static_cast<size_t>(rows - 1U) * c.hidden;
    mtp_last_hidden.assign(final_hidden, final_hidden + c.hidden);
    std::vector<float> dn(c.hidden);
    rmsnorm(final_hidden, w.mtp_draft_norm, dn.data(), 1, c.hidden, c.eps);
    mtp_logits.resize(c.draft_vocab);
    nvfp4_gemv(w.head, 0, c.draft_vocab, dn.data(), 1, mtp_logits.data());
    if (rq) {
      *dist = distribution(mtp_logits.data(), c.draft_vocab, *rq, proposal_presence.data());
      *token = sample_distribution(*dist, counter_uniform(rq->seed, sample_position, stream, 0));
    } else {
      *token = argmax(mtp_logits.data(), c.draft_vocab);
      *dist = Dist{{*token}, {1.0}};
    }
    return true;
  }

  // dense_fp4_provider.cpp:8809-8852
  void extend_rollout(const qo_request& rq, uint32_t first_token, Dist first_dist) {
    const auto& c = cfg;
    if (c.draft_depth == 0U || rq.context_limit > c.max_context || mtp_length >= rq.context_limit ||
        !(first_dist.probability(first_token) > 0.0))
      throw std::runtime_error("invalid MTP rollout root");
    draft_tokens.clear();
    draft_dists.clear();
    const uint32_t committed = mtp_length;
    if (committed + 1U >= rq.context_limit) throw std::runtime_error("MTP rollout root exceeds context");
    draft_tokens.push_back(first_token);
    draft_dists.push_back(std::move(first_dist));
    proposal_presence[first_token] = 1U;   // mark speculative proposal presence, :8822-8825
    while (draft_tokens.size() < c.draft_depth && mtp_length + 2U < rq.context_limit) {
      const std::vector<float> prev = mtp_last_hidden;
      const uint32_t sample_position = mtp_length;
      const uint32_t token = draft_tokens.back();
      const uint32_t rotary = mtp_length + 1U;
      uint32_t next;
      Dist d;
      run_mtp(&token, prev.data(), &rotary, 1, true, &rq, sample_position,
              1U + static_cast<uint32_t>(draft_tokens.size()), &next, &d);
      draft_tokens.push_back(next);
      draft_dists.push_back(std::move(d));
      proposal_presence[next] = 1U;
    }
    draft_valid = !draft_tokens.empty();
    mtp_length = committed;
  }
};

extern "C" {

const char* qo_last_error(void) { return g_error.c_str(); }
float qo_e2m1_decode(uint8_t c) { return e2m1_decode(c); }
uint8_t qo_e2m1_encode(float v) { return e2m1_encode(v); }
float qo_e4m3_decode(uint8_t c) { return e4m3_decode(c); }
uint8_t qo_e4m3_encode(float v) { return e4m3_encode(v); }
float qo_bf16_round(float v) { return bf16_round(v); }
uint16_t qo_f16_bits(float v) { return f16_bits(v); }
float qo_f16_value(uint16_t b) { return f16_value(b); }

void qo_nvfp4_quantize_weights(const float* w, uint32_t rows, uint32_t cols, float g,
                               uint8_t* codes, uint8_t* scales) {
  nvfp4_quantize_weights(w, rows, cols, g, codes, scales);
}
void qo_nvfp4_dequant(const qo_matrix* m, float* out) {
  for (uint32_t r = 0; r < m->rows; ++r)
    for (uint32_t c = 0; c < m->cols; ++c)
      out[static_cast<size_t>(r) * m->cols + c] = nvfp4_weight(*m, r, c);
}
void qo_nvfp4_fake_quant(const float* x, uint32_t rows, uint32_t cols, float g, float* out) {
  nvfp4_fake_quant(x, rows, cols, g, out);
}
void qo_nvfp4_quantize_activations(const float* x, uint32_t rows, uint32_t cols, float g,
                                   uint8_t* codes, uint8_t* scales) {
  nvfp4_quantize_activations(x, rows, cols, g, codes, scales);
}
void qo_nvfp4_gemv(const qo_matrix* m, uint32_t first_row, uint32_t row_count, const float* x,
                   uint32_t batch, float* y) {
  nvfp4_gemv(*m, first_row, row_count, x, batch, y);
}
void qo_rmsnorm(const float* x, const float* w, float* out, uint32_t rows, uint32_t cols, float eps) {
  rmsnorm(x, w, out, rows, cols, eps);
}
void qo_rope(float* heads, uint32_t rows, uint32_t head_count, uint32_t head_dim,
             uint32_t rotary_dim, float theta, const uint32_t* positions, int bf16) {
  rope(heads, rows, head_count, head_dim, rotary_dim, theta, positions, bf16 != 0);
}
size_t qo_kv_layer_bytes(uint32_t enc, uint32_t pt, uint32_t kv, uint32_t hd) {
  return kv_layer_bytes(enc, pt, kv, hd);
}
void qo_kv_store(uint32_t enc, uint8_t* const* pages, size_t layer_offset, uint32_t pt,
                 uint32_t kv, uint32_t hd, const float* key, const float* value, uint32_t rows,
                 uint32_t row_stride, uint32_t first_pos) {
  kv_store(enc, pages, layer_offset, pt, kv, hd, key, value, rows, row_stride, first_pos);
}
void qo_attention(uint32_t enc, const uint8_t* const* pages, size_t layer_offset, uint32_t pt,
                  const float* query, uint32_t q_stride, uint32_t rows, uint32_t first_ctx,
                  uint32_t qh, uint32_t kvh, uint32_t hd, uint32_t split_tokens, int bf16,
                  float* out) {
  attention(enc, pages, layer_offset, pt, query, q_stride, rows, first_ctx, qh, kvh, hd,
            split_tokens, bf16 != 0, out);
}
uint32_t qo_argmax(const float* v, uint32_t count) { return argmax(v, count); }
void qo_moe_route(const float* logits, uint32_t experts, uint32_t top_k, float route_scale, uint32_t* indices,
                  float* scores) {
  if (top_k <= 8U && top_k <= experts) moe_route(logits, experts, top_k, route_scale, indices, scores);
}
// Host threads the parallel loops (GEMV rows, attention heads) use; for the timed baseline.
void qo_set_threads(uint32_t threads) { omp_set_num_threads(threads ? static_cast<int>(threads) : 1); }
uint32_t qo_max_threads(void) { return static_cast<uint32_t>(omp_get_max_threads()); }
void qo_topk(const float* v, uint32_t count, uint32_t k, float* ov, uint32_t* ot) {
  topk(v, count, k, ov, ot);
}
double qo_counter_uniform(uint64_t seed, uint32_t position, uint32_t stream, uint32_t index) {
  return counter_uniform(seed, position, stream, index);
}
int qo_make_distribution(const float* logits, const uint32_t* tokens, uint32_t count,
                         uint32_t temperature_ppm, uint32_t top_p_ppm, uint32_t min_p_ppm,
                         uint32_t* out_tokens, double* out_probabilities) {
  try {
    const Dist d = make_distribution(logits, tokens, count, temperature_ppm, top_p_ppm, min_p_ppm);
    for (size_t i = 0; i < d.tokens.size(); ++i) {
      out_tokens[i] = d.tokens[i];
      out_probabilities[i] = d.probs[i];
    }
    return static_cast<int>(d.tokens.size());
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}
uint32_t qo_sample_distribution(const uint32_t* tokens, const double* probs, uint32_t count,
                                double u) {
  Dist d{std::vector<uint32_t>(tokens, tokens + count), std::vector<double>(probs, probs + count)};
  return sample_distribution(d, u);
}
// sample_token, runtime/tools/dense_fp4_provider.cpp:771-802 (the scalar decode fallback's sampler
// for top_k == 0 or > 64) with sample_sorted_candidates :748-769.  The reference's comparator leaves
// the order among NaN logits open; here they follow each other by id (their weight is 0 either way).
int qo_sample_token(const float* logits, uint32_t vocabulary, const qo_request* rq, uint32_t position,
                    uint32_t* token) {
  try {
    if (!vocabulary || rq->top_k > vocabulary) throw std::invalid_argument("invalid token sampling contract");
    const size_t candidate_count = rq->top_k == 0U ? vocabulary : rq->top_k;
    std::vector<uint32_t> candidates(vocabulary);
    for (uint32_t i = 0; i < vocabulary; ++i) candidates[i] = i;
    const auto greater_logit = [&](uint32_t left, uint32_t right) {
      const float a = logits[left], b = logits[right];
      if (std::isnan(a) || std::isnan(b)) return std::isnan(a) == std::isnan(b) ? left < right : std::isnan(b);
      return a == b ? left < right : a > b;
    };
    if (candidate_count != candidates.size()) {
      std::partial_sort(candidates.begin(), candidates.begin() + static_cast<long>(candidate_count), candidates.end(),
                        greater_logit);
      candidates.resize(candidate_count);
    } else {
      std::sort(candidates.begin(), candidates.end(), greater_logit);
    }
    std::vector<float> sorted(candidates.size());
    for (size_t i = 0; i < candidates.size(); ++i) sorted[i] = logits[candidates[i]];
    const Dist d = make_distribution(sorted.data(), candidates.data(), static_cast<uint32_t>(candidates.size()),
                                     rq->temperature_ppm, rq->top_p_ppm, rq->min_p_ppm);
    *token = sample_distribution(d, counter_uniform(rq->seed, position, 0U, 0U));
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}
int qo_rejection_sample(uint32_t proposal, const uint32_t* tt, const double* tp, uint32_t tc,
                        const uint32_t* dt, const double* dp, uint32_t dc, double ua, double uc,
                        uint32_t* token) {
  try {
    Dist t{std::vector<uint32_t>(tt, tt + tc), std::vector<double>(tp, tp + tc)};
    Dist d{std::vector<uint32_t>(dt, dt + dc), std::vector<double>(dp, dp + dc)};
    return rejection_sample(proposal, t, d, ua, uc, token) ? 1 : 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

qo_session* qo_session_create(const qo_config* config, const qo_weights* weights) {
  try {
    const auto& c = *config;
    if (!c.layers || !c.hidden || !c.kv_heads || c.q_heads % c.kv_heads || c.head_dim % 32U ||
        c.hidden % 16U || c.ffn % 16U || !c.page_tokens || c.page_tokens % 32U ||
        c.draft_depth > 4U || !c.split_tokens || c.split_tokens % 32U || c.draft_vocab > c.vocab)
      throw std::runtime_error("invalid oracle configuration");
    if (c.experts && (!c.route_width || c.route_width > 8U || c.route_width > c.experts || !c.expert_ffn ||
                      c.expert_ffn % 16U || !(c.route_scale > 0.0F)))
      throw std::runtime_error("invalid routed-expert configuration");
    auto* s = new qo_session;
    s->cfg = c;
    s->w = *weights;
    size_t off = 0;
    for (uint32_t l = 0; l < c.layers; ++l) {
      s->layer_off.push_back(off);
      off += kv_layer_bytes(c.kv_encoding, c.page_tokens, c.kv_heads, c.head_dim);
    }
    s->layer_off.push_back(off);
    off += kv_layer_bytes(c.mtp_kv_encoding, c.page_tokens, c.kv_heads, c.head_dim);
    s->page_bytes = off;
    const uint32_t count = (c.max_context + c.page_tokens - 1U) / c.page_tokens;
    s->page_store.resize(count);
    for (auto& p : s->page_store) {
      p.assign(off, 0);
      s->pages.push_back(p.data());
    }
    return s;
  } catch (const std::exception& e) {
    g_error = e.what();
    return nullptr;
  }
}
void qo_session_destroy(qo_session* s) { delete s; }

namespace {
uint32_t hash32(uint64_t x) {
  x ^= x >> 33U; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33U; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33U;
  return static_cast<uint32_t>(x);
}
}  // namespace

// Seeded synthetic cache records for positions [first, first + count) of every layer (target
// layers, then the draft layer): the host twin of the CUDA library's synthetic cache fill, so
// that long contexts need no prompt pass on either side.  Same bytes: a record's scale is
// f16(0.1 + 0.2 u) with u from a 64-bit mix of (seed, position, kv head, K|V), its codes are
// uniform over the encoding's range.  The cached prefix then ends at first + count.
int qo_fill_synthetic_kv(qo_session* s, uint32_t first, uint32_t count, uint64_t seed) {
  try {
    const auto& c = s->cfg;
    if (first != s->mtp_length || first + count > c.max_context)
      throw std::runtime_error("synthetic cache fill must extend the cached prefix");
    const uint32_t pt = c.page_tokens, kv = c.kv_heads, hd = c.head_dim;
    const size_t records = static_cast<size_t>(pt) * kv;
    for (uint32_t l = 0; l <= c.layers; ++l) {
      const uint32_t enc = l < c.layers ? c.kv_encoding : c.mtp_kv_encoding;
      const uint64_t layer_seed = seed + 0x9e3779b97f4a7c15ULL * (l + 1U);
#pragma omp parallel for schedule(static)
      for (int64_t item = 0; item < static_cast<int64_t>(count) * kv * 2; ++item) {
        const uint32_t which = static_cast<uint32_t>(item & 1);
        const uint32_t h = static_cast<uint32_t>((item >> 1) % kv);
        const uint32_t pos = first + static_cast<uint32_t>((item >> 1) / kv);
        uint8_t* layer = s->pages[pos / pt] + s->layer_off[l];
        const uint32_t slot = pos % pt;
        const uint64_t key = layer_seed ^ (static_cast<uint64_t>(pos) << 20U) ^ (static_cast<uint64_t>(h) << 4U) ^ which;
        const uint16_t scale = f16_bits(0.1F + 0.2F * static_cast<float>(hash32(key) & 0xffffU) / 65536.0F);
        if (enc == QO_KV_Q4H) {
          const size_t rec = static_cast<size_t>(h) * pt + slot;
          uint8_t* codes = layer + (which ? records * (hd / 2U) + records * 2U : 0U) + rec * (hd / 2U);
          uint8_t* sc = layer + records * (hd / 2U) + (which ? records * (hd / 2U) + records * 2U : 0U);
          std::memcpy(sc + rec * 2U, &scale, 2);
          for (uint32_t d = 0; d < hd / 2U; ++d) {
            const uint32_t r = hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U);
            const int lo = static_cast<int>(r % 15U) - 7, hi = static_cast<int>((r >> 8U) % 15U) - 7;
            codes[d] = static_cast<uint8_t>((lo & 15) | ((hi & 15) << 4));
          }
        } else if (enc == QO_KV_Q8) {
          const size_t rec = static_cast<size_t>(slot) * kv + h;
          uint8_t* r8 = layer + (which ? records * (hd + 2U) : 0U) + rec * (hd + 2U);
          const uint16_t small = f16_bits(f16_value(scale) / 16.0F);
          std::memcpy(r8 + hd, &small, 2);
          for (uint32_t d = 0; d < hd; ++d)
            r8[d] = static_cast<uint8_t>(static_cast<int8_t>(
                static_cast<int>(hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U) % 255U) - 127));
        } else {
          const size_t rec = static_cast<size_t>(slot) * kv + h;
          uint8_t* r16 = layer + (which ? records * hd * 2U : 0U) + rec * hd * 2U;
          for (uint32_t d = 0; d < hd; ++d) {
            const uint16_t bits = f16_bits(
                (static_cast<float>(hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U) & 0xffffU) / 32768.0F - 1.0F) * 1.4F);
            std::memcpy(r16 + 2U * d, &bits, 2);
          }
        }
      }
    }
    s->mtp_length = first + count;
    s->draft_valid = false;
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

int qo_prefill(qo_session* s, const uint32_t* tokens, uint32_t count, uint32_t chunk_rows,
               const qo_request* rq, uint32_t* first_token) {
  s->mtp_length = 0;
  return qo_prefill_at(s, tokens, count, 0U, chunk_rows, rq, first_token);
}

// The prompt tokens of positions [base, base + count) behind a cached prefix of `base` positions.
int qo_prefill_at(qo_session* s, const uint32_t* tokens, uint32_t count, uint32_t base, uint32_t chunk_rows,
                  const qo_request* rq, uint32_t* first_token) {
  try {
    const auto& c = s->cfg;
    (void)qo_session::presence_penalty(*rq);   // validates the field
    if (s->emitted.size() != c.vocab) {
      s->emitted.assign(c.vocab, 0U);
      s->proposal_presence.assign(c.vocab, 0U);
    }
    if (!count || !chunk_rows || base + count + 1U >= rq->context_limit || rq->context_limit > c.max_context ||
        s->mtp_length != base)
      throw std::runtime_error("invalid prefill request");
    s->draft_valid = false;
    tokens -= base;  // indexed by absolute position below
    count += base;
    for (uint32_t first = base; first < count; first += chunk_rows) {
      const uint32_t rows = std::min(chunk_rows, count - first);
      const bool last = first + rows == count;
      std::vector<uint32_t> positions(rows), next(rows), rotary(rows);
      for (uint32_t r = 0; r < rows; ++r) positions[r] = first + r;
      s->run_target(tokens + first, positions.data(), rows, last);
      if (last) {
        // first output token: scalar head branch (dense_fp4_provider.cpp:8453-8480),
        // uniform stream 0 at the last prompt position
        // the penalty and the emitted mark apply to output positions only (:8440-8453, :8514-8516)
        float* row_logits = s->logits.data() + static_cast<size_t>(rows - 1U) * c.vocab;
        const bool output_sampling = count - 1U >= rq->first_output_position;
        qo_request head_request = *rq;
        if (!output_sampling) head_request.presence_penalty_biased_ppm = 2000000U;
        const Dist d = s->distribution(row_logits, c.vocab, head_request, s->emitted.data());
        *first_token = rq->temperature_ppm == 0U
                           ? d.tokens[0]
                           : sample_distribution(d, counter_uniform(rq->seed, count - 1U, 0, 0));
        if (output_sampling) s->emitted[*first_token] = 1U;
      }
      // synchronize_exact_decode_batch (dense_fp4_provider.cpp:11011-11137)
      if (s->mtp_length != first) throw std::runtime_error("MTP synchronization stream is invalid");
      for (uint32_t r = 0; r < rows; ++r) {
        next[r] = first + r + 1U < count ? tokens[first + r + 1U] : *first_token;
        rotary[r] = first + r + 1U;
      }
      s->synchronized_token = next.back();
      const std::vector<float> target_hidden = s->hidden;
      uint32_t token = 0;
      Dist d;
      if (last) s->proposal_presence = s->emitted;   // initialize speculative proposal presence, :11091-11098
      const bool produced = s->run_mtp(next.data(), target_hidden.data(), rotary.data(), rows,
                                       last, last ? rq : nullptr, first + rows, 1U, &token, &d);
      if (last) {
        if (!produced) throw std::runtime_error("MTP synchronization produced no draft");
        s->extend_rollout(*rq, token, std::move(d));
      }
    }
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

// dense_fp4_provider.cpp:11139-11318 (ABI-2 multi-draft branch)
int qo_execute_exact_decode(qo_session* s, const qo_request* rq, uint32_t guaranteed_token,
                            uint32_t position, qo_step_result* result) {
  try {
    const auto& c = s->cfg;
    if (!s->draft_valid || guaranteed_token != s->synchronized_token ||
        position != s->mtp_length || position + 1U >= rq->context_limit ||
        rq->context_limit > c.max_context)
      throw std::runtime_error("exact MTP invocation stream is invalid");
    const uint32_t proposals = static_cast<uint32_t>(s->draft_tokens.size());
    if (!proposals || proposals > c.draft_depth || position + proposals >= rq->context_limit)
      throw std::runtime_error("multi-draft MTP state is invalid");
    std::vector<uint32_t> tt{guaranteed_token}, tp{position};
    for (uint32_t i = 0; i < proposals; ++i) {
      tt.push_back(s->draft_tokens[i]);
      tp.push_back(position + i + 1U);
    }
    s->run_target(tt.data(), tp.data(), proposals + 1U, true);
    if (s->emitted.size() != c.vocab) {
      s->emitted.assign(c.vocab, 0U);
      s->proposal_presence.assign(c.vocab, 0U);
    }
    // row r is judged against what was emitted plus the proposals before it, :11182-11202
    s->proposal_presence = s->emitted;
    std::vector<Dist> target;
    for (uint32_t r = 0; r <= proposals; ++r) {
      target.push_back(s->distribution(s->logits.data() + static_cast<size_t>(r) * c.vocab, c.vocab, *rq,
                                       s->proposal_presence.data()));
      if (r < proposals) s->proposal_presence[s->draft_tokens[r]] = 1U;
    }
    uint32_t accepted = 0, next_token = 0;
    bool rejected = false;
    for (; accepted < proposals; ++accepted) {
      uint32_t token;
      const bool ok = rejection_sample(
          s->draft_tokens[accepted], target[accepted], s->draft_dists[accepted],
          counter_uniform(rq->seed, position + accepted, 100U, accepted),
          counter_uniform(rq->seed, position + accepted, 200U, accepted), &token);
      if (!ok) { next_token = token; rejected = true; break; }
    }
    if (!rejected)
      next_token = sample_distribution(target.back(),
                                       counter_uniform(rq->seed, position + accepted, 300U, 0));
    // commit accepted proposal presence and the sampled next token, :11261-11270
    for (uint32_t i = 0; i < accepted; ++i) s->emitted[s->draft_tokens[i]] = 1U;
    s->emitted[next_token] = 1U;
    std::vector<uint32_t> mt, mp;
    for (uint32_t i = 0; i < accepted; ++i) mt.push_back(s->draft_tokens[i]);
    mt.push_back(next_token);
    for (uint32_t i = 0; i < mt.size(); ++i) mp.push_back(position + i + 1U);
    const uint32_t advanced = accepted + 1U;
    const bool future = position + advanced + 1U < rq->context_limit;
    std::memset(result, 0, sizeof(*result));
    result->emitted[0] = guaranteed_token;
    for (uint32_t i = 0; i < accepted; ++i) result->emitted[i + 1U] = s->draft_tokens[i];
    result->emitted_count = advanced;
    result->next_token = next_token;
    result->positions_advanced = advanced;
    result->rejected = rejected ? 1U : 0U;
    s->mtp_length = position;
    s->draft_valid = false;
    s->draft_tokens.clear();
    s->draft_dists.clear();
    const std::vector<float> target_hidden = s->hidden;
    uint32_t token = 0;
    Dist d;
    s->proposal_presence = s->emitted;   // initialize next MTP rollout presence, :11290-11292
    const bool produced =
        s->run_mtp(mt.data(), target_hidden.data(), mp.data(), advanced, future,
                   future ? rq : nullptr, position + advanced, 1U, &token, &d);
    // keep the verify rows visible to the parity tests after the draft passes
    s->hidden = target_hidden;
    if (future) {
      if (!produced) throw std::runtime_error("next MTP rollout produced no root");
      s->extend_rollout(*rq, token, std::move(d));
    }
    s->hidden = target_hidden;
    s->last_rows = proposals + 1U;
    s->synchronized_token = next_token;
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  }
}

uint32_t qo_draft_count(const qo_session* s) { return static_cast<uint32_t>(s->draft_tokens.size()); }
void qo_drafts(const qo_session* s, uint32_t* tokens) {
  std::copy(s->draft_tokens.begin(), s->draft_tokens.end(), tokens);
}
const float* qo_last_logits(const qo_session* s) { return s->logits.data(); }
const float* qo_last_hidden(const qo_session* s) { return s->hidden.data(); }
size_t qo_page_bytes(const qo_session* s) { return s->page_bytes; }
uint32_t qo_page_count(const qo_session* s) { return static_cast<uint32_t>(s->pages.size()); }
const uint8_t* qo_page(const qo_session* s, uint32_t i) { return s->pages[i]; }
size_t qo_layer_offset(const qo_session* s, uint32_t l) { return s->layer_off[l]; }
uint32_t qo_mtp_length(const qo_session* s) { return s->mtp_length; }

}  // extern "C"
