// RoPE + K/V record store, split flash-decode attention over the paged cache with
// the dequantisation fused into the kernel, and the split combine.
//
// Page layout per layer (byte-identical to the reference's records,
// runtime/src/cuda/transformer_kernels.cu:229-288, 560-625, 4208-4230):
//   Q4H: [K codes kv*pt*hd/2][K scales f16 kv*pt][V codes][V scales], record = kv_head*pt + pos%pt
//   Q8 : [K records pt*kv*(hd+2)][V records], record = (pos%pt)*kv + kv_head, int8[hd] + f16 scale
//   F16: [K pt*kv*hd f16][V ...], token-major
#include "common.cuh"
#include "fused.h"
#include "kernels.h"
#include "launch.cuh"

namespace qllm {

size_t kv_layer_bytes(uint32_t enc, uint32_t pt, uint32_t kv, uint32_t hd) {
  const size_t records = static_cast<size_t>(pt) * kv;
  switch (enc) {
    case QLLM_KV_F16: return records * hd * 2U * 2U;
    case QLLM_KV_Q4H: return records * (hd / 2U + 2U) * 2U;
    case QLLM_KV_Q8: return records * (hd + 2U) * 2U;
  }
  return 0;
}

__device__ __forceinline__ float block_max_small(float v, float* scratch) {
  // blockDim.x <= 256, all threads participate
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31U) == 0U) scratch[threadIdx.x >> 5U] = v;
  __syncthreads();
  float r = scratch[0];
  for (uint32_t w = 1; w < (blockDim.x + 31U) / 32U; ++w) r = fmaxf(r, scratch[w]);
  return r;
}

// grid (q_heads + kv_heads, rows), block head_dim threads.
// With `fused` the projections are read from the GEMV result `src` (final values or split-K
// partials) and the rotated queries are written to q_out [rows, q_heads*head_dim].
__global__ void rope_kv_store_kernel(RopeStoreArgs a, GemvOut src_out, float* q_out, bool fused,
                                     int8_t* q8_out, float* q8_scale) {
  __shared__ float src[256];
  pdl_trigger();  // the attention kernel may be scheduled; it waits for this grid before reading
  pdl_wait();
  __shared__ float scratch[8];
  const uint32_t head = blockIdx.x, row = blockIdx.y, d = threadIdx.x;
  const uint32_t hd = a.head_dim;
  const uint32_t width = (a.q_heads + 2U * a.kv_heads) * hd;
  const uint32_t cache_position = *a.first_position + a.position_offset + row;
  const uint32_t rotary_position = cache_position + a.rotary_offset;
  float* v = fused ? (head < a.q_heads ? q_out + (static_cast<size_t>(row) * a.q_heads + head) * hd : nullptr)
                   : a.qkv + static_cast<size_t>(row) * width + static_cast<size_t>(head) * hd;
  src[d] = actv(fused ? gemv_value(src_out, row, head * hd + d) : v[d], a.bf16);
  __syncthreads();
  float result = src[d];
  if (d < a.rotary_dim) {
    const uint32_t half = a.rotary_dim / 2U;
    const uint32_t pair = d % half;
    const float angle = static_cast<float>(rotary_position) * a.inv_freq[pair];
    const float other = d < half ? -src[d + half] : src[d - half];
    float sine, cosine;
    if (a.exact) det_sincosf(angle, &sine, &cosine);
    else { sine = sinf(angle); cosine = cosf(angle); }
    result = src[d] * actv(cosine, a.bf16) + other * actv(sine, a.bf16);
  }
  result = actv(result, a.bf16);
  if (v) v[d] = result;
  if (head < a.q_heads) {
    if (q8_out) {  // uniform per block
      const float qmax = block_max_small(fabsf(result), scratch);
      const float qsc = fmaxf(qmax / 127.0F, 0x1p-24F);
      const size_t item = static_cast<size_t>(row) * a.q_heads + head;
      q8_out[item * hd + d] = static_cast<int8_t>(max(-127, min(127, __float2int_rn(result / qsc))));
      if (d == 0U) q8_scale[item] = qsc;
    }
    return;
  }

  // K head: quantise and store the K record and the V record of the same kv head
  const uint32_t kvh = head - a.q_heads;
  const float key = result;
  const float value = fused ? gemv_value(src_out, row, (a.q_heads + a.kv_heads + kvh) * hd + d)
                            : a.qkv[static_cast<size_t>(row) * width +
                                    static_cast<size_t>(a.q_heads + a.kv_heads + kvh) * hd + d];
  const uint32_t pt = a.page_tokens;
  uint8_t* layer = a.page_table[cache_position / pt] + a.layer_offset;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  const uint32_t slot = cache_position % pt;
  if (a.encoding == QLLM_KV_F16) {
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    reinterpret_cast<__half*>(layer)[rec * hd + d] = __float2half_rn(key);
    reinterpret_cast<__half*>(layer + records * hd * 2U)[rec * hd + d] = __float2half_rn(value);
    return;
  }
  const float kmax = block_max_small(fabsf(key), scratch);
  const float vmax = block_max_small(fabsf(value), scratch);
  // the pair partner's values travel through shared memory
  __shared__ float kbuf[256], vbuf[256];
  kbuf[d] = key;
  vbuf[d] = value;
  __syncthreads();
  if (a.encoding == QLLM_KV_Q4H) {
    const __half ksh = __float2half_rn(fmaxf(kmax / 7.0F, 0x1p-24F));
    const __half vsh = __float2half_rn(fmaxf(vmax / 7.0F, 0x1p-24F));
    const float ks = __half2float(ksh), vs = __half2float(vsh);
    uint8_t* kc = layer;
    uint8_t* ksc = kc + records * (hd / 2U);
    uint8_t* vc = ksc + records * 2U;
    uint8_t* vsc = vc + records * (hd / 2U);
    const size_t rec = static_cast<size_t>(kvh) * pt + slot;
    if (d == 0U) {
      reinterpret_cast<__half*>(ksc)[rec] = ksh;
      reinterpret_cast<__half*>(vsc)[rec] = vsh;
    }
    if (d < hd / 2U) {
      const int kl = max(-7, min(7, __float2int_rn(kbuf[2U * d] / ks)));
      const int kh = max(-7, min(7, __float2int_rn(kbuf[2U * d + 1U] / ks)));
      const int vl = max(-7, min(7, __float2int_rn(vbuf[2U * d] / vs)));
      const int vh = max(-7, min(7, __float2int_rn(vbuf[2U * d + 1U] / vs)));
      kc[rec * (hd / 2U) + d] = static_cast<uint8_t>((kl & 15) | ((kh & 15) << 4));
      vc[rec * (hd / 2U) + d] = static_cast<uint8_t>((vl & 15) | ((vh & 15) << 4));
    }
  } else {  // Q8
    const __half ksh = __float2half_rn(fmaxf(kmax / 127.0F, 0x1p-24F));
    const __half vsh = __float2half_rn(fmaxf(vmax / 127.0F, 0x1p-24F));
    const float ks = __half2float(ksh), vs = __half2float(vsh);
    const size_t rb = hd + 2U;
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    uint8_t* kr = layer + rec * rb;
    uint8_t* vr = layer + records * rb + rec * rb;
    if (d == 0U) {
      *reinterpret_cast<__half*>(kr + hd) = ksh;
      *reinterpret_cast<__half*>(vr + hd) = vsh;
    }
    kr[d] = static_cast<uint8_t>(static_cast<int8_t>(max(-127, min(127, __float2int_rn(key / ks)))));
    vr[d] = static_cast<uint8_t>(static_cast<int8_t>(max(-127, min(127, __float2int_rn(value / vs)))));
  }
}

// head_dim 128, fused form: one warp per (head, row), a lane owns 4 consecutive dims, every
// reduction is a warp shuffle (no shared memory, no block barrier) and the rotation partner
// d +- rotary_dim/2 lives in another lane at the same element index.  Same arithmetic as
// rope_kv_store_kernel.  grid = ceil(heads*rows / 4), block = 128 (4 warps).
__global__ void __launch_bounds__(128)
rope_kv_store_warp128_kernel(RopeStoreArgs a, GemvOut src_out, float* q_out, int8_t* q8_out, float* q8_scale) {
  pdl_trigger();  // the attention kernel may be scheduled; it waits for this grid before reading
  pdl_wait();
  constexpr uint32_t hd = 128;
  const uint32_t lane = threadIdx.x & 31U;
  const uint32_t item = blockIdx.x * 4U + (threadIdx.x >> 5U);
  const uint32_t heads = a.q_heads + a.kv_heads;
  if (item >= heads * a.rows) return;
  const uint32_t head = item % heads, row = item / heads;
  const uint32_t cache_position = *a.first_position + a.position_offset + row;
  const uint32_t rotary_position = cache_position + a.rotary_offset;
  const uint32_t d0 = 4U * lane, half = a.rotary_dim / 2U;
  const float4 s4 = gemv_value4(src_out, row, head * hd + d0);
  const float src[4] = {actv(s4.x, a.bf16), actv(s4.y, a.bf16), actv(s4.z, a.bf16), actv(s4.w, a.bf16)};
  const bool rotated = d0 < a.rotary_dim;      // rotary_dim % 8 == 0: a lane is inside or outside
  const bool low = d0 < half;
  const uint32_t partner = rotated ? (low ? lane + half / 4U : lane - half / 4U) : lane;
  float result[4];
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
  if (head < a.q_heads) {
    const size_t item_q = static_cast<size_t>(row) * a.q_heads + head;
    *reinterpret_cast<float4*>(q_out + item_q * hd + d0) = make_float4(result[0], result[1], result[2], result[3]);
    if (q8_out) {
      const float qmax = warp_max(fmaxf(fmaxf(fabsf(result[0]), fabsf(result[1])), fmaxf(fabsf(result[2]), fabsf(result[3]))));
      const float qsc = fmaxf(qmax / 127.0F, 0x1p-24F);
      uint32_t packed = 0U;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        packed |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(result[i] / qsc)))) & 0xffU) << (8 * i);
      *reinterpret_cast<uint32_t*>(q8_out + item_q * hd + d0) = packed;
      if (lane == 0U) q8_scale[item_q] = qsc;
    }
    return;
  }
  // K head: quantise and store the K record and the V record of the same kv head
  const uint32_t kvh = head - a.q_heads;
  const float4 v4 = gemv_value4(src_out, row, (a.q_heads + a.kv_heads + kvh) * hd + d0);
  const float value[4] = {v4.x, v4.y, v4.z, v4.w};
  const uint32_t pt = a.page_tokens;
  uint8_t* layer = a.page_table[cache_position / pt] + a.layer_offset;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  const uint32_t slot = cache_position % pt;
  if (a.encoding == QLLM_KV_F16) {
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    __half* kdst = reinterpret_cast<__half*>(layer) + rec * hd + d0;
    __half* vdst = reinterpret_cast<__half*>(layer + records * hd * 2U) + rec * hd + d0;
#pragma unroll
    for (int i = 0; i < 4; ++i) { kdst[i] = __float2half_rn(result[i]); vdst[i] = __float2half_rn(value[i]); }
    return;
  }
  const float kmax = warp_max(fmaxf(fmaxf(fabsf(result[0]), fabsf(result[1])), fmaxf(fabsf(result[2]), fabsf(result[3]))));
  const float vmax = warp_max(fmaxf(fmaxf(fabsf(value[0]), fabsf(value[1])), fmaxf(fabsf(value[2]), fabsf(value[3]))));
  if (a.encoding == QLLM_KV_Q4H) {
    const __half ksh = __float2half_rn(fmaxf(kmax / 7.0F, 0x1p-24F));
    const __half vsh = __float2half_rn(fmaxf(vmax / 7.0F, 0x1p-24F));
    const float ks = __half2float(ksh), vs = __half2float(vsh);
    uint8_t* kc = layer;
    uint8_t* ksc = kc + records * (hd / 2U);
    uint8_t* vc = ksc + records * 2U;
    uint8_t* vsc = vc + records * (hd / 2U);
    const size_t rec = static_cast<size_t>(kvh) * pt + slot;
    if (lane == 0U) {
      reinterpret_cast<__half*>(ksc)[rec] = ksh;
      reinterpret_cast<__half*>(vsc)[rec] = vsh;
    }
    uint32_t kb = 0U, vb = 0U;  // two bytes each: dims (d0, d0+1) and (d0+2, d0+3)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int kq = max(-7, min(7, __float2int_rn(result[i] / ks)));
      const int vq = max(-7, min(7, __float2int_rn(value[i] / vs)));
      kb |= (static_cast<uint32_t>(kq) & 15U) << (4 * i);
      vb |= (static_cast<uint32_t>(vq) & 15U) << (4 * i);
    }
    reinterpret_cast<uint16_t*>(kc + rec * (hd / 2U))[lane] = static_cast<uint16_t>(kb);
    reinterpret_cast<uint16_t*>(vc + rec * (hd / 2U))[lane] = static_cast<uint16_t>(vb);
  } else {  // Q8: records are 2-byte aligned
    const __half ksh = __float2half_rn(fmaxf(kmax / 127.0F, 0x1p-24F));
    const __half vsh = __float2half_rn(fmaxf(vmax / 127.0F, 0x1p-24F));
    const float ks = __half2float(ksh), vs = __half2float(vsh);
    const size_t rb = hd + 2U;
    const size_t rec = static_cast<size_t>(slot) * a.kv_heads + kvh;
    uint8_t* kr = layer + rec * rb;
    uint8_t* vr = layer + records * rb + rec * rb;
    if (lane == 0U) {
      *reinterpret_cast<__half*>(kr + hd) = ksh;
      *reinterpret_cast<__half*>(vr + hd) = vsh;
    }
    uint32_t kb = 0U, vb = 0U;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      kb |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(result[i] / ks)))) & 0xffU) << (8 * i);
      vb |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(value[i] / vs)))) & 0xffU) << (8 * i);
    }
    reinterpret_cast<uint16_t*>(kr)[2U * lane] = static_cast<uint16_t>(kb & 0xffffU);
    reinterpret_cast<uint16_t*>(kr)[2U * lane + 1U] = static_cast<uint16_t>(kb >> 16U);
    reinterpret_cast<uint16_t*>(vr)[2U * lane] = static_cast<uint16_t>(vb & 0xffffU);
    reinterpret_cast<uint16_t*>(vr)[2U * lane + 1U] = static_cast<uint16_t>(vb >> 16U);
  }
}

int launch_rope_kv_store(const RopeStoreArgs& a, cudaStream_t stream) {
  if (a.head_dim > 256U || a.head_dim % 32U || a.rotary_dim > a.head_dim || a.rotary_dim % 2U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported head geometry for RoPE/KV store");
  rope_kv_store_kernel<<<dim3(a.q_heads + a.kv_heads, a.rows), a.head_dim, 0, stream>>>(a, GemvOut{}, nullptr, false,
                                                                                             nullptr, nullptr);
  count_launch();
  return check_launch("rope_kv_store");
}

int launch_rope_kv_store_fused(const RopeStoreFusedArgs& f, cudaStream_t stream) {
  const RopeStoreArgs& a = f.base;
  if (a.head_dim > 256U || a.head_dim % 32U || a.rotary_dim > a.head_dim || a.rotary_dim % 2U || !f.q_out)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported head geometry for RoPE/KV store");
  count_launch();
  if (a.head_dim == 128U && a.rotary_dim % 8U == 0U && f.qkv.n % 4U == 0U) {
    const uint32_t items = (a.q_heads + a.kv_heads) * a.rows;
    return check_cuda(launch_pdl(rope_kv_store_warp128_kernel, dim3((items + 3U) / 4U), dim3(128), 0, stream, a, f.qkv,
                                 f.q_out, f.q8_out, f.q8_scale), "rope_kv_store");
  }
  return check_cuda(launch_pdl(rope_kv_store_kernel, dim3(a.q_heads + a.kv_heads, a.rows), dim3(a.head_dim), 0, stream,
                               a, f.qkv, f.q_out, true, f.q8_out, f.q8_scale), "rope_kv_store");
}

// ------------------------------------------------------------------ partials
struct Partials {
  float* maxima;   // [rows, max_splits, q_heads]
  float* sums;     // same
  float* outputs;  // [rows, max_splits, q_heads, head_dim]
};
size_t attention_workspace_bytes(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                                 uint32_t max_splits) {
  const size_t items = attention_partial_items(rows, max_splits, q_heads);
  // partials, then room for INT8 queries made on the fly (tensor-memory kernel without ready-made ones)
  return ((items * (2U + head_dim) * sizeof(float) + 255U) & ~static_cast<size_t>(255U)) +
         attention_q4h_tc_query_bytes(rows, q_heads);
}
static Partials partials_of(const AttentionArgs& a) {
  const size_t items = attention_partial_items(a.rows, a.max_splits, a.q_heads);
  float* base = static_cast<float*>(a.workspace);
  return {base, base + items, base + 2U * items};
}

// ------------------------------------------------- scalar attention (all encodings)
// CTA = (kv head, split), 256 threads, 32-key tiles staged in shared memory.
// Dynamic shared memory: q[MR][hd] | tile[32][hd+1] | S[MR][33] | P[MR][33] | stats.
// Decodes the K (or V) records of up to 32 tokens into tile[j][d] (FP32, row stride hd+1).
// 256 threads: thread = (token j, eighth of the head); every thread resolves its page and
// record once and then issues independent vector loads.
template <uint32_t ENC>
__device__ __forceinline__ void load_kv_tile(const AttentionArgs& a, uint32_t kvh, uint32_t t0, uint32_t n,
                                             bool is_value, float* tile) {
  const uint32_t hd = a.head_dim, pt = a.page_tokens;
  const uint32_t j = threadIdx.x >> 3U, part = threadIdx.x & 7U;
  const uint32_t dpp = hd / 8U, d0 = part * dpp;  // dims per thread (multiple of 8)
  float* out = tile + j * (hd + 1U) + d0;
  if (j >= n) {
    for (uint32_t e = 0; e < dpp; ++e) out[e] = 0.0F;
    return;
  }
  const uint32_t tok = t0 + j;
  const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  if (ENC == QLLM_KV_Q4H) {
    const size_t rec = static_cast<size_t>(kvh) * pt + tok % pt;
    const uint8_t* codes = layer + (is_value ? records * (hd / 2U) + records * 2U : 0U) + rec * (hd / 2U) + d0 / 2U;
    for (uint32_t w = 0; w < dpp / 8U; ++w) {
      const uint32_t word = reinterpret_cast<const uint32_t*>(codes)[w];
#pragma unroll
      for (uint32_t i = 0; i < 8U; ++i) {
        const int nib = static_cast<int>((word >> (4U * i)) & 15U);
        out[8U * w + i] = static_cast<float>(nib >= 8 ? nib - 16 : nib);
      }
    }
  } else if (ENC == QLLM_KV_Q8) {
    const size_t rec = static_cast<size_t>(tok % pt) * a.kv_heads + kvh;
    const uint8_t* r8 = layer + (is_value ? records * (hd + 2U) : 0U) + rec * (hd + 2U);
    const float sc = __half2float(*reinterpret_cast<const __half*>(r8 + hd));
    const uint16_t* pairs = reinterpret_cast<const uint16_t*>(r8 + d0);  // records are 2-byte aligned
    for (uint32_t e = 0; e < dpp / 2U; ++e) {
      const uint16_t two = pairs[e];
      out[2U * e] = bf16r(static_cast<float>(static_cast<int8_t>(two & 0xffU)) * sc);
      out[2U * e + 1U] = bf16r(static_cast<float>(static_cast<int8_t>(two >> 8U)) * sc);
    }
  } else {
    const size_t rec = static_cast<size_t>(tok % pt) * a.kv_heads + kvh;
    const uint4* r16 = reinterpret_cast<const uint4*>(layer + (is_value ? records * hd * 2U : 0U) + (rec * hd + d0) * 2U);
    for (uint32_t w = 0; w < dpp / 8U; ++w) {
      const uint4 q = r16[w];
      const uint32_t words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (uint32_t i = 0; i < 4U; ++i) {
        out[8U * w + 2U * i] = __half2float(__ushort_as_half(static_cast<unsigned short>(words[i] & 0xffffU)));
        out[8U * w + 2U * i + 1U] = __half2float(__ushort_as_half(static_cast<unsigned short>(words[i] >> 16U)));
      }
    }
  }
}

template <uint32_t ENC, bool kTiled>
__global__ void __launch_bounds__(256)
attention_scalar_kernel(AttentionArgs a, Partials part) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  if constexpr (kTiled) attention_row_tile(a, part);
  const uint32_t hd = a.head_dim, group = a.q_heads / a.kv_heads;
  const uint32_t MR = a.rows * group;
  float* qs = smem;
  float* tile = qs + MR * hd;
  float* S = tile + 32U * (hd + 1U);
  float* P = S + MR * 33U;
  float* rmax = P + MR * 33U;
  float* rsum = rmax + MR;
  float* rprev = rsum + MR;
  float* rpscale = rprev + MR;
  float* rqscale = rpscale + MR;
  float* kscale = rqscale + MR;  // [32]
  float* vscale = kscale + 32U;  // [32]
  const uint32_t tid = threadIdx.x, warp = tid >> 5U, lane = tid & 31U;
  const uint32_t kvh = blockIdx.x, split = blockIdx.y;
  const uint32_t first_ctx = *a.first_position + a.position_offset + 1U;
  const uint32_t total = first_ctx + a.rows - 1U;
  const uint32_t first = split * a.split_tokens;
  if (first >= total) return;  // inactive split: the combine never reads it
  const uint32_t last = min(total, first + a.split_tokens);
  const uint32_t pt = a.page_tokens;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  const float inv_sqrt = 1.0F / sqrtf(static_cast<float>(hd));

  // queries: quantise / round per encoding
  for (uint32_t mr = warp; mr < MR; mr += 8U) {
    const uint32_t row = mr / group, head = kvh * group + mr % group;
    const float* q = a.query + static_cast<size_t>(row) * a.query_row_stride + static_cast<size_t>(head) * hd;
    if (ENC == QLLM_KV_Q4H) {
      float m = 0.0F;
      for (uint32_t d = lane; d < hd; d += 32U) m = fmaxf(m, fabsf(q[d]));
      m = warp_max(m);
      const float sc = fmaxf(m / 127.0F, 0x1p-24F);
      for (uint32_t d = lane; d < hd; d += 32U)
        qs[mr * hd + d] = static_cast<float>(max(-127, min(127, __float2int_rn(q[d] / sc))));
      if (lane == 0U) rqscale[mr] = sc;
    } else {
      for (uint32_t d = lane; d < hd; d += 32U)
        qs[mr * hd + d] = ENC == QLLM_KV_Q8 ? bf16r(q[d]) : __half2float(__float2half_rn(q[d]));
    }
    if (lane == 0U) { rmax[mr] = kNegInf; rsum[mr] = 0.0F; }
  }
  constexpr uint32_t kAcc = 32;  // MR*hd/256 <= 64*256/256 = 64 -> two passes of 32
  float acc[2][kAcc];
#pragma unroll
  for (int p = 0; p < 2; ++p)
#pragma unroll
    for (uint32_t i = 0; i < kAcc; ++i) acc[p][i] = 0.0F;
  const uint32_t outputs = MR * hd;
  __syncthreads();

  for (uint32_t t0 = first; t0 < last; t0 += 32U) {
    const uint32_t n = min(32U, last - t0);
    // ---- K tile
    load_kv_tile<ENC>(a, kvh, t0, n, false, tile);
    if (ENC == QLLM_KV_Q4H && tid < 64U) {
      const uint32_t j = tid & 31U;
      float sc = 0.0F;
      if (j < n) {
        const uint32_t tok = t0 + j;
        const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
        const size_t rec = static_cast<size_t>(kvh) * pt + tok % pt;
        const uint8_t* base = tid < 32U ? layer + records * (hd / 2U)
                                        : layer + records * (hd / 2U) * 2U + records * 2U;
        sc = __half2float(reinterpret_cast<const __half*>(base)[rec]);
      }
      (tid < 32U ? kscale : vscale)[j] = sc;
    }
    __syncthreads();
    // ---- scores
    for (uint32_t pair = tid; pair < MR * 32U; pair += 256U) {
      const uint32_t mr = pair / 32U, j = pair % 32U;
      const float* qr = qs + mr * hd;
      const float* kr = tile + j * (hd + 1U);
      float dot;
      if (ENC == QLLM_KV_Q4H) {
        float idot = 0.0F;  // integer-valued terms: exact in FP32
        for (uint32_t d = 0; d < hd; ++d) idot += qr[d] * kr[d];
        dot = idot * rqscale[mr] * kscale[j];
      } else {
        double ddot = 0.0;  // products of BF16/F16 values are exact; sum once
        for (uint32_t d = 0; d < hd; ++d) ddot += static_cast<double>(qr[d] * kr[d]);
        dot = static_cast<float>(ddot);
      }
      S[mr * 33U + j] = dot * inv_sqrt;
    }
    __syncthreads();
    // ---- online softmax, one warp per matrix row, lane = key
    for (uint32_t mr = warp; mr < MR; mr += 8U) {
      const uint32_t ctx = first_ctx + mr / group;
      const bool visible = lane < n && t0 + lane < ctx;
      const float score = visible ? S[mr * 33U + lane] : kNegInf;
      const float tmax = warp_max(score);
      const float old = rmax[mr];
      const float next = fmaxf(old, tmax);
      const float prev = old == kNegInf ? 0.0F : det_expf(old - next);
      float p = visible ? det_expf(score - next) : 0.0F;
      float stored;
      if (ENC == QLLM_KV_Q4H) {
        const float w = visible ? p * vscale[lane] : 0.0F;
        const float wmax = warp_max(w);
        const float pscale = fmaxf(wmax / 127.0F, 0x1p-24F);
        stored = static_cast<float>(max(0, min(127, __float2int_rn(w / pscale))));
        if (lane == 0U) rpscale[mr] = pscale;
      } else {
        p = ENC == QLLM_KV_Q8 ? bf16r(p) : __half2float(__float2half_rn(p));
        stored = p;
      }
      const float tsum = static_cast<float>(warp_sum_f64(static_cast<double>(p)));
      P[mr * 33U + lane] = stored;
      if (lane == 0U) {
        rsum[mr] = rsum[mr] * prev + tsum;
        rmax[mr] = next;
        rprev[mr] = prev;
      }
    }
    __syncthreads();
    // ---- V tile (reuses the K buffer)
    load_kv_tile<ENC>(a, kvh, t0, n, true, tile);
    __syncthreads();
    // ---- P.V, each thread owns outputs tid, tid+256, ...
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
#pragma unroll 4
      for (uint32_t i = 0; i < kAcc; ++i) {
        const uint32_t o = (pass * kAcc + i) * 256U + tid;
        if (o < outputs) {
          const uint32_t mr = o / hd, d = o % hd;
          if (ENC == QLLM_KV_Q4H) {
            float idot = 0.0F;  // integer-valued terms: exact in FP32
            for (uint32_t j = 0; j < 32U; ++j) idot += P[mr * 33U + j] * tile[j * (hd + 1U) + d];
            acc[pass][i] = fmaf(idot, rpscale[mr], acc[pass][i] * rprev[mr]);
          } else {
            double ddot = 0.0;
            for (uint32_t j = 0; j < 32U; ++j)
              ddot += static_cast<double>(P[mr * 33U + j] * tile[j * (hd + 1U) + d]);
            acc[pass][i] = acc[pass][i] * rprev[mr] + static_cast<float>(ddot);
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- partials
#pragma unroll
  for (int pass = 0; pass < 2; ++pass)
#pragma unroll 4
    for (uint32_t i = 0; i < kAcc; ++i) {
      const uint32_t o = (pass * kAcc + i) * 256U + tid;
      if (o < outputs) {
        const uint32_t mr = o / hd, d = o % hd;
        const uint32_t row = mr / group, head = kvh * group + mr % group;
        const size_t pidx = (static_cast<size_t>(row) * a.max_splits + split) * a.q_heads + head;
        part.outputs[pidx * hd + d] = acc[pass][i];
        if (d == 0U) { part.maxima[pidx] = rmax[mr]; part.sums[pidx] = rsum[mr]; }
      }
    }
}

// grid (q_heads, rows), block head_dim.
__global__ void attention_combine_kernel(AttentionArgs a, Partials part) {
  __shared__ float gmax, gsum;
  const uint32_t head = blockIdx.x, row = blockIdx.y, d = threadIdx.x, hd = a.head_dim;
  const uint32_t ctx = *a.first_position + a.position_offset + 1U + row;
  const uint32_t active = (ctx + a.split_tokens - 1U) / a.split_tokens;
  const size_t base = static_cast<size_t>(row) * a.max_splits * a.q_heads + head;
  if (d == 0U) {
    float m = kNegInf;
    for (uint32_t s = 0; s < active; ++s) m = fmaxf(m, part.maxima[base + static_cast<size_t>(s) * a.q_heads]);
    float sum = 0.0F;
    for (uint32_t s = 0; s < active; ++s) {
      const size_t p = base + static_cast<size_t>(s) * a.q_heads;
      sum += part.sums[p] * det_expf(part.maxima[p] - m);
    }
    gmax = m;
    gsum = sum;
  }
  __syncthreads();
  float result = 0.0F;
  for (uint32_t s = 0; s < active; ++s) {
    const size_t p = base + static_cast<size_t>(s) * a.q_heads;
    result += part.outputs[p * hd + d] * det_expf(part.maxima[p] - gmax);
  }
  a.out[(static_cast<size_t>(row) * a.q_heads + head) * hd + d] = actv(result / gsum, a.bf16);
}

int launch_attention(const AttentionArgs& a, cudaStream_t stream) {
  const uint32_t group = a.kv_heads ? a.q_heads / a.kv_heads : 0U;
  const uint32_t MR = a.rows * group;
  if (!a.rows || !group || a.q_heads % a.kv_heads || a.head_dim % 64U || a.head_dim > 256U ||
      a.split_tokens % 32U || !a.split_tokens || a.page_tokens % 32U || !a.max_splits || MR > 64U)
    return fail(QLLM_INVALID_ARGUMENT, "unsupported attention geometry");
  const Partials part = partials_of(a);
  const dim3 grid(a.kv_heads, a.max_splits, a.tiles > 1U ? a.tiles : 1U);
  if (a.tiles > 1U && !a.skip_combine) return fail(QLLM_INVALID_ARGUMENT, "row tiles are merged by the caller");
  const bool mma = a.impl >= 1;   // 2 asks for the tensor-memory kernel where one exists (Q4H)
  if (a.impl == 2 && a.encoding == QLLM_KV_Q4H && attention_q4h_tc_supported(a)) {
    const size_t items = attention_partial_items(a.rows, a.max_splits, a.q_heads) * (a.tiles > 1U ? a.tiles : 1U);
    uint8_t* scratch = static_cast<uint8_t*>(a.workspace) +
                       ((items * (2U + a.head_dim) * sizeof(float) + 255U) & ~static_cast<size_t>(255U));
    const int rc = launch_attention_q4h_tc(a, part.maxima, part.sums, part.outputs, a.error, scratch, stream);
    if (rc) return rc;
  } else if (mma && a.encoding == QLLM_KV_F16) {
    if (!attention_f16_mma_supported(a))
      return fail(QLLM_INVALID_ARGUMENT,
                  "tensor-core F16 attention needs head_dim 128, rows*group <= 32, 32-token aligned pages and splits");
    const int rc = launch_attention_f16_mma(a, part.maxima, part.sums, part.outputs, a.error, stream);
    if (rc) return rc;
  } else if (mma && a.encoding == QLLM_KV_Q8) {
    if (!attention_q8_mma_supported(a))
      return fail(QLLM_INVALID_ARGUMENT,
                  "tensor-core Q8 attention needs head_dim 128, at most 8 kv heads, rows*group <= 32, "
                  "32-token aligned pages and splits");
    const int rc = launch_attention_q8_mma(a, part.maxima, part.sums, part.outputs, a.error, stream);
    if (rc) return rc;
  } else if (mma) {
    if (a.encoding != QLLM_KV_Q4H || a.head_dim != 128U || MR > 64U || a.query_row_stride % 4U ||
        a.page_tokens % 64U || a.split_tokens % 64U)
      return fail(QLLM_INVALID_ARGUMENT,
                  "tensor-core attention needs Q4H, head_dim 128, rows*group <= 64, 64-token aligned pages and splits");
    const int rc = launch_attention_q4h_pipelined(a, part.maxima, part.sums, part.outputs, a.error, stream);
    if (rc) return rc;
  } else {
    const size_t smem = (static_cast<size_t>(MR) * a.head_dim + 32U * (a.head_dim + 1U) +
                         2U * MR * 33U + 5U * MR + 64U) * sizeof(float);
    // The opt-in limit is a property of the function, not of a launch: it is only ever
    // raised (to the largest geometry the kernel accepts), because launches captured into a
    // graph earlier keep their own, possibly larger, shared-memory size.
    constexpr size_t kLargest = (64U * 256U + 32U * 257U + 2U * 64U * 33U + 5U * 64U + 64U) * sizeof(float);
    static bool configured[64][3] = {};  // per device, per encoding (both forms of the kernel)
    const bool tiled = a.tiles > 1U;
    bool both = true;
    int device = 0;
    cudaGetDevice(&device);
    auto set = [&](auto kernel) {
      bool& done = configured[device & 63][a.encoding == QLLM_KV_Q4H ? 0 : a.encoding == QLLM_KV_Q8 ? 1 : 2];
      if (done) return cudaSuccess;
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kLargest));
      both = both && e == cudaSuccess;
      return e;
    };
    cudaError_t e;
    switch (a.encoding) {
      case QLLM_KV_Q4H:
        e = set(attention_scalar_kernel<QLLM_KV_Q4H, false>);
        if (e == cudaSuccess) e = set(attention_scalar_kernel<QLLM_KV_Q4H, true>);
        if (e == cudaSuccess)
          e = tiled ? launch_ordered(attention_scalar_kernel<QLLM_KV_Q4H, true>, grid, dim3(256), smem, stream, a, part)
                    : launch_ordered(attention_scalar_kernel<QLLM_KV_Q4H, false>, grid, dim3(256), smem, stream, a, part);
        break;
      case QLLM_KV_Q8:
        e = set(attention_scalar_kernel<QLLM_KV_Q8, false>);
        if (e == cudaSuccess) e = set(attention_scalar_kernel<QLLM_KV_Q8, true>);
        if (e == cudaSuccess)
          e = tiled ? launch_ordered(attention_scalar_kernel<QLLM_KV_Q8, true>, grid, dim3(256), smem, stream, a, part)
                    : launch_ordered(attention_scalar_kernel<QLLM_KV_Q8, false>, grid, dim3(256), smem, stream, a, part);
        break;
      case QLLM_KV_F16:
        e = set(attention_scalar_kernel<QLLM_KV_F16, false>);
        if (e == cudaSuccess) e = set(attention_scalar_kernel<QLLM_KV_F16, true>);
        if (e == cudaSuccess)
          e = tiled ? launch_ordered(attention_scalar_kernel<QLLM_KV_F16, true>, grid, dim3(256), smem, stream, a, part)
                    : launch_ordered(attention_scalar_kernel<QLLM_KV_F16, false>, grid, dim3(256), smem, stream, a, part);
        break;
      default:
        return fail(QLLM_INVALID_ARGUMENT, "unknown KV encoding");
    }
    if (e != cudaSuccess) return check_cuda(e, "attention shared memory opt-in");
    if (both) configured[device & 63][a.encoding == QLLM_KV_Q4H ? 0 : a.encoding == QLLM_KV_Q8 ? 1 : 2] = true;
  }
  count_launch();
  if (a.skip_combine) return check_launch("attention");  // the caller merges the splits itself
  CombineArgs c{};
  c.maxima = part.maxima;
  c.sums = part.sums;
  c.outputs = part.outputs;
  c.first_position = a.first_position;
  c.position_offset = a.position_offset;
  c.q_heads = a.q_heads;
  c.head_dim = a.head_dim;
  c.split_tokens = a.split_tokens;
  c.max_splits = a.max_splits;
  c.bf16 = a.bf16;
  c.out = a.out;
  c.exact = a.impl == 0;
  c.sink = no_sink();
  return launch_combine_quant(c, a.rows, stream);
}

// ------------------------------------------------------- synthetic cache fill
__device__ __forceinline__ uint32_t hash32(uint64_t x) {
  x ^= x >> 33U; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33U; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33U;
  return static_cast<uint32_t>(x);
}
// One thread per (token, kv head, K|V): writes a record with pseudo-random codes and a
// scale near 0.2 (K and V magnitudes of a random-init decoder).
__global__ void fill_synthetic_kv_kernel(uint8_t* const* page_table, size_t layer_offset,
                                         uint32_t enc, uint32_t pt, uint32_t kv, uint32_t hd,
                                         uint32_t first, uint32_t count, uint64_t seed) {
  const uint64_t item = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (item >= static_cast<uint64_t>(count) * kv * 2U) return;
  const uint32_t which = item & 1U;
  const uint32_t h = (item >> 1U) % kv;
  const uint32_t pos = first + static_cast<uint32_t>((item >> 1U) / kv);
  uint8_t* layer = page_table[pos / pt] + layer_offset;
  const size_t records = static_cast<size_t>(pt) * kv;
  const uint32_t slot = pos % pt;
  const uint64_t key = seed ^ (static_cast<uint64_t>(pos) << 20U) ^ (static_cast<uint64_t>(h) << 4U) ^ which;
  const __half scale = __float2half_rn(0.1F + 0.2F * static_cast<float>(hash32(key) & 0xffffU) / 65536.0F);
  if (enc == QLLM_KV_Q4H) {
    const size_t rec = static_cast<size_t>(h) * pt + slot;
    uint8_t* codes = layer + (which ? records * (hd / 2U) + records * 2U : 0U) + rec * (hd / 2U);
    uint8_t* sc = layer + records * (hd / 2U) + (which ? records * (hd / 2U) + records * 2U : 0U);
    reinterpret_cast<__half*>(sc)[rec] = scale;
    for (uint32_t d = 0; d < hd / 2U; ++d) {
      const uint32_t r = hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U);
      int lo = static_cast<int>(r % 15U) - 7, hi = static_cast<int>((r >> 8U) % 15U) - 7;
      codes[d] = static_cast<uint8_t>((lo & 15) | ((hi & 15) << 4));
    }
  } else if (enc == QLLM_KV_Q8) {
    const size_t rec = static_cast<size_t>(slot) * kv + h;
    uint8_t* r8 = layer + (which ? records * (hd + 2U) : 0U) + rec * (hd + 2U);
    *reinterpret_cast<__half*>(r8 + hd) = __float2half_rn(__half2float(scale) / 16.0F);
    for (uint32_t d = 0; d < hd; ++d)
      r8[d] = static_cast<uint8_t>(static_cast<int8_t>(static_cast<int>(hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U) % 255U) - 127));
  } else {
    const size_t rec = static_cast<size_t>(slot) * kv + h;
    __half* r16 = reinterpret_cast<__half*>(layer + (which ? records * hd * 2U : 0U)) + rec * hd;
    for (uint32_t d = 0; d < hd; ++d)
      r16[d] = __float2half_rn((static_cast<float>(hash32(key * 0x9e3779b97f4a7c15ULL + d + 1U) & 0xffffU) / 32768.0F - 1.0F) * 1.4F);
  }
}

int launch_fill_synthetic_kv(uint8_t* const* page_table, size_t layer_offset, uint32_t encoding,
                             uint32_t page_tokens, uint32_t kv_heads, uint32_t head_dim,
                             uint32_t first, uint32_t count, uint64_t seed, cudaStream_t stream) {
  const uint64_t items = static_cast<uint64_t>(count) * kv_heads * 2U;
  if (!items) return 0;
  fill_synthetic_kv_kernel<<<static_cast<unsigned>((items + 127U) / 128U), 128, 0, stream>>>(
      page_table, layer_offset, encoding, page_tokens, kv_heads, head_dim, first, count, seed);
  count_launch();
  return check_launch("fill_synthetic_kv");
}

}  // namespace qllm
