// Flash-decode attention over the Q8 (int8 codes + f16 scale per head) paged cache of the
// draft layer, head_dim 128, on BF16 tensor cores.
//
// Arithmetic of the reference's Q8 kernels (runtime/src/cuda/transformer_kernels.cu:4985-5340):
// queries, dequantised keys/values (code * scale) and probabilities are rounded to BF16, the
// products accumulate in FP32, online softmax over tiles of 32 keys.
//
// The records of one token are token-major ([token][kv head][128 codes + f16 scale], 130 bytes
// each), so a whole tile of 32 tokens is contiguous for ALL kv heads: CTA = (context split,
// 16-row matrix tile), one warp per kv head, and one bulk asynchronous copy per tile for the
// keys and one for the values, through a three-stage mbarrier ring.  Every warp dequantises
// the K and V bytes of its own head straight into mma.m16n8k16 B fragments (the k-slot order
// inside an MMA is free as long as A and B agree, so a lane always converts 4 neighbouring
// codes of one record for K; V needs one byte per key, read from shared memory without bank
// conflicts because consecutive tokens are 260 words apart).
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

#include <cuda_bf16.h>

namespace qllm {

namespace {

constexpr uint32_t HD = 128;
constexpr uint32_t kTile = 32;            // keys per stage
constexpr uint32_t kStages = 3;
constexpr uint32_t kRecord = HD + 2U;     // 130 bytes
constexpr uint32_t kSpin = 1U << 20;
constexpr uint32_t kFull = 0xffffffffU;

__device__ __forceinline__ uint32_t s32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ bool wait_parity(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag) {
  const uint32_t addr = s32(bar);
  for (uint32_t spin = 0; spin < kSpin; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 255U) == 255U && *abort_flag) return false;
  }
  *abort_flag = 1U;
  return false;
}
__device__ __forceinline__ void bulk(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(s32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), round to nearest even
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float code_f(uint32_t word, uint32_t byte) {
  return static_cast<float>(static_cast<int8_t>((word >> (8U * byte)) & 0xffU));
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(kFull, v, 1));
  return fmaxf(v, __shfl_xor_sync(kFull, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(kFull, v, 1);
  return v + __shfl_xor_sync(kFull, v, 2);
}

}  // namespace

struct Q8Partials {
  float* maxima;
  float* sums;
  float* outputs;
};

// grid (context splits, 16-row matrix tiles), block 32 * kv_heads; dynamic shared memory =
// kStages * 2 * kTile * kv_heads * 130 bytes.
template <bool kTiled>  // grid z = row tile of a wide pass
__global__ void __launch_bounds__(256)
attention_q8_mma_kernel(AttentionArgs a, Q8Partials part, uint32_t* error) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ uint32_t abort_word;
  pdl_trigger();  // the combine kernel may be scheduled; it waits for this grid
  pdl_wait();     // queries and the newest records come from the RoPE kernel before this one
  if constexpr (kTiled) attention_row_tile(a, part);
  const uint32_t tid = threadIdx.x, kvh = tid >> 5U, lane = tid & 31U;
  const uint32_t g = lane >> 2U, t = lane & 3U;
  const uint32_t split = blockIdx.x, mtile = blockIdx.y;
  const uint32_t kv = a.kv_heads, group = a.q_heads / kv;
  const uint32_t MR = a.rows * group;
  const uint32_t first_ctx = *a.first_position + a.position_offset + 1U;
  const uint32_t total = first_ctx + a.rows - 1U;
  const uint32_t first = split * a.split_tokens;
  if (first >= total) return;
  const uint32_t last = min(total, first + a.split_tokens);
  const uint32_t tiles = (last - first + kTile - 1U) / kTile;
  const uint32_t pt = a.page_tokens;
  const uint32_t token_bytes = kv * kRecord;             // 1040 for 8 kv heads
  const uint32_t half_bytes = kTile * token_bytes;       // K (or V) bytes of one stage
  const size_t v_region = static_cast<size_t>(pt) * token_bytes;
  const float inv_sqrt = 1.0F / sqrtf(static_cast<float>(HD));
  volatile uint32_t* abort_flag = &abort_word;

  if (tid == 0U) {
    for (uint32_t s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&full_bar[s])), "r"(1U));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&empty_bar[s])), "r"(kv));
    }
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](uint32_t tile) {
    const uint32_t s = tile % kStages;
    const uint32_t tok = first + tile * kTile;
    const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
    const uint8_t* ksrc = layer + static_cast<size_t>(tok % pt) * token_bytes;
    uint8_t* dst = ring + static_cast<size_t>(s) * 2U * half_bytes;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&full_bar[s])),
                 "r"(2U * half_bytes) : "memory");
    bulk(dst, ksrc, half_bytes, &full_bar[s]);
    bulk(dst + half_bytes, ksrc + v_region, half_bytes, &full_bar[s]);
  };
  if (tid == 0U)
    for (uint32_t c = 0; c < min(tiles, kStages); ++c) issue(c);

  // A fragments of the BF16 queries: in k-step ks the slots {2t, 2t+1, 2t+8, 2t+9} of this
  // thread carry the dims 16*ks + 4t + {0, 1, 2, 3}
  const uint32_t row_lo = 16U * mtile + g, row_hi = row_lo + 8U;
  uint32_t qa[8][4];
  {
    float4 lo[8], hi[8];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) lo[ks] = hi[ks] = make_float4(0.0F, 0.0F, 0.0F, 0.0F);
    if (row_lo < MR) {
      const float* q = a.query + static_cast<size_t>(row_lo / group) * a.query_row_stride +
                       static_cast<size_t>(kvh * group + row_lo % group) * HD + 4U * t;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) lo[ks] = *reinterpret_cast<const float4*>(q + 16 * ks);
    }
    if (row_hi < MR) {
      const float* q = a.query + static_cast<size_t>(row_hi / group) * a.query_row_stride +
                       static_cast<size_t>(kvh * group + row_hi % group) * HD + 4U * t;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) hi[ks] = *reinterpret_cast<const float4*>(q + 16 * ks);
    }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = pack_bf16(lo[ks].x, lo[ks].y);
      qa[ks][1] = pack_bf16(hi[ks].x, hi[ks].y);
      qa[ks][2] = pack_bf16(lo[ks].z, lo[ks].w);
      qa[ks][3] = pack_bf16(hi[ks].z, hi[ks].w);
    }
  }
  const uint32_t ctx_lo = row_lo < MR ? first_ctx + row_lo / group : 0U;
  const uint32_t ctx_hi = row_hi < MR ? first_ctx + row_hi / group : 0U;
  float m_lo = kNegInf, m_hi = kNegInf, sum_lo = 0.0F, sum_hi = 0.0F;
  float out[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) out[j][e] = 0.0F;
  bool ok = true;

  for (uint32_t c = 0; c < tiles && ok; ++c) {
    const uint32_t s = c % kStages;
    ok = wait_parity(&full_bar[s], (c / kStages) & 1U, abort_flag);
    if (!ok) break;
    const uint8_t* kbase = ring + static_cast<size_t>(s) * 2U * half_bytes + kvh * kRecord;
    const uint8_t* vbase = kbase + half_bytes;
    const uint32_t tok0 = first + c * kTile;
    const bool masked = tok0 + kTile > min(last, first_ctx);
    // ---- S = Q K^T
    float sc_lo[8], sc_hi[8];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const uint8_t* rec = kbase + (8U * nt + g) * token_bytes;
      const float ksc = __half2float(*reinterpret_cast<const __half*>(rec + HD));
      float cfrag[4] = {0.0F, 0.0F, 0.0F, 0.0F};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        // records are 2-byte aligned: two 16-bit reads
        const uint32_t w01 = *reinterpret_cast<const uint16_t*>(rec + 16 * ks + 4U * t);
        const uint32_t w23 = *reinterpret_cast<const uint16_t*>(rec + 16 * ks + 4U * t + 2U);
        const uint32_t b0 = pack_bf16(code_f(w01, 0) * ksc, code_f(w01, 1) * ksc);
        const uint32_t b1 = pack_bf16(code_f(w23, 0) * ksc, code_f(w23, 1) * ksc);
        mma_bf16(cfrag, qa[ks], b0, b1);
      }
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        float lo = cfrag[e] * inv_sqrt, hi = cfrag[2 + e] * inv_sqrt;
        if (masked) {
          const uint32_t tok = tok0 + 8U * nt + 2U * t + e;
          const bool in = tok < last;
          if (!(in && tok < ctx_lo)) lo = kNegInf;
          if (!(in && tok < ctx_hi)) hi = kNegInf;
        }
        sc_lo[2 * nt + e] = lo;
        sc_hi[2 * nt + e] = hi;
      }
    }
    // ---- online softmax per row (a row's 32 keys live in the 4 lanes of a quad)
    float tmax_lo = sc_lo[0], tmax_hi = sc_hi[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) { tmax_lo = fmaxf(tmax_lo, sc_lo[i]); tmax_hi = fmaxf(tmax_hi, sc_hi[i]); }
    tmax_lo = quad_max(tmax_lo);
    tmax_hi = quad_max(tmax_hi);
    const float next_lo = fmaxf(m_lo, tmax_lo), next_hi = fmaxf(m_hi, tmax_hi);
    // kNegInf is the lowest finite float: exp(-huge) = 0 for a first tile, exp(0) = 1 on
    // still-zero accumulators for a row that has seen no visible key yet
    const float prev_lo = __expf(m_lo - next_lo), prev_hi = __expf(m_hi - next_hi);
    float ts_lo = 0.0F, ts_hi = 0.0F;
    uint32_t pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float p[4];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int i = 2 * nt + e;
        float p_lo = __expf(sc_lo[i] - next_lo), p_hi = __expf(sc_hi[i] - next_hi);
        if (masked) {
          if (sc_lo[i] == kNegInf) p_lo = 0.0F;
          if (sc_hi[i] == kNegInf) p_hi = 0.0F;
        }
        p[e] = bf16r(p_lo);
        p[2 + e] = bf16r(p_hi);
        ts_lo += p[e];
        ts_hi += p[2 + e];
      }
      // P.V k-step nt/2: slots {2t, 2t+1} = keys of an even key tile, {2t+8, 2t+9} = of the odd one
      pa[nt >> 1][(nt & 1) * 2] = pack_bf16(p[0], p[1]);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p[2], p[3]);
    }
    sum_lo = sum_lo * prev_lo + quad_sum(ts_lo);
    sum_hi = sum_hi * prev_hi + quad_sum(ts_hi);
    m_lo = next_lo;
    m_hi = next_hi;
    if (__any_sync(kFull, prev_lo != 1.0F || prev_hi != 1.0F)) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        out[j][0] *= prev_lo; out[j][1] *= prev_lo;
        out[j][2] *= prev_hi; out[j][3] *= prev_hi;
      }
    }
    // ---- O += P V: B column n = g is dim 8j + g; slots {2t, 2t+1, 2t+8, 2t+9} are keys
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const uint8_t* r0 = vbase + (16U * kk + 2U * t) * token_bytes;   // keys 16kk+2t, +1
      const uint8_t* r1 = r0 + 8U * token_bytes;                       // keys 16kk+8+2t, +1
      const float v00 = __half2float(*reinterpret_cast<const __half*>(r0 + HD));
      const float v01 = __half2float(*reinterpret_cast<const __half*>(r0 + token_bytes + HD));
      const float v10 = __half2float(*reinterpret_cast<const __half*>(r1 + HD));
      const float v11 = __half2float(*reinterpret_cast<const __half*>(r1 + token_bytes + HD));
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t d = 8U * j + g;
        const float a0 = static_cast<float>(static_cast<int8_t>(r0[d])) * v00;
        const float a1 = static_cast<float>(static_cast<int8_t>(r0[token_bytes + d])) * v01;
        const float b0f = static_cast<float>(static_cast<int8_t>(r1[d])) * v10;
        const float b1f = static_cast<float>(static_cast<int8_t>(r1[token_bytes + d])) * v11;
        mma_bf16(out[j], pa[kk], pack_bf16(a0, a1), pack_bf16(b0f, b1f));
      }
    }
    // this warp is done with stage s
    __syncwarp();
    if (lane == 0U) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&empty_bar[s])) : "memory");
    if (tid == 0U && c + kStages < tiles) {
      ok = wait_parity(&empty_bar[s], (c / kStages) & 1U, abort_flag);
      if (ok) issue(c + kStages);
    }
    if (kvh == 0U) ok = __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
  }
  if (*abort_flag) {
    if (tid == 0U && error) atomicExch(error, 300U);
    return;
  }
  // ---- partials: C column 2t+e of tile j is dim 8j + 2t + e
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t mr = half ? row_hi : row_lo;
    if (mr >= MR) continue;
    const uint32_t row = mr / group, head = kvh * group + mr % group;
    const size_t pidx = (static_cast<size_t>(row) * a.max_splits + split) * a.q_heads + head;
    float* dst = part.outputs + pidx * HD + 2U * t;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      *reinterpret_cast<float2*>(dst + 8 * j) = make_float2(out[j][2 * half], out[j][2 * half + 1]);
    if (t == 0U) {
      part.maxima[pidx] = half ? m_hi : m_lo;
      part.sums[pidx] = half ? sum_hi : sum_lo;
    }
  }
}

bool attention_q8_mma_supported(const AttentionArgs& a) {
  const uint32_t group = a.kv_heads ? a.q_heads / a.kv_heads : 0U;
  return a.encoding == QLLM_KV_Q8 && a.head_dim == HD && a.kv_heads && a.kv_heads <= 8U && group &&
         a.rows * group <= 64U && a.page_tokens % kTile == 0U && a.split_tokens % kTile == 0U &&
         a.query_row_stride % 4U == 0U;
}

int launch_attention_q8_mma(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                            cudaStream_t stream) {
  Q8Partials part{maxima, sums, outputs};
  const uint32_t group = a.q_heads / a.kv_heads;
  const uint32_t mtiles = (a.rows * group + 15U) / 16U;
  const size_t smem = static_cast<size_t>(kStages) * 2U * kTile * a.kv_heads * kRecord;
  // raised once per device to the largest size the kernel accepts (8 kv heads)
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attention_q8_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kStages * 2U * kTile * 8U * kRecord));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_q8_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(kStages * 2U * kTile * 8U * kRecord));
    if (e != cudaSuccess) return check_cuda(e, "Q8 attention shared memory opt-in");
    configured[device & 63] = true;
  }
  if (a.tiles > 1U)
    return check_cuda(launch_ordered(attention_q8_mma_kernel<true>, dim3(a.max_splits, mtiles, a.tiles), dim3(32U * a.kv_heads),
                                     smem, stream, a, part, error), "attention_q8_mma");
  return check_cuda(launch_ordered(attention_q8_mma_kernel<false>, dim3(a.max_splits, mtiles), dim3(32U * a.kv_heads), smem,
                                   stream, a, part, error), "attention_q8_mma");
}

}  // namespace qllm
