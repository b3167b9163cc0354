// Flash-decode attention over the Q4H (int4 codes + f16 scale per head) paged cache with the
// dequantisation fused into the kernel, head_dim 128.
//
// CTA = (kv head, context split), two warps: warp w owns matrix rows 16w..16w+15
// (matrix row = verify row * group + grouped head, up to 32).  K/V codes and scales of 64 keys
// at a time are staged into shared memory by bulk asynchronous copies (the records of one kv
// head are contiguous inside a page) through a 4-stage mbarrier ring, so HBM latency is hidden
// behind the tensor-core work.  Per 32 keys, as in the reference
// (runtime/src/cuda/transformer_kernels.cu:4421-4976): INT8 queries, integer Q.K^T, FP32 online
// softmax, P*v-scale re-quantised to INT8 per row, integer P.V.  Both products are INT8
// m16n8k32 MMAs fed straight from the packed nibbles: a code c is used as the byte 16*c
// (one shift/mask per 8 codes) and the 1/16 is folded into the scale; the k-slot order inside
// an MMA is free as long as A and B agree, so no nibble is ever moved across lanes, and the
// probabilities go from the C fragment of Q.K^T to the A fragment of P.V in registers.
#include "common.cuh"
#include "kernels.h"

namespace qllm {

namespace {

constexpr uint32_t HD = 128;
constexpr uint32_t kChunk = 64;                 // keys per pipeline stage
constexpr uint32_t kStages = 4;
constexpr uint32_t kCodeBytes = kChunk * HD / 2;  // 4096
constexpr uint32_t kScaleBytes = kChunk * 2;      // 128
constexpr uint32_t kStageBytes = 2 * kCodeBytes + 2 * kScaleBytes;
constexpr uint32_t kSpin = 1U << 20;

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
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffU, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffU, v, 2));
}
__device__ __forceinline__ double quad_sum(double v) {
  v += __shfl_xor_sync(0xffffffffU, v, 1);
  return v + __shfl_xor_sync(0xffffffffU, v, 2);
}

}  // namespace

struct Q4hPartials {
  float* maxima;
  float* sums;
  float* outputs;
};

__global__ void __launch_bounds__(64)
attention_q4h_pipelined_kernel(AttentionArgs a, Q4hPartials part, uint32_t* error) {
  __shared__ __align__(128) uint8_t ring[kStages][kStageBytes];
  __shared__ __align__(16) int8_t qs[32][HD + 16];
  __shared__ float qscale_s[32];
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ uint32_t abort_word;
  const uint32_t tid = threadIdx.x, warp = tid >> 5U, lane = tid & 31U;
  const uint32_t g = lane >> 2U, t = lane & 3U;
  const uint32_t kvh = blockIdx.x, split = blockIdx.y;
  const uint32_t group = a.q_heads / a.kv_heads;
  const uint32_t MR = a.rows * group;
  const uint32_t first_ctx = *a.first_position + a.position_offset + 1U;
  const uint32_t total = first_ctx + a.rows - 1U;
  const uint32_t first = split * a.split_tokens;
  if (first >= total) return;
  const uint32_t last = min(total, first + a.split_tokens);
  const uint32_t chunks = (last - first + kChunk - 1U) / kChunk;
  const uint32_t pt = a.page_tokens;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;
  const float inv_sqrt = 1.0F / sqrtf(static_cast<float>(HD));
  volatile uint32_t* abort_flag = &abort_word;

  if (tid == 0U) {
    for (uint32_t s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&full_bar[s])), "r"(1U));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&empty_bar[s])), "r"(2U));
    }
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // INT8 queries of this warp's 16 matrix rows (lane owns 4 dims)
  for (uint32_t i = 0; i < 16U; ++i) {
    const uint32_t mr = 16U * warp + i;
    float v[4] = {0.0F, 0.0F, 0.0F, 0.0F};
    if (mr < MR) {
      const uint32_t row = mr / group, head = kvh * group + mr % group;
      const float4 q4 = *reinterpret_cast<const float4*>(
          a.query + static_cast<size_t>(row) * a.query_row_stride + static_cast<size_t>(head) * HD + lane * 4U);
      v[0] = q4.x; v[1] = q4.y; v[2] = q4.z; v[3] = q4.w;
    }
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    m = warp_max(m);
    const float sc = fmaxf(m / 127.0F, 0x1p-24F);
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int q = mr < MR ? max(-127, min(127, __float2int_rn(v[e] / sc))) : 0;
      packed |= (static_cast<uint32_t>(q) & 0xffU) << (8 * e);
    }
    *reinterpret_cast<uint32_t*>(&qs[mr][lane * 4U]) = packed;
    if (lane == 0U) qscale_s[mr] = mr < MR ? sc : 0.0F;
  }
  __syncthreads();

  // producer state (thread 0) -------------------------------------------------------------
  auto issue = [&](uint32_t chunk) {
    const uint32_t s = chunk % kStages;
    const uint32_t tok = first + chunk * kChunk;
    const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
    const size_t rec = static_cast<size_t>(kvh) * pt + tok % pt;
    const uint8_t* kc = layer + rec * (HD / 2U);
    const uint8_t* ks = layer + records * (HD / 2U) + rec * 2U;
    const uint8_t* vc = layer + records * (HD / 2U) + records * 2U + rec * (HD / 2U);
    const uint8_t* vs = layer + records * (HD / 2U) * 2U + records * 2U + rec * 2U;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&full_bar[s])),
                 "r"(kStageBytes) : "memory");
    bulk(&ring[s][0], kc, kCodeBytes, &full_bar[s]);
    bulk(&ring[s][kCodeBytes], vc, kCodeBytes, &full_bar[s]);
    bulk(&ring[s][2U * kCodeBytes], ks, kScaleBytes, &full_bar[s]);
    bulk(&ring[s][2U * kCodeBytes + kScaleBytes], vs, kScaleBytes, &full_bar[s]);
  };
  if (tid == 0U)
    for (uint32_t c = 0; c < min(chunks, kStages); ++c) issue(c);

  // A fragments of the queries: for k-step ks this thread's k slots carry dims 8*(4t+ks)+{0..7}
  uint32_t qa[4][4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    const uint2 lo = *reinterpret_cast<const uint2*>(&qs[16U * warp + g][8U * (4U * t + ks)]);
    const uint2 hi = *reinterpret_cast<const uint2*>(&qs[16U * warp + g + 8U][8U * (4U * t + ks)]);
    qa[ks][0] = __byte_perm(lo.x, lo.y, 0x6420);  // even dims -> slots 4t..4t+3
    qa[ks][1] = __byte_perm(hi.x, hi.y, 0x6420);
    qa[ks][2] = __byte_perm(lo.x, lo.y, 0x7531);  // odd dims -> slots 16+4t..
    qa[ks][3] = __byte_perm(hi.x, hi.y, 0x7531);
  }
  const uint32_t row_lo = 16U * warp + g, row_hi = row_lo + 8U;
  // K bytes carry 16*code: the exact factor 1/16 rides on the query scale
  const float qs_lo = qscale_s[row_lo] * 0.0625F, qs_hi = qscale_s[row_hi] * 0.0625F;
  const uint32_t ctx_lo = row_lo < MR ? first_ctx + row_lo / group : 0U;
  const uint32_t ctx_hi = row_hi < MR ? first_ctx + row_hi / group : 0U;
  float m_lo = kNegInf, m_hi = kNegInf, sum_lo = 0.0F, sum_hi = 0.0F;
  float out[2][8][4];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) out[h][j][e] = 0.0F;
  const bool warp_active = 16U * warp < MR;
  bool ok = true;

  for (uint32_t c = 0; c < chunks && ok; ++c) {
    const uint32_t s = c % kStages;
    ok = wait_parity(&full_bar[s], (c / kStages) & 1U, abort_flag);
    if (!ok) break;
    if (warp_active) {
      const uint8_t* kcodes = &ring[s][0];
      const uint8_t* vcodes = &ring[s][kCodeBytes];
      const __half* kscales = reinterpret_cast<const __half*>(&ring[s][2U * kCodeBytes]);
      const __half* vscales = reinterpret_cast<const __half*>(&ring[s][2U * kCodeBytes + kScaleBytes]);
#pragma unroll 1
      for (uint32_t sub = 0; sub < 2U; ++sub) {
        const uint32_t t0 = first + c * kChunk + sub * 32U;
        if (t0 >= last) break;
        const uint32_t kb = sub * 32U;  // first key of the sub-tile inside the stage
        // ---- S = Q K^T: 4 key tiles of 8, one 16-byte read per key
        float sc_lo[8], sc_hi[8];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
          const uint4 w = *reinterpret_cast<const uint4*>(kcodes + (kb + 8U * nt + g) * (HD / 2U) + 16U * t);
          int cfrag[4] = {0, 0, 0, 0};
          mma_s8(cfrag, qa[0][0], qa[0][1], qa[0][2], qa[0][3], (w.x << 4U) & 0xf0f0f0f0U, w.x & 0xf0f0f0f0U);
          mma_s8(cfrag, qa[1][0], qa[1][1], qa[1][2], qa[1][3], (w.y << 4U) & 0xf0f0f0f0U, w.y & 0xf0f0f0f0U);
          mma_s8(cfrag, qa[2][0], qa[2][1], qa[2][2], qa[2][3], (w.z << 4U) & 0xf0f0f0f0U, w.z & 0xf0f0f0f0U);
          mma_s8(cfrag, qa[3][0], qa[3][1], qa[3][2], qa[3][3], (w.w << 4U) & 0xf0f0f0f0U, w.w & 0xf0f0f0f0U);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const uint32_t key = kb + 8U * nt + 2U * t + e;
            const float ksc = __half2float(kscales[key]);
            const uint32_t tok = t0 - kb + key;
            const bool in = tok < last;
            sc_lo[2 * nt + e] = (in && tok < ctx_lo)
                ? static_cast<float>(cfrag[e]) * qs_lo * ksc * inv_sqrt : kNegInf;
            sc_hi[2 * nt + e] = (in && tok < ctx_hi)
                ? static_cast<float>(cfrag[2 + e]) * qs_hi * ksc * inv_sqrt : kNegInf;
          }
        }
        // ---- online softmax per row (a row's 32 keys live in the 4 lanes of a quad)
        float tmax_lo = sc_lo[0], tmax_hi = sc_hi[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) { tmax_lo = fmaxf(tmax_lo, sc_lo[i]); tmax_hi = fmaxf(tmax_hi, sc_hi[i]); }
        tmax_lo = quad_max(tmax_lo);
        tmax_hi = quad_max(tmax_hi);
        const float next_lo = fmaxf(m_lo, tmax_lo), next_hi = fmaxf(m_hi, tmax_hi);
        const float prev_lo = m_lo == kNegInf ? 0.0F : expf(m_lo - next_lo);
        const float prev_hi = m_hi == kNegInf ? 0.0F : expf(m_hi - next_hi);
        float w_lo[8], w_hi[8];
        double ts_lo = 0.0, ts_hi = 0.0;
        float wmax_lo = 0.0F, wmax_hi = 0.0F;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t key = kb + 8U * (i >> 1) + 2U * t + (i & 1);
          const float vsc = __half2float(vscales[key]);
          const float p_lo = sc_lo[i] == kNegInf ? 0.0F : expf(sc_lo[i] - next_lo);
          const float p_hi = sc_hi[i] == kNegInf ? 0.0F : expf(sc_hi[i] - next_hi);
          ts_lo += static_cast<double>(p_lo);
          ts_hi += static_cast<double>(p_hi);
          w_lo[i] = sc_lo[i] == kNegInf ? 0.0F : p_lo * vsc;
          w_hi[i] = sc_hi[i] == kNegInf ? 0.0F : p_hi * vsc;
          wmax_lo = fmaxf(wmax_lo, w_lo[i]);
          wmax_hi = fmaxf(wmax_hi, w_hi[i]);
        }
        ts_lo = quad_sum(ts_lo);
        ts_hi = quad_sum(ts_hi);
        wmax_lo = quad_max(wmax_lo);
        wmax_hi = quad_max(wmax_hi);
        const float ps_lo = fmaxf(wmax_lo / 127.0F, 0x1p-24F), ps_hi = fmaxf(wmax_hi / 127.0F, 0x1p-24F);
        sum_lo = sum_lo * prev_lo + static_cast<float>(ts_lo);
        sum_hi = sum_hi * prev_hi + static_cast<float>(ts_hi);
        m_lo = next_lo;
        m_hi = next_hi;
        // A fragments of P: slots 4t..4t+3 = keys {2t, 2t+1, 8+2t, 9+2t}; slots 16+4t.. = keys {16+2t, ..}
        uint32_t pa[4] = {0U, 0U, 0U, 0U};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t q_lo = static_cast<uint32_t>(max(0, min(127, __float2int_rn(w_lo[i] / ps_lo))));
          const uint32_t q_hi = static_cast<uint32_t>(max(0, min(127, __float2int_rn(w_hi[i] / ps_hi))));
          pa[(i >> 2) * 2] |= q_lo << (8 * (i & 3));
          pa[(i >> 2) * 2 + 1] |= q_hi << (8 * (i & 3));
        }
        // ---- O += P V: B column = 8-dim chunk (g, g+8), k slots = the same key order as P
        const float psl = ps_lo * 0.0625F, psh = ps_hi * 0.0625F;  // V bytes carry 16*code
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t bl[2][4], bh[2][4];
#pragma unroll
          for (int set = 0; set < 2; ++set) {
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t key = kb + 16U * set + 8U * (i >> 1) + 2U * t + (i & 1);
              const uint32_t w = *reinterpret_cast<const uint32_t*>(vcodes + key * (HD / 2U) + 4U * (g + 8U * h));
              lo[i] = (w << 4U) & 0xf0f0f0f0U;  // dims 0,2,4,6 of the chunk
              hi[i] = w & 0xf0f0f0f0U;          // dims 1,3,5,7
            }
            uint32_t x0 = __byte_perm(lo[0], lo[1], 0x5140), x1 = __byte_perm(lo[2], lo[3], 0x5140);
            uint32_t x2 = __byte_perm(lo[0], lo[1], 0x7362), x3 = __byte_perm(lo[2], lo[3], 0x7362);
            bl[set][0] = __byte_perm(x0, x1, 0x5410); bl[set][1] = __byte_perm(x0, x1, 0x7632);
            bl[set][2] = __byte_perm(x2, x3, 0x5410); bl[set][3] = __byte_perm(x2, x3, 0x7632);
            x0 = __byte_perm(hi[0], hi[1], 0x5140); x1 = __byte_perm(hi[2], hi[3], 0x5140);
            x2 = __byte_perm(hi[0], hi[1], 0x7362); x3 = __byte_perm(hi[2], hi[3], 0x7362);
            bh[set][0] = __byte_perm(x0, x1, 0x5410); bh[set][1] = __byte_perm(x0, x1, 0x7632);
            bh[set][2] = __byte_perm(x2, x3, 0x5410); bh[set][3] = __byte_perm(x2, x3, 0x7632);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            int cfrag[4] = {0, 0, 0, 0};
            const uint32_t b0 = (j & 1) ? bh[0][j >> 1] : bl[0][j >> 1];
            const uint32_t b1 = (j & 1) ? bh[1][j >> 1] : bl[1][j >> 1];
            mma_s8(cfrag, pa[0], pa[1], pa[2], pa[3], b0, b1);
            // x * 1.0f is x: the rescale is skipped once the running maximum has settled
            if (prev_lo != 1.0F) { out[h][j][0] *= prev_lo; out[h][j][1] *= prev_lo; }
            if (prev_hi != 1.0F) { out[h][j][2] *= prev_hi; out[h][j][3] *= prev_hi; }
            out[h][j][0] = fmaf(static_cast<float>(cfrag[0]), psl, out[h][j][0]);
            out[h][j][1] = fmaf(static_cast<float>(cfrag[1]), psl, out[h][j][1]);
            out[h][j][2] = fmaf(static_cast<float>(cfrag[2]), psh, out[h][j][2]);
            out[h][j][3] = fmaf(static_cast<float>(cfrag[3]), psh, out[h][j][3]);
          }
        }
      }
    }
    // this warp is done with stage s
    __syncwarp();
    if (lane == 0U) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&empty_bar[s])) : "memory");
    if (tid == 0U && c + kStages < chunks) {
      ok = wait_parity(&empty_bar[s], (c / kStages) & 1U, abort_flag);
      if (ok) issue(c + kStages);
    }
    ok = __shfl_sync(0xffffffffU, ok ? 1 : 0, 0) != 0;
  }
  if (*abort_flag) {
    if (tid == 0U && error) atomicExch(error, 200U);
    return;
  }
  if (!warp_active) return;
  // ---- partials: C column n = 2t+e is chunk n (+8h) -> dim 8*(n+8h) + j
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t mr = (e >= 2) ? row_hi : row_lo;
        if (mr >= MR) continue;
        const uint32_t d = 8U * ((2U * t + (e & 1)) + 8U * h) + j;
        const uint32_t row = mr / group, head = kvh * group + mr % group;
        const size_t pidx = (static_cast<size_t>(row) * a.max_splits + split) * a.q_heads + head;
        part.outputs[pidx * HD + d] = out[h][j][e];
        if (d == 0U) {
          part.maxima[pidx] = (e >= 2) ? m_hi : m_lo;
          part.sums[pidx] = (e >= 2) ? sum_hi : sum_lo;
        }
      }
}

int launch_attention_q4h_pipelined(const AttentionArgs& a, float* maxima, float* sums, float* outputs,
                                   uint32_t* error, cudaStream_t stream) {
  Q4hPartials part{maxima, sums, outputs};
  attention_q4h_pipelined_kernel<<<dim3(a.kv_heads, a.max_splits), 64, 0, stream>>>(a, part, error);
  return check_launch("attention_q4h");
}

}  // namespace qllm
