// Flash-decode attention over the Q4H (int4 codes + f16 scale per head) paged cache with the
// dequantisation fused into the kernel, head_dim 128.
//
// CTA = (kv head, context split), one warp per 16 matrix rows: warp w owns rows 16w..16w+15
// (matrix row = verify row * group + grouped head, up to 64 = four warps).  K/V codes and scales of 64 keys
// at a time are staged into shared memory by bulk asynchronous copies (the records of one kv
// head are contiguous inside a page) through a 4-stage mbarrier ring, so HBM latency is hidden
// behind the tensor-core work.  Per 32 keys, as in the reference
// (runtime/src/cuda/transformer_kernels.cu:4421-4976): INT8 queries, integer Q.K^T, FP32 online
// softmax, P*v-scale re-quantised to INT8 per row, integer P.V.  Both products are INT8
// m16n8k32 MMAs fed straight from the packed nibbles: a code c is used as the byte 16*c
// (one shift/mask per 8 codes) and the 1/16 is folded into the scale; the k-slot order inside
// an MMA is free as long as A and B agree, so no nibble is ever moved across lanes, and the
// probabilities go from the C fragment of Q.K^T to the A fragment of P.V in registers.
//
// The kernel is bound by instruction issue, not by HBM, so the inner loop is written for a
// low instruction count: exp through ex2.approx, the P quantiser as one fused multiply-add
// against 1.5*2^23 (round to nearest even integer in the low mantissa bits) followed by byte
// permutes, causal masks only in the sub-tiles that can contain an invisible key, and INT8
// queries taken ready-made from the RoPE kernel when the caller provides them.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace qllm {

namespace {

constexpr uint32_t HD = 128;
constexpr uint32_t kChunk = 64;                 // keys per pipeline stage
constexpr uint32_t kStages = 4;
constexpr uint32_t kCodeBytes = kChunk * HD / 2;  // 4096
constexpr uint32_t kScaleBytes = kChunk * 2;      // 128
constexpr uint32_t kStageBytes = 2 * kCodeBytes + 2 * kScaleBytes;
constexpr uint32_t kSpin = 1U << 20;
constexpr uint32_t kFull = 0xffffffffU;
constexpr uint32_t kNibbles = 0xf0f0f0f0U;

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
  v = fmaxf(v, __shfl_xor_sync(kFull, v, 1));
  return fmaxf(v, __shfl_xor_sync(kFull, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(kFull, v, 1);
  return v + __shfl_xor_sync(kFull, v, 2);
}
// low bytes of four floats that hold small integers in their low mantissa bits
__device__ __forceinline__ uint32_t pack_low_bytes(float a, float b, float c, float d) {
  const uint32_t ab = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040);
  const uint32_t cd = __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

// Online-softmax state of one thread: rows g ("lo") and g+8 ("hi") of the warp's 16 matrix
// rows; out[h][j][e] = C fragments of the 16 output tiles.
struct RowState {
  float m_lo, m_hi, sum_lo, sum_hi;
  float out[2][8][4];
};

// One sub-tile of 32 keys at stage offset kb (0 or 32).  tok0 = cache position of its first
// key.  MASKED: some key may lie beyond `last` or beyond a row's causal limit.
template <bool MASKED>
__device__ __forceinline__ void subtile(const uint8_t* kcodes, const uint8_t* vcodes, const __half* kscales,
                                        const __half* vscales, uint32_t kb, uint32_t tok0, uint32_t last,
                                        uint32_t ctx_lo, uint32_t ctx_hi, const uint32_t (&qa)[4][4],
                                        float f_lo, float f_hi, uint32_t g, uint32_t t, RowState& st) {
  // ---- S = Q K^T: 4 key tiles of 8, one 16-byte read per key
  float sc_lo[8], sc_hi[8];
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const uint4 w = *reinterpret_cast<const uint4*>(kcodes + (kb + 8U * nt + g) * (HD / 2U) + 16U * t);
    int cfrag[4] = {0, 0, 0, 0};
    mma_s8(cfrag, qa[0][0], qa[0][1], qa[0][2], qa[0][3], (w.x << 4U) & kNibbles, w.x & kNibbles);
    mma_s8(cfrag, qa[1][0], qa[1][1], qa[1][2], qa[1][3], (w.y << 4U) & kNibbles, w.y & kNibbles);
    mma_s8(cfrag, qa[2][0], qa[2][1], qa[2][2], qa[2][3], (w.z << 4U) & kNibbles, w.z & kNibbles);
    mma_s8(cfrag, qa[3][0], qa[3][1], qa[3][2], qa[3][3], (w.w << 4U) & kNibbles, w.w & kNibbles);
    const float2 ksc = __half22float2(*reinterpret_cast<const __half2*>(kscales + kb + 8U * nt + 2U * t));
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const float k1 = e ? ksc.y : ksc.x;
      float lo = static_cast<float>(cfrag[e]) * (f_lo * k1);
      float hi = static_cast<float>(cfrag[2 + e]) * (f_hi * k1);
      if (MASKED) {
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
  const float next_lo = fmaxf(st.m_lo, tmax_lo), next_hi = fmaxf(st.m_hi, tmax_hi);
  // kNegInf is the lowest finite float: a first tile gives exp(-huge) = 0, and a row that has
  // seen no visible key yet gives exp(0) = 1 on accumulators that are still zero
  const float prev_lo = __expf(st.m_lo - next_lo), prev_hi = __expf(st.m_hi - next_hi);
  float w_lo[8], w_hi[8];
  float ts_lo = 0.0F, ts_hi = 0.0F, wmax_lo = 0.0F, wmax_hi = 0.0F;
#pragma unroll
  for (int nt = 0; nt < 4; ++nt) {
    const float2 vsc = __half22float2(*reinterpret_cast<const __half2*>(vscales + kb + 8U * nt + 2U * t));
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = 2 * nt + e;
      const float v1 = e ? vsc.y : vsc.x;
      float p_lo = __expf(sc_lo[i] - next_lo), p_hi = __expf(sc_hi[i] - next_hi);
      if (MASKED) {
        if (sc_lo[i] == kNegInf) p_lo = 0.0F;
        if (sc_hi[i] == kNegInf) p_hi = 0.0F;
      }
      ts_lo += p_lo;
      ts_hi += p_hi;
      w_lo[i] = p_lo * v1;
      w_hi[i] = p_hi * v1;
      wmax_lo = fmaxf(wmax_lo, w_lo[i]);
      wmax_hi = fmaxf(wmax_hi, w_hi[i]);
    }
  }
  ts_lo = quad_sum(ts_lo);
  ts_hi = quad_sum(ts_hi);
  wmax_lo = quad_max(wmax_lo);
  wmax_hi = quad_max(wmax_hi);
  const float ps_lo = fmaxf(wmax_lo * (1.0F / 127.0F), 0x1p-24F), ps_hi = fmaxf(wmax_hi * (1.0F / 127.0F), 0x1p-24F);
  const float rcp_lo = __fdividef(1.0F, ps_lo), rcp_hi = __fdividef(1.0F, ps_hi);
  st.sum_lo = st.sum_lo * prev_lo + ts_lo;
  st.sum_hi = st.sum_hi * prev_hi + ts_hi;
  st.m_lo = next_lo;
  st.m_hi = next_hi;
  // A fragments of P: slots 4t..4t+3 = keys {2t, 2t+1, 8+2t, 9+2t}; slots 16+4t.. = keys {16+2t, ..}
  constexpr float kMagic = 12582912.0F;  // 1.5 * 2^23
  float c_lo[8], c_hi[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    c_lo[i] = fmaf(w_lo[i], rcp_lo, kMagic);
    c_hi[i] = fmaf(w_hi[i], rcp_hi, kMagic);
  }
  const uint32_t pa0 = pack_low_bytes(c_lo[0], c_lo[1], c_lo[2], c_lo[3]);
  const uint32_t pa1 = pack_low_bytes(c_hi[0], c_hi[1], c_hi[2], c_hi[3]);
  const uint32_t pa2 = pack_low_bytes(c_lo[4], c_lo[5], c_lo[6], c_lo[7]);
  const uint32_t pa3 = pack_low_bytes(c_hi[4], c_hi[5], c_hi[6], c_hi[7]);
  // ---- rescale the accumulators when some row of the warp moved its maximum
  if (__any_sync(kFull, prev_lo != 1.0F || prev_hi != 1.0F)) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        st.out[h][j][0] *= prev_lo; st.out[h][j][1] *= prev_lo;
        st.out[h][j][2] *= prev_hi; st.out[h][j][3] *= prev_hi;
      }
  }
  // ---- O += P V: B column = 8-dim chunk (g, g+8), k slots = the same key order as P
  const float psl = ps_lo * 0.0625F, psh = ps_hi * 0.0625F;  // V bytes carry 16*code
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    // x[set][b]: byte b (= dims 2b, 2b+1 of the chunk) of the four keys of a k-slot group
    uint32_t x[2][4];
#pragma unroll
    for (int set = 0; set < 2; ++set) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t key = kb + 16U * set + 8U * (i >> 1) + 2U * t + (i & 1);
        w[i] = *reinterpret_cast<const uint32_t*>(vcodes + key * (HD / 2U) + 4U * (g + 8U * h));
      }
      const uint32_t y0 = __byte_perm(w[0], w[1], 0x5140), y1 = __byte_perm(w[2], w[3], 0x5140);
      const uint32_t y2 = __byte_perm(w[0], w[1], 0x7362), y3 = __byte_perm(w[2], w[3], 0x7362);
      x[set][0] = __byte_perm(y0, y1, 0x5410); x[set][1] = __byte_perm(y0, y1, 0x7632);
      x[set][2] = __byte_perm(y2, y3, 0x5410); x[set][3] = __byte_perm(y2, y3, 0x7632);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int cfrag[4] = {0, 0, 0, 0};
      const uint32_t b0 = (j & 1) ? (x[0][j >> 1] & kNibbles) : ((x[0][j >> 1] << 4U) & kNibbles);
      const uint32_t b1 = (j & 1) ? (x[1][j >> 1] & kNibbles) : ((x[1][j >> 1] << 4U) & kNibbles);
      mma_s8(cfrag, pa0, pa1, pa2, pa3, b0, b1);
      st.out[h][j][0] = fmaf(static_cast<float>(cfrag[0]), psl, st.out[h][j][0]);
      st.out[h][j][1] = fmaf(static_cast<float>(cfrag[1]), psl, st.out[h][j][1]);
      st.out[h][j][2] = fmaf(static_cast<float>(cfrag[2]), psh, st.out[h][j][2]);
      st.out[h][j][3] = fmaf(static_cast<float>(cfrag[3]), psh, st.out[h][j][3]);
    }
  }
}

}  // namespace

struct Q4hPartials {
  float* maxima;
  float* sums;
  float* outputs;
};

template <bool kTiled>  // grid z = row tile of a wide pass
__global__ void __launch_bounds__(128)
attention_q4h_pipelined_kernel(AttentionArgs a, Q4hPartials part, uint32_t* error) {
  __shared__ __align__(128) uint8_t ring[kStages][kStageBytes];
  // staging of in-kernel quantised queries (callers without ready-made INT8 queries): lives in
  // the last pipeline stage, which is not filled before the queries are in registers
  int8_t (*qs)[HD + 16] = reinterpret_cast<int8_t (*)[HD + 16]>(&ring[kStages - 2U][0]);
  float* qscale_s = reinterpret_cast<float*>(&ring[kStages - 2U][64U * (HD + 16U)]);
  static_assert(64U * (HD + 16U) + 64U * sizeof(float) <= 2U * kStageBytes, "query staging must fit two stages");
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ uint32_t abort_word;
  pdl_trigger();  // the combine kernel may be scheduled; it waits for this grid
  pdl_wait();     // queries and the newest records come from the RoPE kernel before this one
  if constexpr (kTiled) attention_row_tile(a, part);
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
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&empty_bar[s])), "r"(blockDim.x >> 5U));
    }
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const uint32_t row_lo = 16U * warp + g, row_hi = row_lo + 8U;
  // A fragments of the queries: for k-step ks this thread's k slots carry dims 8*(4t+ks)+{0..7}
  uint32_t qa[4][4];
  float qscale_lo, qscale_hi;
  if (a.query_q8) {
    // ready-made INT8 queries [rows, q_heads, HD] and scales [rows, q_heads]
    __syncthreads();  // barrier initialisation
    uint4 lo[2] = {}, hi[2] = {};
    qscale_lo = qscale_hi = 0.0F;
    if (row_lo < MR) {
      const size_t item = static_cast<size_t>(row_lo / group) * a.q_heads + kvh * group + row_lo % group;
      const uint4* src = reinterpret_cast<const uint4*>(a.query_q8 + item * HD + 32U * t);
      lo[0] = src[0]; lo[1] = src[1];
      qscale_lo = a.query_q8_scale[item];
    }
    if (row_hi < MR) {
      const size_t item = static_cast<size_t>(row_hi / group) * a.q_heads + kvh * group + row_hi % group;
      const uint4* src = reinterpret_cast<const uint4*>(a.query_q8 + item * HD + 32U * t);
      hi[0] = src[0]; hi[1] = src[1];
      qscale_hi = a.query_q8_scale[item];
    }
    const uint32_t lw[8] = {lo[0].x, lo[0].y, lo[0].z, lo[0].w, lo[1].x, lo[1].y, lo[1].z, lo[1].w};
    const uint32_t hw[8] = {hi[0].x, hi[0].y, hi[0].z, hi[0].w, hi[1].x, hi[1].y, hi[1].z, hi[1].w};
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      qa[ks][0] = __byte_perm(lw[2 * ks], lw[2 * ks + 1], 0x6420);  // even dims -> slots 4t..4t+3
      qa[ks][1] = __byte_perm(hw[2 * ks], hw[2 * ks + 1], 0x6420);
      qa[ks][2] = __byte_perm(lw[2 * ks], lw[2 * ks + 1], 0x7531);  // odd dims -> slots 16+4t..
      qa[ks][3] = __byte_perm(hw[2 * ks], hw[2 * ks + 1], 0x7531);
    }
  } else {
    // quantise this warp's 16 matrix rows here (lane owns 4 dims)
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
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      const uint2 lo = *reinterpret_cast<const uint2*>(&qs[row_lo][8U * (4U * t + ks)]);
      const uint2 hi = *reinterpret_cast<const uint2*>(&qs[row_hi][8U * (4U * t + ks)]);
      qa[ks][0] = __byte_perm(lo.x, lo.y, 0x6420);
      qa[ks][1] = __byte_perm(hi.x, hi.y, 0x6420);
      qa[ks][2] = __byte_perm(lo.x, lo.y, 0x7531);
      qa[ks][3] = __byte_perm(hi.x, hi.y, 0x7531);
    }
    qscale_lo = qscale_s[row_lo];
    qscale_hi = qscale_s[row_hi];
    __syncthreads();  // the staging area is about to be reused as a pipeline stage ...
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // ... written by bulk copies
  }

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

  // K bytes carry 16*code: the exact factor 1/16 rides on the query scale
  const float f_lo = qscale_lo * 0.0625F * inv_sqrt, f_hi = qscale_hi * 0.0625F * inv_sqrt;
  const uint32_t ctx_lo = row_lo < MR ? first_ctx + row_lo / group : 0U;
  const uint32_t ctx_hi = row_hi < MR ? first_ctx + row_hi / group : 0U;
  RowState st;
  st.m_lo = st.m_hi = kNegInf;
  st.sum_lo = st.sum_hi = 0.0F;
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) st.out[h][j][e] = 0.0F;
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
        const uint32_t tok0 = first + c * kChunk + sub * 32U;
        if (tok0 >= last) break;
        // every key of the sub-tile is stored and visible to every row (row r sees first_ctx + r keys)
        if (tok0 + 32U <= min(last, first_ctx))
          subtile<false>(kcodes, vcodes, kscales, vscales, sub * 32U, tok0, last, ctx_lo, ctx_hi, qa, f_lo, f_hi, g, t, st);
        else
          subtile<true>(kcodes, vcodes, kscales, vscales, sub * 32U, tok0, last, ctx_lo, ctx_hi, qa, f_lo, f_hi, g, t, st);
      }
    }
    // this warp is done with stage s
    __syncwarp();
    if (lane == 0U) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&empty_bar[s])) : "memory");
    if (tid == 0U && c + kStages < chunks) {
      ok = wait_parity(&empty_bar[s], (c / kStages) & 1U, abort_flag);
      if (ok) issue(c + kStages);
    }
    ok = __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
  }
  if (*abort_flag) {
    if (tid == 0U && error) atomicExch(error, 200U);
    return;
  }
  if (!warp_active) return;
  // ---- partials: C column n = 2t+e is chunk n (+8h) -> dim 8*(n+8h) + j
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const uint32_t mr = half ? row_hi : row_lo;
    if (mr >= MR) continue;
    const uint32_t row = mr / group, head = kvh * group + mr % group;
    const size_t pidx = (static_cast<size_t>(row) * a.max_splits + split) * a.q_heads + head;
    float* dst = part.outputs + pidx * HD;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const uint32_t d0 = 8U * ((2U * t + e) + 8U * h);
        float4 v0, v1;
        v0.x = st.out[h][0][2 * half + e]; v0.y = st.out[h][1][2 * half + e];
        v0.z = st.out[h][2][2 * half + e]; v0.w = st.out[h][3][2 * half + e];
        v1.x = st.out[h][4][2 * half + e]; v1.y = st.out[h][5][2 * half + e];
        v1.z = st.out[h][6][2 * half + e]; v1.w = st.out[h][7][2 * half + e];
        *reinterpret_cast<float4*>(dst + d0) = v0;
        *reinterpret_cast<float4*>(dst + d0 + 4U) = v1;
      }
    if (t == 0U) {
      part.maxima[pidx] = half ? st.m_hi : st.m_lo;
      part.sums[pidx] = half ? st.sum_hi : st.sum_lo;
    }
  }
}

int launch_attention_q4h_pipelined(const AttentionArgs& a, float* maxima, float* sums, float* outputs,
                                   uint32_t* error, cudaStream_t stream) {
  Q4hPartials part{maxima, sums, outputs};
  // Ordinary stream order on purpose: started early, the thousand CTAs of this grid (and, behind
  // them, those of the next GEMVs) sit on the SMs waiting; measured 0.5 ms per step slower.
  const uint32_t mtiles = (a.rows * (a.q_heads / a.kv_heads) + 15U) / 16U;  // one warp per 16 matrix rows
  if (a.tiles > 1U)
    return check_cuda(launch_ordered(attention_q4h_pipelined_kernel<true>, dim3(a.kv_heads, a.max_splits, a.tiles),
                                     dim3(32U * mtiles), 0, stream, a, part, error), "attention_q4h");
  return check_cuda(launch_ordered(attention_q4h_pipelined_kernel<false>, dim3(a.kv_heads, a.max_splits), dim3(32U * mtiles), 0,
                                   stream, a, part, error), "attention_q4h");
}

}  // namespace qllm
