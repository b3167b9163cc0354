// Flash-decode attention over the exact-F16 paged cache, head_dim 128, on F16 tensor cores.
//
// Arithmetic of the reference's exact-F16 path (runtime/src/cuda/transformer_kernels.cu:10215-10476,
// softmax 6610-6665): queries and probabilities rounded to F16, F16 keys/values as stored,
// FP32 accumulation, online softmax over tiles of 32 keys.
//
// Cache layout: [K: page_tokens * kv_heads * head_dim f16][V: ...], token-major, so the record
// of one (token, kv head) is 256 contiguous bytes.  CTA = (kv head, context split), one warp per
// 16-row matrix tile of a kv head (matrix row = verify row * group + grouped head, up to 64).
// A tile of 32 keys is 64 bulk asynchronous copies of 256 bytes (one per record, issued by the
// 32 lanes of warp 0) into rows padded to 272 bytes, which makes every ldmatrix of the tile free
// of bank conflicts; three stages on an mbarrier ring.  No value passes through a conversion:
// K feeds mma.m16n8k16 through ldmatrix, V through ldmatrix.trans.
//
// Records of positions beyond the context are read (and masked) like the others: they must hold
// finite values, which holds for pages that start zeroed and are only written by the KV store.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

#include <cuda_fp16.h>

namespace qllm {

namespace {

constexpr uint32_t HD = 128;
constexpr uint32_t kTile = 32;                  // keys per stage
constexpr uint32_t kStages = 3;
constexpr uint32_t kRecord = HD * 2U;           // 256 bytes in the cache
constexpr uint32_t kRow = kRecord + 16U;        // 272 bytes in shared memory
constexpr uint32_t kHalf = kTile * kRow;        // K (or V) part of a stage
constexpr uint32_t kStageBytes = 2U * kHalf;    // 17408
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
__device__ __forceinline__ void bulk(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&d)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&d)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);  // .x = lo (low half), round to nearest even
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float f16r(float v) { return __half2float(__float2half_rn(v)); }
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(kFull, v, 1));
  return fmaxf(v, __shfl_xor_sync(kFull, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(kFull, v, 1);
  return v + __shfl_xor_sync(kFull, v, 2);
}

}  // namespace

struct F16Partials {
  float* maxima;
  float* sums;
  float* outputs;
};

// grid (kv heads, context splits), block 64; dynamic shared memory kStages * kStageBytes.
template <bool kTiled>  // grid z = row tile of a wide pass
__global__ void __launch_bounds__(128)
attention_f16_mma_kernel(AttentionArgs a, F16Partials part, uint32_t* error) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
  __shared__ uint32_t abort_word;
  pdl_trigger();  // the combine kernel may be scheduled; it waits for this grid
  pdl_wait();     // queries and the newest records come from the RoPE kernel before this one
  if constexpr (kTiled) attention_row_tile(a, part);
  const uint32_t tid = threadIdx.x, warp = tid >> 5U, lane = tid & 31U;
  const uint32_t g = lane >> 2U, t = lane & 3U;
  const uint32_t kvh = blockIdx.x, split = blockIdx.y;
  const uint32_t kv = a.kv_heads, group = a.q_heads / kv;
  const uint32_t MR = a.rows * group;
  const uint32_t first_ctx = *a.first_position + a.position_offset + 1U;
  const uint32_t total = first_ctx + a.rows - 1U;
  const uint32_t first = split * a.split_tokens;
  if (first >= total) return;
  const uint32_t last = min(total, first + a.split_tokens);
  const uint32_t tiles = (last - first + kTile - 1U) / kTile;
  const uint32_t pt = a.page_tokens;
  const size_t v_region = static_cast<size_t>(pt) * kv * kRecord;
  const float inv_sqrt = 1.0F / sqrtf(static_cast<float>(HD));
  volatile uint32_t* abort_flag = &abort_word;
  const uint32_t ring_base = s32(ring);

  if (tid == 0U) {
    for (uint32_t s = 0; s < kStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&full_bar[s])), "r"(1U));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&empty_bar[s])), "r"(blockDim.x >> 5U));
    }
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // warp 0, all lanes: lane l copies the K and the V record of key l of the tile
  auto issue = [&](uint32_t tile) {
    const uint32_t s = tile % kStages;
    if (lane == 0U)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&full_bar[s])),
                   "r"(2U * kTile * kRecord) : "memory");
    __syncwarp();
    const uint32_t tok = first + tile * kTile + lane;
    const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
    const uint8_t* ksrc = layer + (static_cast<size_t>(tok % pt) * kv + kvh) * kRecord;
    const uint32_t dst = ring_base + s * kStageBytes + lane * kRow;
    bulk(dst, ksrc, kRecord, &full_bar[s]);
    bulk(dst + kHalf, ksrc + v_region, kRecord, &full_bar[s]);
  };
  if (warp == 0U)
    for (uint32_t c = 0; c < min(tiles, kStages); ++c) issue(c);

  // A fragments of the F16 queries (k-step ks = dims 16ks .. 16ks+15)
  const uint32_t row_lo = 16U * warp + g, row_hi = row_lo + 8U;
  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) qa[ks][0] = qa[ks][1] = qa[ks][2] = qa[ks][3] = 0U;
  if (row_lo < MR) {
    const float* q = a.query + static_cast<size_t>(row_lo / group) * a.query_row_stride +
                     static_cast<size_t>(kvh * group + row_lo % group) * HD + 2U * t;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const float2 x = *reinterpret_cast<const float2*>(q + 16 * ks);
      const float2 y = *reinterpret_cast<const float2*>(q + 16 * ks + 8);
      qa[ks][0] = pack_f16(x.x, x.y);
      qa[ks][2] = pack_f16(y.x, y.y);
    }
  }
  if (row_hi < MR) {
    const float* q = a.query + static_cast<size_t>(row_hi / group) * a.query_row_stride +
                     static_cast<size_t>(kvh * group + row_hi % group) * HD + 2U * t;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const float2 x = *reinterpret_cast<const float2*>(q + 16 * ks);
      const float2 y = *reinterpret_cast<const float2*>(q + 16 * ks + 8);
      qa[ks][1] = pack_f16(x.x, x.y);
      qa[ks][3] = pack_f16(y.x, y.y);
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
  const bool warp_active = 16U * warp < MR;
  // ldmatrix row of this lane: matrix m = lane / 8, row r = lane % 8
  const uint32_t lm = lane >> 3U, lr = lane & 7U;
  bool ok = true;

  for (uint32_t c = 0; c < tiles && ok; ++c) {
    const uint32_t s = c % kStages;
    ok = wait_parity(&full_bar[s], (c / kStages) & 1U, abort_flag);
    if (!ok) break;
    if (warp_active) {
      const uint32_t kbase = ring_base + s * kStageBytes, vbase = kbase + kHalf;
      const uint32_t tok0 = first + c * kTile;
      const bool masked = tok0 + kTile > min(last, first_ctx);
      // ---- S = Q K^T: per key tile of 8, ldmatrix.x4 = the B fragments of two k-steps
      float sc_lo[8], sc_hi[8];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        float cfrag[4] = {0.0F, 0.0F, 0.0F, 0.0F};
        const uint32_t row_addr = kbase + (8U * nt + lr) * kRow + 16U * lm;
#pragma unroll
        for (int kp = 0; kp < 4; ++kp) {   // dims 32kp .. 32kp+31
          uint32_t b[4];
          ldmatrix_x4(b, row_addr + 64U * kp);
          mma_f16(cfrag, qa[2 * kp], b[0], b[1]);
          mma_f16(cfrag, qa[2 * kp + 1], b[2], b[3]);
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
          p[e] = f16r(p_lo);
          p[2 + e] = f16r(p_hi);
          ts_lo += p[e];
          ts_hi += p[2 + e];
        }
        pa[nt >> 1][(nt & 1) * 2] = pack_f16(p[0], p[1]);
        pa[nt >> 1][(nt & 1) * 2 + 1] = pack_f16(p[2], p[3]);
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
      // ---- O += P V: ldmatrix.x4.trans = the B fragments of two dim tiles for one k-step
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const uint32_t row_addr = vbase + (16U * kk + 8U * (lm & 1U) + lr) * kRow + 16U * (lm >> 1U);
#pragma unroll
        for (int jp = 0; jp < 8; ++jp) {   // dims 16jp .. 16jp+15
          uint32_t b[4];
          ldmatrix_x4_trans(b, row_addr + 32U * jp);
          mma_f16(out[2 * jp], pa[kk], b[0], b[1]);
          mma_f16(out[2 * jp + 1], pa[kk], b[2], b[3]);
        }
      }
    }
    // this warp is done with stage s
    __syncwarp();
    if (lane == 0U) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&empty_bar[s])) : "memory");
    if (warp == 0U && c + kStages < tiles) {
      if (lane == 0U) ok = wait_parity(&empty_bar[s], (c / kStages) & 1U, abort_flag);
      ok = __shfl_sync(kFull, ok ? 1 : 0, 0) != 0;
      if (ok) issue(c + kStages);
    }
  }
  if (*abort_flag) {
    if (tid == 0U && error) atomicExch(error, 400U);
    return;
  }
  if (!warp_active) return;
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

bool attention_f16_mma_supported(const AttentionArgs& a) {
  const uint32_t group = a.kv_heads ? a.q_heads / a.kv_heads : 0U;
  return a.encoding == QLLM_KV_F16 && a.head_dim == HD && a.kv_heads && group && a.rows * group <= 64U &&
         a.page_tokens % kTile == 0U && a.split_tokens % kTile == 0U && a.query_row_stride % 2U == 0U;
}

int launch_attention_f16_mma(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                             cudaStream_t stream) {
  F16Partials part{maxima, sums, outputs};
  constexpr size_t smem = static_cast<size_t>(kStages) * kStageBytes;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device & 63]) {
    cudaError_t e = cudaFuncSetAttribute(attention_f16_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_f16_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
    if (e != cudaSuccess) return check_cuda(e, "F16 attention shared memory opt-in");
    configured[device & 63] = true;
  }
  const uint32_t mtiles = (a.rows * (a.q_heads / a.kv_heads) + 15U) / 16U;  // one warp per 16 matrix rows
  if (a.tiles > 1U)
    return check_cuda(launch_ordered(attention_f16_mma_kernel<true>, dim3(a.kv_heads, a.max_splits, a.tiles),
                                     dim3(32U * mtiles), smem, stream, a, part, error), "attention_f16_mma");
  return check_cuda(launch_ordered(attention_f16_mma_kernel<false>, dim3(a.kv_heads, a.max_splits), dim3(32U * mtiles), smem,
                                   stream, a, part, error), "attention_f16_mma");
}

}  // namespace qllm
