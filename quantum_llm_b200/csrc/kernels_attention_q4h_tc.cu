// Flash-decode attention over the Q4H cache on the 5th-generation tensor cores (sm_100a):
// both products are tcgen05.mma.kind::i8 with the accumulators in tensor memory, head_dim 128.
//
// CTA = (kv head, context split).  The matrix rows (verify row x grouped query head, at most 32)
// are replicated into the four 32-lane quadrants of the 128-row MMA, and quadrant w owns keys
// 32w..32w+31 of every 128-key tile: a thread is one (quadrant, matrix row) pair, it finds its
// row's 32 scores of the tile in its own tensor-memory lane, and every reduction of the online
// softmax is thread-local -- no shuffles, no shared-memory exchange.
//
// Per tile of 128 keys:
//   1. the producer thread has the tile's records (K codes, V codes, scales: 16.5 KB, contiguous
//      per kv head inside a page) in a two-stage ring of bulk asynchronous copies;
//   2. the 128 compute threads expand the 4-bit codes to INT8 operands in shared memory, one
//      mask/shift per 4 codes (byte = 16 * code; the 1/16 rides on the scales): K as the K-major
//      B operand of Q.K^T, V as an MN-major B operand of P.V -- both are "one key per 128-byte
//      row", so nothing is transposed;
//   3. S[128 x 128] = Qrep . K^T (4 MMAs of k = 32) into tensor memory; a thread reads the 32
//      columns of its quadrant, applies the query / key scales and the causal mask, updates its
//      running maximum and sum, and quantises P * v-scale to INT8 with one scale per row and
//      32 keys -- the arithmetic of the reference kernel
//      (runtime/src/cuda/transformer_kernels.cu:4421-4976), written into its row of a
//      block-diagonal A operand (quadrant w: key columns 32w..32w+31, zero elsewhere);
//   4. O[128 x 128] = Pdiag . V (4 MMAs): lane (w, r) receives exactly the product of its own 32
//      keys; the thread reads its 128 integer sums and accumulates them, scaled, in registers.
// At the end the four quadrants of a row are merged through shared memory and the split's
// partial (maximum, sum, 128 outputs) goes to the workspace for the combine kernel.
//
// Every wait is bounded and reports through the error word; tensor memory is freed on every path.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace qllm {

namespace {

constexpr uint32_t HD = 128;
constexpr uint32_t kTile = 128;                          // keys per tile
constexpr uint32_t kOperandBytes = 128U * 128U;          // one INT8 operand tile
constexpr uint32_t kCodeBytes = kTile * HD / 2U;         // 8192
constexpr uint32_t kScaleBytes = kTile * 2U;             // 256
constexpr uint32_t kRawBytes = 2U * kCodeBytes + 2U * kScaleBytes;  // 16896
constexpr uint32_t kRawStages = 2;
constexpr uint32_t kSmemBytes = 4U * kOperandBytes + kRawStages * kRawBytes + 1024U;
constexpr uint32_t kComputeThreads = 128;
constexpr uint32_t kThreads = kComputeThreads + 32U;     // + one control warp (copies, MMA issue)
constexpr uint32_t kSpin = 1U << 20;
constexpr uint32_t kNib = 0xf0f0f0f0U;
constexpr uint32_t kTmemCols = 256;                      // S: 128 columns, O: 128 columns
constexpr float kMagic = 12582912.0F;                    // 1.5 * 2^23

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
__device__ __forceinline__ void arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void bulk(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(s32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(s32(bar)) : "memory");
}
// 128-byte rows, 8-row groups 1024 bytes apart, 16-byte chunks XOR-swizzled with the row index
// (the 128B swizzle of the UMMA shared-memory descriptors).
__device__ __forceinline__ uint32_t tile_offset(uint32_t row, uint32_t chunk) {
  return (row >> 3U) * 1024U + (row & 7U) * 128U + ((chunk ^ (row & 7U)) << 4U);
}
// K-major operand (k runs along the 128-byte row): a k step of 32 bytes is +32 on the address.
// MN-major operand (m/n runs along the row, 8 k values per 1024-byte group): a k step of 32 is
// +4096.  Both: stride between 8-row groups 1024 bytes, 128B swizzle, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3ffffU) >> 4U);
  d |= static_cast<uint64_t>(1024U >> 4U) << 16U;   // leading byte offset (one 128-wide atom: not stepped)
  d |= static_cast<uint64_t>(1024U >> 4U) << 32U;   // stride byte offset
  d |= static_cast<uint64_t>(1U) << 46U;
  d |= static_cast<uint64_t>(2U) << 61U;            // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
// 32 consecutive columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_low_bytes(float a, float b, float c, float d) {
  const uint32_t ab = __byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040);
  const uint32_t cd = __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}
// position p (0..127) inside an operand row <-> head dimension: within each group of 32, the
// 16 even dimensions come first (that is how one mask/shift per word expands the nibbles)
__device__ __forceinline__ uint32_t dim_of_position(uint32_t p) {
  const uint32_t q = p & 31U;
  return (p & ~31U) + (q < 16U ? 2U * q : 2U * (q - 16U) + 1U);
}
// 128 records of 64 code bytes -> INT8 operand tile, one record per 128-byte row
__device__ __forceinline__ void expand_codes(const uint8_t* raw, uint8_t* tile, uint32_t tid) {
#pragma unroll
  for (uint32_t u = 0; u < 4U; ++u) {
    const uint32_t item = tid + kComputeThreads * u;
    const uint32_t key = item >> 2U, g = item & 3U;
    const uint4 w = *reinterpret_cast<const uint4*>(raw + key * 64U + g * 16U);
    const uint4 even = make_uint4((w.x << 4U) & kNib, (w.y << 4U) & kNib, (w.z << 4U) & kNib, (w.w << 4U) & kNib);
    const uint4 odd = make_uint4(w.x & kNib, w.y & kNib, w.z & kNib, w.w & kNib);
    *reinterpret_cast<uint4*>(tile + tile_offset(key, 2U * g)) = even;
    *reinterpret_cast<uint4*>(tile + tile_offset(key, 2U * g + 1U)) = odd;
  }
}

struct TcPartials {
  float* maxima;
  float* sums;
  float* outputs;
};

__global__ void __launch_bounds__(kThreads, 2)
attention_q4h_tc_kernel(AttentionArgs a, TcPartials part, uint32_t* error) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t raw_full[kRawStages], raw_free[kRawStages], expanded, s_full, p_ready, o_full,
      merge_a, merge_b;
  __shared__ uint32_t tmem_slot, abort_word;
  pdl_trigger();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023U) & ~uintptr_t(1023));
  uint8_t* a_q = smem;                         // Qrep        [128 x 128] K-major
  uint8_t* b_k = smem + kOperandBytes;         // K tile      [128 keys x 128] K-major
  uint8_t* b_v = smem + 2U * kOperandBytes;    // V tile      [128 keys x 128] MN-major
  uint8_t* a_p = smem + 3U * kOperandBytes;    // Pdiag       [128 x 128 keys] K-major
  uint8_t* ring = smem + 4U * kOperandBytes;   // raw records, kRawStages x kRawBytes
  const uint32_t tid = threadIdx.x, warp = tid >> 5U, lane = tid & 31U;
  const uint32_t kvh = blockIdx.x, split = blockIdx.y;
  const uint32_t group = a.q_heads / a.kv_heads;
  const uint32_t MR = a.rows * group;
  volatile uint32_t* abort_flag = &abort_word;

  if (tid == 0U) {
    for (uint32_t s = 0; s < kRawStages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&raw_full[s])), "r"(1U));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&raw_free[s])), "r"(kComputeThreads));
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&expanded)), "r"(kComputeThreads));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&p_ready)), "r"(kComputeThreads));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&merge_a)), "r"(kComputeThreads));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&merge_b)), "r"(kComputeThreads));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&s_full)), "r"(1U));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&o_full)), "r"(1U));
    abort_word = 0U;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4U) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(&tmem_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // static operands: Pdiag is zero outside the quadrant blocks, Qrep is filled below
  for (uint32_t i = tid; i < kOperandBytes / 16U; i += kThreads)
    reinterpret_cast<uint4*>(a_p)[i] = make_uint4(0U, 0U, 0U, 0U);
  pdl_wait();  // queries and the newest records come from the kernels before this one
  const uint32_t first_ctx = *a.first_position + a.position_offset + 1U;
  const uint32_t total = first_ctx + a.rows - 1U;
  const uint32_t first = split * a.split_tokens;
  const bool active = first < total;   // uniform over the CTA
  const uint32_t last = active ? min(total, first + a.split_tokens) : first;
  const uint32_t tiles = active ? (last - first + kTile - 1U) / kTile : 0U;
  const uint32_t pt = a.page_tokens;
  const size_t records = static_cast<size_t>(pt) * a.kv_heads;

  // Qrep: thread (row r = tid % 32, 32-dimension group g = tid / 32) permutes one 32-byte piece of an
  // INT8 query row and stores it into the same place of all four quadrants
  float qscale = 0.0F;
  if (tid < kComputeThreads) {
    const uint32_t r = tid & 31U, g = tid >> 5U;
    uint4 lo = make_uint4(0U, 0U, 0U, 0U), hi = lo;
    if (r < MR && active) {
      const size_t item = static_cast<size_t>(r / group) * a.q_heads + kvh * group + r % group;
      const uint4* src = reinterpret_cast<const uint4*>(a.query_q8 + item * HD + 32U * g);
      lo = src[0];
      hi = src[1];
      qscale = a.query_q8_scale[item];
    }
    const uint4 even = make_uint4(__byte_perm(lo.x, lo.y, 0x6420), __byte_perm(lo.z, lo.w, 0x6420),
                                  __byte_perm(hi.x, hi.y, 0x6420), __byte_perm(hi.z, hi.w, 0x6420));
    const uint4 odd = make_uint4(__byte_perm(lo.x, lo.y, 0x7531), __byte_perm(lo.z, lo.w, 0x7531),
                                 __byte_perm(hi.x, hi.y, 0x7531), __byte_perm(hi.z, hi.w, 0x7531));
#pragma unroll
    for (uint32_t w = 0; w < 4U; ++w) {
      *reinterpret_cast<uint4*>(a_q + tile_offset(32U * w + r, 2U * g)) = even;
      *reinterpret_cast<uint4*>(a_q + tile_offset(32U * w + r, 2U * g + 1U)) = odd;
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_s = tmem_slot, tmem_o = tmem_slot + 128U;

  if (warp == 4U) {
    // ------------------------------------------------------------ control warp
    if (lane == 0U && active) {
      auto issue = [&](uint32_t tile) {
        const uint32_t s = tile % kRawStages;
        const uint32_t tok = first + tile * kTile;
        const uint8_t* layer = a.page_table[tok / pt] + a.layer_offset;
        const size_t rec = static_cast<size_t>(kvh) * pt + tok % pt;
        const uint8_t* kc = layer + rec * (HD / 2U);
        const uint8_t* ks = layer + records * (HD / 2U) + rec * 2U;
        const uint8_t* vc = layer + records * (HD / 2U) + records * 2U + rec * (HD / 2U);
        const uint8_t* vs = layer + records * (HD / 2U) * 2U + records * 2U + rec * 2U;
        uint8_t* dst = ring + s * kRawBytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&raw_full[s])), "r"(kRawBytes)
                     : "memory");
        bulk(dst, kc, kCodeBytes, &raw_full[s]);
        bulk(dst + kCodeBytes, vc, kCodeBytes, &raw_full[s]);
        bulk(dst + 2U * kCodeBytes, ks, kScaleBytes, &raw_full[s]);
        bulk(dst + 2U * kCodeBytes + kScaleBytes, vs, kScaleBytes, &raw_full[s]);
      };
      for (uint32_t t = 0; t < min(tiles, kRawStages); ++t) issue(t);
      // M = 128, N = 128, signed 8-bit operands, 32-bit integer accumulator; P.V takes V as an
      // MN-major B operand (bit 16)
      const uint32_t idesc_qk = (2U << 4U) | (1U << 7U) | (1U << 10U) | ((128U >> 3U) << 17U) | ((128U >> 4U) << 24U);
      const uint32_t idesc_pv = idesc_qk | (1U << 16U);
      for (uint32_t t = 0; t < tiles; ++t) {
        if (!wait_parity(&expanded, t & 1U, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (uint32_t kb = 0; kb < 4U; ++kb)
          mma_i8(tmem_s, umma_desc(s32(a_q) + kb * 32U), umma_desc(s32(b_k) + kb * 32U), idesc_qk, kb > 0U ? 1U : 0U);
        commit(&s_full);
        // the raw stage of this tile is free once every compute thread has expanded its codes and
        // read its scales (that is before it signals p_ready)
        if (t + kRawStages < tiles) {
          if (!wait_parity(&raw_free[t % kRawStages], (t / kRawStages) & 1U, abort_flag)) break;
          issue(t + kRawStages);
        }
        if (!wait_parity(&p_ready, t & 1U, abort_flag)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (uint32_t kb = 0; kb < 4U; ++kb)
          mma_i8(tmem_o, umma_desc(s32(a_p) + kb * 32U), umma_desc(s32(b_v) + kb * 4096U), idesc_pv, kb > 0U ? 1U : 0U);
        commit(&o_full);
      }
    }
  } else if (active) {
    // ------------------------------------------------------------ compute threads
    const uint32_t r = lane;                        // matrix row of this thread
    const bool row_valid = r < MR;
    const uint32_t ctx_row = row_valid ? first_ctx + r / group : 0U;   // keys this row may see
    const float f = qscale * 0.0625F * (1.0F / sqrtf(static_cast<float>(HD)));
    const uint32_t lane_base = (warp * 32U) << 16U;
    float m = kNegInf, sum = 0.0F;
    float acc[HD];
#pragma unroll
    for (uint32_t i = 0; i < HD; ++i) acc[i] = 0.0F;
    bool ok = true;   // kept uniform over the warp: the tensor-memory loads and the vote need all 32 lanes
    for (uint32_t t = 0; t < tiles && ok; ++t) {
      const uint32_t s = t % kRawStages;
      const uint8_t* raw = ring + s * kRawBytes;
      ok = __all_sync(0xffffffffU, wait_parity(&raw_full[s], (t / kRawStages) & 1U, abort_flag));
      if (!ok) break;
      // operands of the previous tile are free: its P.V product has been read (o_full below)
      expand_codes(raw, b_k, tid);
      expand_codes(raw + kCodeBytes, b_v, tid);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      arrive(&expanded);
      // scales of this quadrant's 32 keys (all lanes read the same words)
      const __half2* kw = reinterpret_cast<const __half2*>(raw + 2U * kCodeBytes + warp * 64U);
      const __half2* vw = reinterpret_cast<const __half2*>(raw + 2U * kCodeBytes + kScaleBytes + warp * 64U);
      ok = __all_sync(0xffffffffU, wait_parity(&s_full, t & 1U, abort_flag));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sv[32];
      tmem_ld32(tmem_s + lane_base + 32U * warp, sv);
      const uint32_t tok0 = first + t * kTile + 32U * warp;   // first key of this thread's 32
      const bool all_visible = tok0 + 32U <= min(last, ctx_row);
      float sc[32];
      float tmax = kNegInf;
#pragma unroll
      for (uint32_t j = 0; j < 32U; j += 2U) {
        const float2 k2 = __half22float2(kw[j >> 1U]);
        sc[j] = static_cast<float>(static_cast<int>(sv[j])) * (f * k2.x);
        sc[j + 1U] = static_cast<float>(static_cast<int>(sv[j + 1U])) * (f * k2.y);
        if (!all_visible) {
          if (!(tok0 + j < last && tok0 + j < ctx_row)) sc[j] = kNegInf;
          if (!(tok0 + j + 1U < last && tok0 + j + 1U < ctx_row)) sc[j + 1U] = kNegInf;
        }
        tmax = fmaxf(tmax, fmaxf(sc[j], sc[j + 1U]));
      }
      // kNegInf is the lowest finite float: a first tile gives exp(-huge) = 0, and a row that has
      // seen no visible key yet gives exp(0) = 1 on accumulators that are still zero
      const float next = fmaxf(m, tmax);
      const float prev = __expf(m - next);
      float ts = 0.0F, wmax = 0.0F;
#pragma unroll
      for (uint32_t j = 0; j < 32U; j += 2U) {
        const float2 v2 = __half22float2(vw[j >> 1U]);
        float p0 = __expf(sc[j] - next), p1 = __expf(sc[j + 1U] - next);
        if (!all_visible) {
          if (sc[j] == kNegInf) p0 = 0.0F;
          if (sc[j + 1U] == kNegInf) p1 = 0.0F;
        }
        ts += p0;
        ts += p1;
        sc[j] = p0 * v2.x;         // w = p * v-scale, in place
        sc[j + 1U] = p1 * v2.y;
        wmax = fmaxf(wmax, fmaxf(sc[j], sc[j + 1U]));
      }
      arrive(&raw_free[s]);        // codes expanded, scales read: the stage may be refilled
      const float ps = fmaxf(wmax * (1.0F / 127.0F), 0x1p-24F);
      const float rcp = __fdividef(1.0F, ps);
      sum = sum * prev + ts;
      m = next;
      // INT8 codes of P: fma against 1.5 * 2^23 rounds to nearest even in the low mantissa bits
      uint32_t pw[8];
#pragma unroll
      for (uint32_t i = 0; i < 8U; ++i)
        pw[i] = pack_low_bytes(fmaf(sc[4U * i], rcp, kMagic), fmaf(sc[4U * i + 1U], rcp, kMagic),
                               fmaf(sc[4U * i + 2U], rcp, kMagic), fmaf(sc[4U * i + 3U], rcp, kMagic));
      const uint32_t prow = 32U * warp + r;
      *reinterpret_cast<uint4*>(a_p + tile_offset(prow, 2U * warp)) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      *reinterpret_cast<uint4*>(a_p + tile_offset(prow, 2U * warp + 1U)) = make_uint4(pw[4], pw[5], pw[6], pw[7]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      arrive(&p_ready);
      // rescale while the product runs
      if (__any_sync(0xffffffffU, prev != 1.0F)) {
#pragma unroll
        for (uint32_t i = 0; i < HD; ++i) acc[i] *= prev;
      }
      ok = __all_sync(0xffffffffU, wait_parity(&o_full, t & 1U, abort_flag));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float psl = ps * 0.0625F;   // V bytes carry 16 * code
#pragma unroll
      for (uint32_t c = 0; c < 4U; ++c) {
        uint32_t ov[32];
        tmem_ld32(tmem_o + lane_base + 32U * c, ov);
#pragma unroll
        for (uint32_t j = 0; j < 32U; ++j)
          acc[32U * c + j] = fmaf(static_cast<float>(static_cast<int>(ov[j])), psl, acc[32U * c + j]);
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    // ---- merge the four quadrants of every row through shared memory (the operand tiles are
    // free: every product has been read), then one thread per (row, 32 positions) writes
    // (bounded barriers: a thread whose wait ran out never blocks the others for good)
    arrive(&merge_a);
    ok = ok && wait_parity(&merge_a, 0U, abort_flag) && !*abort_flag;
    if (ok) {
      // every compute thread is past o_full of the last tile: the staging area may overlay a_q .. ring
      float* stage = reinterpret_cast<float*>(smem);        // [4 quadrants][32 rows][132]
      float* mine = stage + (warp * 32U + r) * 132U;
#pragma unroll
      for (uint32_t i = 0; i < HD; i += 4U)
        *reinterpret_cast<float4*>(mine + i) = make_float4(acc[i], acc[i + 1U], acc[i + 2U], acc[i + 3U]);
      mine[128] = m;
      mine[129] = sum;
    }
    arrive(&merge_b);
    ok = ok && wait_parity(&merge_b, 0U, abort_flag) && !*abort_flag;
    if (ok) {
      const float* stage = reinterpret_cast<const float*>(smem);
      const uint32_t quarter = warp;                         // positions 32*quarter .. +31 of row r
      if (row_valid) {
        float mq[4], wq[4];
        float gmax = kNegInf;
#pragma unroll
        for (uint32_t w = 0; w < 4U; ++w) { mq[w] = stage[(w * 32U + r) * 132U + 128U]; gmax = fmaxf(gmax, mq[w]); }
        float gsum = 0.0F;
#pragma unroll
        for (uint32_t w = 0; w < 4U; ++w) {
          wq[w] = __expf(mq[w] - gmax);
          gsum += stage[(w * 32U + r) * 132U + 129U] * wq[w];
        }
        const uint32_t row = r / group, head = kvh * group + r % group;
        const size_t pidx = (static_cast<size_t>(row) * a.max_splits + split) * a.q_heads + head;
        float* dst = part.outputs + pidx * HD;
#pragma unroll 4
        for (uint32_t j = 0; j < 32U; ++j) {
          const uint32_t p = 32U * quarter + j;
          float v = 0.0F;
#pragma unroll
          for (uint32_t w = 0; w < 4U; ++w) v += stage[(w * 32U + r) * 132U + p] * wq[w];
          dst[dim_of_position(p)] = v;
        }
        if (quarter == 0U) {
          part.maxima[pidx] = gmax;
          part.sums[pidx] = gsum;
        }
      }
    }
  }
  if (*abort_flag && tid == 0U && error) atomicExch(error, 210U);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 4U)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_slot), "r"(kTmemCols) : "memory");
}

// INT8 queries for callers that pass FP32 queries only: scale = max(absmax / 127, 2^-24) per
// (row, head), code = rn(q / scale).  One warp per (row, head), head_dim 128.
__global__ void quantize_queries_q8_kernel(const float* query, uint32_t row_stride, uint32_t rows, uint32_t q_heads,
                                           int8_t* q8, float* scales) {
  pdl_trigger();
  pdl_wait();
  const uint32_t item = blockIdx.x * (blockDim.x >> 5U) + (threadIdx.x >> 5U), lane = threadIdx.x & 31U;
  if (item >= rows * q_heads) return;
  const uint32_t row = item / q_heads, head = item % q_heads;
  const float4 v = *reinterpret_cast<const float4*>(query + static_cast<size_t>(row) * row_stride + head * HD + 4U * lane);
  const float amax = warp_max(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  const float sc = fmaxf(amax / 127.0F, 0x1p-24F);
  const float in[4] = {v.x, v.y, v.z, v.w};
  uint32_t packed = 0U;
#pragma unroll
  for (int i = 0; i < 4; ++i)
    packed |= (static_cast<uint32_t>(max(-127, min(127, __float2int_rn(in[i] / sc)))) & 0xffU) << (8 * i);
  *reinterpret_cast<uint32_t*>(q8 + static_cast<size_t>(item) * HD + 4U * lane) = packed;
  if (lane == 0U) scales[item] = sc;
}

}  // namespace

bool attention_q4h_tc_supported(const AttentionArgs& a) {
  const uint32_t group = a.kv_heads ? a.q_heads / a.kv_heads : 0U;
  return a.encoding == QLLM_KV_Q4H && a.head_dim == HD && group && a.rows * group <= 32U && a.tiles <= 1U &&
         a.page_tokens % kTile == 0U && a.split_tokens % kTile == 0U && a.query_row_stride % 4U == 0U;
}

size_t attention_q4h_tc_query_bytes(uint32_t rows, uint32_t q_heads) {
  return static_cast<size_t>(rows) * q_heads * (HD + sizeof(float));
}

// `scratch`: attention_q4h_tc_query_bytes() bytes for the INT8 queries when the caller has none.
int launch_attention_q4h_tc(const AttentionArgs& a, float* maxima, float* sums, float* outputs, uint32_t* error,
                            void* scratch, cudaStream_t stream) {
  AttentionArgs b = a;
  if (!b.query_q8) {
    if (!scratch) return fail(QLLM_INVALID_ARGUMENT, "tensor-memory attention needs INT8 queries or scratch for them");
    int8_t* q8 = static_cast<int8_t*>(scratch);
    float* scales = reinterpret_cast<float*>(q8 + static_cast<size_t>(a.rows) * a.q_heads * HD);
    const uint32_t items = a.rows * a.q_heads;
    count_launch();
    const int rc = check_cuda(launch_pdl(quantize_queries_q8_kernel, dim3((items + 3U) / 4U), dim3(128), 0, stream, a.query,
                                         a.query_row_stride, a.rows, a.q_heads, q8, scales), "quantize_queries_q8");
    if (rc) return rc;
    b.query_q8 = q8;
    b.query_q8_scale = scales;
  }
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (!configured[device & 63]) {
    const int rc = check_cuda(cudaFuncSetAttribute(attention_q4h_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(kSmemBytes)), "tensor-memory attention shared memory opt-in");
    if (rc) return rc;
    configured[device & 63] = true;
  }
  TcPartials part{maxima, sums, outputs};
  return check_cuda(launch_ordered(attention_q4h_tc_kernel, dim3(b.kv_heads, b.max_splits), dim3(kThreads), kSmemBytes,
                                   stream, b, part, error), "attention_q4h_tc");
}

}  // namespace qllm
