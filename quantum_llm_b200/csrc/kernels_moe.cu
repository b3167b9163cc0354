// Routed mixture of experts in place of the dense FFN (NVFP4 experts, W4A4), decode shapes:
// up to 8 rows x up to 8 selected experts.  Arithmetic of the reference's NVFP4 branch
// (run_router / run_routed_moe, runtime/tools/dense_fp4_provider.cpp:8128-8166, 8207-8248;
// runtime/src/cuda/moe_kernels.cu:171-264, 430-510, 633-690, 759-790; router selection
// runtime/src/cuda/transformer_kernels.cu:2947-3006):
//   router logits (BF16) -> top-K by repeated arg-max, ties to the lower expert id
//   -> softmax over the K selected logits x routed scaling factor, rounded to BF16;
//   per selection: gate = bf16(W1 . fq1(x)), up = bf16(W3 . fq3(x)) (each projection quantises
//   its input with its own activation scale), mid = bf16(silu(gate) * up),
//   out = bf16(W2 . fq2(mid)); moe = bf16(sum over the slots, in slot order, of score * out).
// Three launches per layer: selection, gate/up (which also quantises mid for the down
// projection), down fused with the weighted sum.
// Dot products use the exact block arithmetic of the CUDA-core GEMV (integer block sums, block
// terms summed in double), so the results do not depend on the launch shape.
// Every selected expert's weights are streamed once per selection: the step is bound by
// those bytes (selections x 3 x expert_ffn x hidden x 0.5625).
#include "common.cuh"
#include "fp4_dot.cuh"
#include "fused.h"
#include "kernels.h"
#include "launch.cuh"
#include "moe.h"

namespace qllm {

namespace {

template <int R, int LANES>
__device__ __forceinline__ void rows_dot(const ExpertMatrix& m, uint32_t first_row, uint32_t last_row, uint32_t cols,
                                         const int8_t* xi8, const float* xscale, uint32_t lane_in_group,
                                         double (&acc)[R]);  // defined with the expert projections below

// ---- router: one warp per row -------------------------------------------------------------
// Selection and scores of one row by one warp; logit(e) returns the router logit of expert e.
template <class Logit>
__device__ __forceinline__ void route_row(Logit logit, uint32_t row, uint32_t lane, uint32_t experts, uint32_t top_k,
                                          float route_scale, uint32_t* indices, float* scores) {
  constexpr uint32_t kPerLane = 8;  // up to 256 experts
  float value[kPerLane];
#pragma unroll
  for (uint32_t i = 0; i < kPerLane; ++i) {
    const uint32_t e = lane + 32U * i;
    value[i] = e < experts ? bf16r(logit(e)) : kNegInf;
  }
  uint32_t taken = 0U;  // bit i: this lane's i-th expert is already selected
  float chosen_value[8];
  uint32_t chosen_index[8];
#pragma unroll
  for (uint32_t slot = 0; slot < 8U; ++slot) {
    chosen_value[slot] = -INFINITY;
    chosen_index[slot] = 0xffffffffU;
    if (slot >= top_k) continue;
    float best = -INFINITY;
    uint32_t best_index = 0xffffffffU;
#pragma unroll
    for (uint32_t i = 0; i < kPerLane; ++i) {
      const uint32_t e = lane + 32U * i;
      if (e < experts && !((taken >> i) & 1U) && (value[i] > best || (value[i] == best && e < best_index))) {
        best = value[i];
        best_index = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffU, best, o);
      const uint32_t other_index = __shfl_xor_sync(0xffffffffU, best_index, o);
      if (other > best || (other == best && other_index < best_index)) { best = other; best_index = other_index; }
    }
    chosen_value[slot] = best;
    chosen_index[slot] = best_index;
    if (best_index != 0xffffffffU && (best_index & 31U) == lane) taken |= 1U << (best_index >> 5U);
  }
  // lane `slot` takes that slot's exponential (in double, rounded once: the same FP32 value on
  // the device and in a host check); the sum runs in slot order on every lane
  float top = -INFINITY, my_value = 0.0F;
  uint32_t my_index = 0xffffffffU;
#pragma unroll
  for (uint32_t slot = 0; slot < 8U; ++slot) {
    if (slot < top_k) top = fmaxf(top, chosen_value[slot]);
    if (slot == lane) { my_value = chosen_value[slot]; my_index = chosen_index[slot]; }
  }
  const float mine = lane < top_k ? static_cast<float>(exp(static_cast<double>(my_value - top))) : 0.0F;
  float sum = 0.0F;
#pragma unroll
  for (uint32_t slot = 0; slot < 8U; ++slot) {
    const float term = __shfl_sync(0xffffffffU, mine, slot);
    if (slot < top_k) sum += term;
  }
  if (lane < top_k) {
    float v = mine / sum;
    if (route_scale != 1.0F) v *= route_scale;
    scores[row * top_k + lane] = bf16r(v);
    indices[row * top_k + lane] = my_index;
  }
}

// Selection from a router GEMV result that some earlier kernel left behind.
__global__ void __launch_bounds__(32)
moe_router_select_kernel(GemvOut logits, uint32_t experts, uint32_t top_k, float route_scale, uint32_t* indices,
                         float* scores) {
  pdl_trigger();
  pdl_wait();
  const uint32_t row = blockIdx.x;
  route_row([&](uint32_t e) { return gemv_value(logits, row, e); }, row, threadIdx.x, experts, top_k, route_scale,
            indices, scores);
}

// Router projection and selection in one launch: grid (chunks of 16 experts, rows), 8 warps.
// The row's quantised operand (INT8 values + block scales, written by the norm kernel before) is
// dotted with the experts' router rows, two per warp, with the exact block arithmetic of the
// CUDA-core GEMV (logit = bf16(float(S) * weight_scale / input_scale)).  The CTAs of a row leave
// their logits in the workspace and take a ticket; the last one to arrive selects (every other
// CTA's logits are visible to it: fence before the ticket, fence after).  Replaces a GEMV launch,
// its split-K partials and a selection launch.
constexpr uint32_t kRouterChunk = 16;

__global__ void __launch_bounds__(256)
moe_router_kernel(ExpertMatrix router, const int8_t* xi8, const float* xscale, MoeArgs a) {
  __shared__ uint32_t last;
  pdl_trigger();
  pdl_wait();
  const uint32_t row = blockIdx.y, warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t H = a.hidden, blocks = H / 16U;
  const int8_t* x = xi8 + static_cast<size_t>(row) * H;
  const float* xs = xscale + static_cast<size_t>(row) * blocks;
  float* logits = a.router_logits + static_cast<size_t>(row) * 256U;
  const uint32_t first = blockIdx.x * kRouterChunk + warp * 2U;
  if (first < a.experts) {
    double sum[2];
    rows_dot<2, 32>(router, first, a.experts - 1U, H, x, xs, lane, sum);
#pragma unroll
    for (uint32_t r = 0; r < 2U; ++r)
      if (lane == r && first + r < a.experts)
        logits[first + r] = bf16r(static_cast<float>(sum[r]) * router.weight_scale / router.input_scale);
  }
  __syncthreads();
  if (threadIdx.x == 0U) {
    __threadfence();
    const uint32_t ticket = atomicAdd(a.router_tickets + row, 1U);
    last = ticket == gridDim.x - 1U ? 1U : 0U;
    if (last) {
      a.router_tickets[row] = 0U;  // for the next launch (stream order)
      __threadfence();
    }
  }
  __syncthreads();
  if (last && warp == 0U)
    route_row([&](uint32_t e) { return __ldcg(logits + e); }, row, lane, a.experts, a.route_width, a.route_scale,
              a.indices, a.scores);
}

// ---- shared pieces of the two expert projections ---------------------------------------------
// Quantises 16 FP32 values at `x16` into INT8 + a block scale, stored as block `blk` of the
// destination row.
__device__ __forceinline__ void quantize_block(const float* __restrict__ x16, float g, bool round_bf16, uint32_t blk,
                                               int8_t* xi8, float* xscale) {
  float v[16];
  const float4* in4 = reinterpret_cast<const float4*>(x16);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 t = in4[i];
    v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
  }
  if (round_bf16) {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = bf16r(v[i]);
  }
  uint4 packed;
  float local;
  quantize_block16_i8(v, g, packed, local);
  reinterpret_cast<uint4*>(xi8)[blk] = packed;
  xscale[blk] = local;
}

// Exact sums over the blocks of R consecutive weight rows against one quantised activation row.
// A group of LANES lanes (16 or 32) strides the blocks of its rows; the loads of all R rows are
// issued before the arithmetic.  Every lane of the group returns the full sums.
template <int R, int LANES>
__device__ __forceinline__ void rows_dot(const ExpertMatrix& m, uint32_t first_row, uint32_t last_row, uint32_t cols,
                                         const int8_t* xi8, const float* xscale, uint32_t lane_in_group,
                                         double (&acc)[R]) {
  const uint32_t blocks = cols / 16U;
  const uint2* w[R];
  const uint8_t* s[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint32_t row = min(first_row + r, last_row);  // rows past the end repeat the last one (discarded)
    w[r] = reinterpret_cast<const uint2*>(m.codes + static_cast<size_t>(row) * (cols / 2U));
    s[r] = m.scales + static_cast<size_t>(row) * blocks;
    acc[r] = 0.0;
  }
#pragma unroll 2
  for (uint32_t blk = lane_in_group; blk < blocks; blk += LANES) {
    uint2 codes[R];
    uint8_t scale[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      codes[r] = __ldg(w[r] + blk);
      scale[r] = __ldg(s[r] + blk);
    }
    const uint4 xv = reinterpret_cast<const uint4*>(xi8)[blk];
    const float xs = xscale[blk];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = block16_dot(codes[r], xv);
      // exact: |d| < 2^12, the product of the two E4M3 scales has 8 significant bits
      acc[r] += static_cast<double>(static_cast<float>(d) * (e4m3_value(scale[r]) * xs) * 0.25F);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int o = LANES / 2; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(0xffffffffU, acc[r], o);
  }
}

constexpr uint32_t kGateUpRows = 32;   // mid values per CTA of the gate/up kernel: two quantisation blocks
// shared memory of one slot's quantised mid row in the down kernel (values + scales, 16-byte granules)
__host__ __device__ inline uint32_t down_slot_bytes(uint32_t expert_ffn) {
  return (expert_ffn + expert_ffn / 16U * 4U + 15U) & ~15U;
}
constexpr uint32_t kDownColumns = 16;  // hidden columns per CTA of the down kernel (one warp per slot)

// ---- gate / up / SiLU: grid (ceil(expert_ffn / 32), selections), 8 warps x 4 output rows ----------
// The CTA quantises the selection's input row once per projection (once for both when their
// activation scales agree), every warp streams four gate rows and four up rows, and the CTA's
// 32 mid values leave as two blocks already quantised for the down projection.
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(MoeArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ __align__(16) float mid_tile[kGateUpRows];
  pdl_trigger();
  pdl_wait();
  const uint32_t selection = blockIdx.y, row = selection / a.route_width;
  const uint32_t expert = a.indices[selection];
  if (expert >= a.experts) return;  // the router found no candidate (non-finite logits): contributes nothing
  const uint32_t H = a.hidden, blocks = H / 16U, W = a.expert_ffn;
  const ExpertMatrix G = a.gate[expert], U = a.up[expert];
  const bool shared_input = G.input_scale == U.input_scale;
  int8_t* gi8 = reinterpret_cast<int8_t*>(smem);
  int8_t* ui8 = shared_input ? gi8 : gi8 + H;
  float* gscale = reinterpret_cast<float*>(gi8 + 2U * H);
  float* uscale = shared_input ? gscale : gscale + blocks;
  const float* x = a.x + static_cast<size_t>(row) * a.x_stride;
  for (uint32_t i = threadIdx.x; i < (shared_input ? blocks : 2U * blocks); i += blockDim.x) {
    if (i < blocks) quantize_block(x + 16U * i, G.input_scale, true, i, gi8, gscale);
    else quantize_block(x + 16U * (i - blocks), U.input_scale, true, i - blocks, ui8, uscale);
  }
  __syncthreads();
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t first = blockIdx.x * kGateUpRows + warp * 4U;
  double g[4], u[4];
  rows_dot<4, 32>(G, first, W - 1U, H, gi8, gscale, lane, g);
  rows_dot<4, 32>(U, first, W - 1U, H, ui8, uscale, lane, u);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (lane == static_cast<uint32_t>(r)) {
      const float gate = bf16r(static_cast<float>(g[r]) * G.weight_scale / G.input_scale);
      const float up = bf16r(static_cast<float>(u[r]) * U.weight_scale / U.input_scale);
      mid_tile[warp * 4U + r] = bf16r((gate / (1.0F + det_expf(-gate))) * up);
    }
  }
  __syncthreads();
  const uint32_t out_block = blockIdx.x * (kGateUpRows / 16U) + threadIdx.x;
  if (threadIdx.x < kGateUpRows / 16U && out_block < W / 16U)
    quantize_block(mid_tile + 16U * threadIdx.x, a.down[expert].input_scale, false, out_block,
                   a.mid_i8 + static_cast<size_t>(selection) * W, a.mid_scale + static_cast<size_t>(selection) * (W / 16U));
}

// ---- gate / up / SiLU, weights staged through shared memory ------------------------------------
// grid (CTAs per selection, selections), 8 warps.  A CTA works on ONE selection: it quantises the
// row once, then walks over its share of the selection's 16-row tiles.  The 16 gate rows and the
// 16 up rows of a tile are contiguous in the expert's tensors, so one elected thread brings a
// tile in with four bulk asynchronous copies (codes and scales of each projection, 36 KB at
// hidden 2048) that complete on the stage's mbarrier (two rows of each projection per warp).
// One stage and five CTAs per SM: the kernel spends its time at CTA barriers and on the integer
// pipe, so what pays is occupancy (other CTAs stream and compute meanwhile), not a deeper ring
// inside a CTA (two stages at two CTAs per SM were 10 % slower in the whole step).  The grid is
// sized to one wave.  Needs hidden % 256 == 0 (16-byte granules of the scale rows) and 16-byte
// aligned expert tensors; other shapes use the kernel above.
constexpr uint32_t kStagedRows = 16;
constexpr uint32_t kStagedThreads = 256;
constexpr uint32_t kStagedStages = 1;

__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void bulk_to_shared(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(shared_address(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(shared_address(bar))
               : "memory");
}
// Bounded wait for the phase of `bar` with the given parity; false when the limit ran out.
__device__ __forceinline__ bool wait_phase(uint64_t* bar, uint32_t parity) {
  const uint32_t address = shared_address(bar);
  for (uint32_t spin = 0; spin < (1U << 22U); ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(address), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

// Sums of the blocks of R staged weight rows (row-major codes / scales in shared memory).
template <int R>
__device__ __forceinline__ void staged_rows_dot(const uint8_t* codes, const uint8_t* scales, uint32_t first,
                                                uint32_t cols, const int8_t* xi8, const float* xscale, uint32_t lane,
                                                double (&acc)[R]) {
  const uint32_t blocks = cols / 16U;
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0;
  for (uint32_t blk = lane; blk < blocks; blk += 32U) {
    const uint4 xv = reinterpret_cast<const uint4*>(xi8)[blk];
    const float xs = xscale[blk];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const uint2 w = reinterpret_cast<const uint2*>(codes + static_cast<size_t>(first + r) * (cols / 2U))[blk];
      const int d = block16_dot(w, xv);
      acc[r] += static_cast<double>(static_cast<float>(d) *
                                    (e4m3_value(scales[static_cast<size_t>(first + r) * blocks + blk]) * xs) * 0.25F);
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = warp_sum_f64(acc[r]);
}

__host__ __device__ inline uint32_t staged_stage_bytes(uint32_t hidden) {
  return 2U * kStagedRows * (hidden / 2U + hidden / 16U);
}

__global__ void __launch_bounds__(kStagedThreads, 5)
moe_gate_up_staged_kernel(MoeArgs a, uint32_t* error) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(16) float mid_tile[kStagedRows];
  __shared__ __align__(8) uint64_t bar[kStagedStages];
  pdl_trigger();
  if (threadIdx.x == 0U) {
    for (uint32_t s = 0; s < kStagedStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(&bar[s])), "r"(1U));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();
  const uint32_t selection = blockIdx.y, row = selection / a.route_width;
  const uint32_t H = a.hidden, blocks = H / 16U, W = a.expert_ffn;
  const uint32_t expert = a.indices[selection];
  if (expert >= a.experts) return;  // the router found no candidate (non-finite logits): contributes nothing
  const ExpertMatrix G = a.gate[expert], U = a.up[expert];
  // tiles blockIdx.x, blockIdx.x + gridDim.x, ... of this selection
  const uint32_t tiles = W / kStagedRows;
  const uint32_t mine = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1U) / gridDim.x : 0U;
  const uint32_t stage_bytes = staged_stage_bytes(H);
  const uint32_t code_bytes = kStagedRows * (H / 2U), scale_bytes = kStagedRows * blocks;
  auto issue = [&](uint32_t k) {  // elected thread: tile k of this CTA into stage k % stages
    uint8_t* stage = smem + static_cast<size_t>(k % kStagedStages) * stage_bytes;
    uint64_t* full = &bar[k % kStagedStages];
    const size_t first = static_cast<size_t>(blockIdx.x + k * gridDim.x) * kStagedRows;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(full)), "r"(stage_bytes)
                 : "memory");
    bulk_to_shared(stage, G.codes + first * (H / 2U), code_bytes, full);
    bulk_to_shared(stage + code_bytes, U.codes + first * (H / 2U), code_bytes, full);
    bulk_to_shared(stage + 2U * code_bytes, G.scales + first * blocks, scale_bytes, full);
    bulk_to_shared(stage + 2U * code_bytes + scale_bytes, U.scales + first * blocks, scale_bytes, full);
  };
  if (threadIdx.x == 0U)
    for (uint32_t k = 0; k < min(mine, kStagedStages); ++k) issue(k);
  // the row, quantised once per projection (once for both when their activation scales agree)
  const float* x = a.x + static_cast<size_t>(row) * a.x_stride;
  const bool shared_input = G.input_scale == U.input_scale;
  int8_t* gi8 = reinterpret_cast<int8_t*>(smem + static_cast<size_t>(kStagedStages) * stage_bytes);
  int8_t* ui8 = shared_input ? gi8 : gi8 + H;
  float* gscale = reinterpret_cast<float*>(gi8 + 2U * H);
  float* uscale = shared_input ? gscale : gscale + blocks;
  for (uint32_t i = threadIdx.x; i < (shared_input ? blocks : 2U * blocks); i += kStagedThreads) {
    if (i < blocks) quantize_block(x + 16U * i, G.input_scale, true, i, gi8, gscale);
    else quantize_block(x + 16U * (i - blocks), U.input_scale, true, i - blocks, ui8, uscale);
  }
  __syncthreads();
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const float down_scale = a.down[expert].input_scale;
  for (uint32_t k = 0; k < mine; ++k) {
    const uint8_t* stage = smem + static_cast<size_t>(k % kStagedStages) * stage_bytes;
    if (!wait_phase(&bar[k % kStagedStages], (k / kStagedStages) & 1U)) {
      // the copies did not complete within the limit: report and leave (uniform: every thread waits
      // on the same barrier; nothing of this CTA is in flight into a stage it will touch again)
      if (threadIdx.x == 0U && error != nullptr) atomicExch(error, 400U);
      return;
    }
    double g[2], u[2];
    staged_rows_dot<2>(stage, stage + 2U * code_bytes, warp * 2U, H, gi8, gscale, lane, g);
    staged_rows_dot<2>(stage + code_bytes, stage + 2U * code_bytes + scale_bytes, warp * 2U, H, ui8, uscale, lane, u);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (lane == static_cast<uint32_t>(r)) {
        const float gate = bf16r(static_cast<float>(g[r]) * G.weight_scale / G.input_scale);
        const float up = bf16r(static_cast<float>(u[r]) * U.weight_scale / U.input_scale);
        mid_tile[warp * 2U + r] = bf16r((gate / (1.0F + det_expf(-gate))) * up);
      }
    }
    __syncthreads();  // the stage is free, mid_tile is complete
    if (threadIdx.x == 0U && k + kStagedStages < mine) issue(k + kStagedStages);
    if (threadIdx.x == 32U)
      quantize_block(mid_tile, down_scale, false, blockIdx.x + k * gridDim.x,
                     a.mid_i8 + static_cast<size_t>(selection) * W, a.mid_scale + static_cast<size_t>(selection) * (W / 16U));
    __syncthreads();  // mid_tile may be overwritten
  }
}

// ---- down + ordered weighted sum: grid (ceil(hidden / 16), rows), warp = slot ---------------------
// Warp `slot` streams 16 rows of its slot's down projection against that slot's quantised mid row
// (LANES = 16: a half warp per row, LANES = 32 when that leaves no lane idle); 16 threads then add
// score * out over the slots in slot order.
template <int LANES>
__global__ void __launch_bounds__(256)
moe_down_kernel(MoeArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ float out_tile[8][kDownColumns];
  pdl_trigger();
  pdl_wait();
  constexpr uint32_t kGroups = 32U / LANES, kRows = 4U;  // kGroups * kRows columns per pass of a warp
  const uint32_t row = blockIdx.y, W = a.expert_ffn, blocks = W / 16U, K = a.route_width;
  const uint32_t slot = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  if (slot < K) {
    const uint32_t selection = row * K + slot;
    const uint32_t expert = a.indices[selection];
    if (expert < a.experts) {
      int8_t* mi8 = reinterpret_cast<int8_t*>(smem) + static_cast<size_t>(slot) * down_slot_bytes(W);
      float* mscale = reinterpret_cast<float*>(mi8 + W);
      const uint4* src = reinterpret_cast<const uint4*>(a.mid_i8 + static_cast<size_t>(selection) * W);
      const float* src_scale = a.mid_scale + static_cast<size_t>(selection) * blocks;
      for (uint32_t i = lane; i < blocks; i += 32U) {
        reinterpret_cast<uint4*>(mi8)[i] = src[i];
        mscale[i] = src_scale[i];
      }
      __syncwarp();
      const ExpertMatrix D = a.down[expert];
      const uint32_t group = lane / LANES, lane_in_group = lane % LANES;
#pragma unroll
      for (uint32_t pass = 0; pass < kDownColumns / (kGroups * kRows); ++pass) {
        const uint32_t local = pass * kGroups * kRows + group * kRows;
        double t[kRows];
        rows_dot<kRows, LANES>(D, blockIdx.x * kDownColumns + local, a.hidden - 1U, W, mi8, mscale, lane_in_group, t);
#pragma unroll
        for (uint32_t r = 0; r < kRows; ++r)
          if (lane_in_group == r) out_tile[slot][local + r] = bf16r(static_cast<float>(t[r]) * D.weight_scale / D.input_scale);
      }
    } else if (lane < kDownColumns) {
      out_tile[slot][lane] = 0.0F;  // no candidate: contributes score * 0
    }
  }
  __syncthreads();
  const uint32_t column = blockIdx.x * kDownColumns + threadIdx.x;
  if (threadIdx.x < kDownColumns && column < a.hidden) {
    float total = 0.0F;
    for (uint32_t s = 0; s < K; ++s) {
      const float contribution = a.scores[row * K + s] * out_tile[s][threadIdx.x];
      total = total + contribution;
    }
    a.moe[static_cast<size_t>(row) * a.hidden + column] = bf16r(total);
  }
}

// ---- down + ordered weighted sum, weights staged through shared memory -------------------------
// grid (CTAs per row, rows), warp = slot.  A CTA works on ONE row: every warp keeps its slot's
// quantised mid row in shared memory and walks over the CTA's share of the 8-column tiles; the
// 8 weight rows of a tile and slot are contiguous in the expert's tensor, so lane 0 of each warp
// brings them in with two bulk copies (codes, scales) onto the stage's mbarrier, which expects
// one arrival per warp.  One stage, four CTAs per SM (occupancy over ring depth, as above).
// Needs expert_ffn % 32 == 0 and 16-byte aligned expert tensors.
constexpr uint32_t kDownTile = 8;
constexpr uint32_t kDownStages = 1;

__host__ __device__ inline uint32_t down_tile_bytes(uint32_t expert_ffn) {
  return kDownTile * (expert_ffn / 2U + expert_ffn / 16U);  // one slot's codes + scales of a tile
}

template <int LANES>
__global__ void __launch_bounds__(256, 4)
moe_down_staged_kernel(MoeArgs a, uint32_t* error) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float out_tile[8][kDownTile];
  __shared__ __align__(8) uint64_t bar[kDownStages];
  pdl_trigger();
  if (threadIdx.x == 0U) {
    for (uint32_t s = 0; s < kDownStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(&bar[s])), "r"(8U));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();
  const uint32_t row = blockIdx.y, W = a.expert_ffn, blocks = W / 16U, K = a.route_width;
  const uint32_t slot = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t selection = row * K + min(slot, K - 1U);
  const uint32_t expert = slot < K ? a.indices[selection] : 0xffffffffU;
  const bool valid = expert < a.experts;
  ExpertMatrix D{};
  if (valid) D = a.down[expert];
  const uint32_t tiles = a.hidden / kDownTile;
  const uint32_t mine = blockIdx.x < tiles ? (tiles - blockIdx.x + gridDim.x - 1U) / gridDim.x : 0U;
  const uint32_t tile_bytes = down_tile_bytes(W), code_bytes = kDownTile * (W / 2U);
  uint8_t* ring = smem;  // [stage][slot][codes | scales]
  int8_t* mi8 = reinterpret_cast<int8_t*>(smem + static_cast<size_t>(kDownStages) * 8U * tile_bytes) +
                static_cast<size_t>(slot) * down_slot_bytes(W);
  float* mscale = reinterpret_cast<float*>(mi8 + W);
  auto issue = [&](uint32_t k) {  // lane 0 of every warp: its slot's part of tile k, or a bare arrival
    uint64_t* full = &bar[k % kDownStages];
    if (!valid) {
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(full)) : "memory");
      return;
    }
    uint8_t* dst = ring + (static_cast<size_t>(k % kDownStages) * 8U + slot) * tile_bytes;
    const size_t first = static_cast<size_t>(blockIdx.x + k * gridDim.x) * kDownTile;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(full)), "r"(tile_bytes)
                 : "memory");
    bulk_to_shared(dst, D.codes + first * (W / 2U), code_bytes, full);
    bulk_to_shared(dst + code_bytes, D.scales + first * blocks, tile_bytes - code_bytes, full);
  };
  if (lane == 0U)
    for (uint32_t k = 0; k < min(mine, kDownStages); ++k) issue(k);
  if (valid) {
    const uint4* src = reinterpret_cast<const uint4*>(a.mid_i8 + static_cast<size_t>(selection) * W);
    const float* src_scale = a.mid_scale + static_cast<size_t>(selection) * blocks;
    for (uint32_t i = lane; i < blocks; i += 32U) {
      reinterpret_cast<uint4*>(mi8)[i] = src[i];
      mscale[i] = src_scale[i];
    }
  }
  __syncwarp();
  constexpr uint32_t kGroups = 32U / LANES;
  const uint32_t group = lane / LANES, lane_in_group = lane % LANES;
  for (uint32_t k = 0; k < mine; ++k) {
    if (!wait_phase(&bar[k % kDownStages], (k / kDownStages) & 1U)) {
      if (threadIdx.x == 0U && error != nullptr) atomicExch(error, 401U);
      return;
    }
    if (valid) {
      const uint8_t* codes = ring + (static_cast<size_t>(k % kDownStages) * 8U + slot) * tile_bytes;
      const uint8_t* scales = codes + code_bytes;
#pragma unroll
      for (uint32_t pass = 0; pass < kDownTile / kGroups; ++pass) {
        const uint32_t r = pass * kGroups + group;
        double acc = 0.0;
        for (uint32_t blk = lane_in_group; blk < blocks; blk += LANES) {
          const uint2 w = reinterpret_cast<const uint2*>(codes + static_cast<size_t>(r) * (W / 2U))[blk];
          const int d = block16_dot(w, reinterpret_cast<const uint4*>(mi8)[blk]);
          acc += static_cast<double>(static_cast<float>(d) * (e4m3_value(scales[r * blocks + blk]) * mscale[blk]) * 0.25F);
        }
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffU, acc, o);
        if (lane_in_group == 0U) out_tile[slot][r] = bf16r(static_cast<float>(acc) * D.weight_scale / D.input_scale);
      }
    } else if (lane < kDownTile) {
      out_tile[slot][lane] = 0.0F;  // no candidate (or no such slot): contributes score * 0
    }
    __syncthreads();  // the stage is free, out_tile is complete
    if (lane == 0U && k + kDownStages < mine) issue(k + kDownStages);
    if (threadIdx.x < kDownTile) {
      const uint32_t column = (blockIdx.x + k * gridDim.x) * kDownTile + threadIdx.x;
      float total = 0.0F;
      for (uint32_t s = 0; s < K; ++s) {
        const float contribution = a.scores[row * K + s] * out_tile[s][threadIdx.x];
        total = total + contribution;
      }
      a.moe[static_cast<size_t>(row) * a.hidden + column] = bf16r(total);
    }
    __syncthreads();  // out_tile may be overwritten
  }
}

}  // namespace

namespace {
inline size_t round4(size_t n) { return (n + 3U) & ~static_cast<size_t>(3U); }  // 16-byte granules of floats
}  // namespace

// one arrival counter of the router kernel per row: the widest pass holds fewer rows than this
constexpr uint32_t kRouterTickets = 128;

size_t moe_workspace_floats(uint32_t rows, uint32_t route_width, uint32_t hidden, uint32_t expert_ffn) {
  const size_t selections = static_cast<size_t>(rows) * route_width;
  // router tickets (fixed place) | router logits | indices | scores | quantised mid (INT8 values,
  // then FP32 block scales) | moe
  return kRouterTickets + static_cast<size_t>(rows) * 256U + round4(2U * selections) + round4(selections * (expert_ffn / 4U)) +
         round4(selections * (expert_ffn / 16U)) + static_cast<size_t>(rows) * hidden;
}

void moe_carve_workspace(float* base, MoeArgs& a) {
  const size_t selections = static_cast<size_t>(a.rows) * a.route_width;
  a.router_tickets = reinterpret_cast<uint32_t*>(base);  // zero between launches, whatever the row count
  a.router_logits = base + kRouterTickets;
  base += kRouterTickets + static_cast<size_t>(a.rows) * 256U;
  a.indices = reinterpret_cast<uint32_t*>(base);
  a.scores = base + selections;
  float* mid = base + round4(2U * selections);
  a.mid_i8 = reinterpret_cast<int8_t*>(mid);
  a.mid_scale = mid + round4(selections * (a.expert_ffn / 4U));
  a.moe = a.mid_scale + round4(selections * (a.expert_ffn / 16U));
}

int launch_moe_router_select(const GemvOut& logits, const MoeArgs& a, cudaStream_t stream) {
  if (!a.rows || !a.route_width || a.route_width > 8U || a.route_width > a.experts || a.experts > 256U)
    return fail(QLLM_INVALID_ARGUMENT, "router needs 1..8 selections out of at most 256 experts");
  count_launch();
  return check_cuda(launch_pdl(moe_router_select_kernel, dim3(a.rows), dim3(32), 0, stream, logits, a.experts,
                               a.route_width, a.route_scale, a.indices, a.scores), "moe_router_select");
}

int launch_moe_router(const ExpertMatrix& router, const QuantSink& operand, const MoeArgs& a, cudaStream_t stream) {
  if (a.rows > kRouterTickets) return fail(QLLM_INVALID_ARGUMENT, "router pass is wider than its arrival counters");
  if (!a.rows || !a.route_width || a.route_width > 8U || a.route_width > a.experts || a.experts > 256U)
    return fail(QLLM_INVALID_ARGUMENT, "router needs 1..8 selections out of at most 256 experts");
  if (operand.kind != 0 || operand.cols != a.hidden || a.hidden % 16U)
    return fail(QLLM_INVALID_ARGUMENT, "the router reads the CUDA-core operand form of the normalised row");
  count_launch();
  if (!a.router_logits || !a.router_tickets) return fail(QLLM_INVALID_ARGUMENT, "router workspace is missing");
  return check_cuda(launch_pdl(moe_router_kernel, dim3((a.experts + kRouterChunk - 1U) / kRouterChunk, a.rows),
                               dim3(256), 0, stream, router,
                               static_cast<const int8_t*>(operand.xi8), static_cast<const float*>(operand.xscale), a),
                    "moe_router");
}

int launch_moe_experts(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 16U || a.expert_ffn % 16U || a.x_stride % 4U || a.hidden > 16384U || a.expert_ffn > 16384U)
    return fail(QLLM_INVALID_ARGUMENT, "expert widths must be multiples of 16 (at most 16384)");
  if (!a.route_width || a.route_width > 8U) return fail(QLLM_INVALID_ARGUMENT, "1..8 experts per token");
  const uint32_t selections = a.rows * a.route_width;
  const size_t smem_gu = 2U * (static_cast<size_t>(a.hidden) + a.hidden / 16U * sizeof(float));
  const size_t smem_d = 8U * down_slot_bytes(a.expert_ffn);
  if (smem_gu > 48U * 1024U || smem_d > 48U * 1024U)
    return fail(QLLM_INVALID_ARGUMENT, "expert input rows do not fit the shared-memory staging");
  int rc = 0;
  const size_t smem_staged = static_cast<size_t>(kStagedStages) * staged_stage_bytes(a.hidden) + smem_gu;
  if (a.staged && a.hidden % 256U == 0U && smem_staged <= 110U * 1024U) {
    static size_t opted_by_device[64] = {};  // the opt-in belongs to the device
    int device = 0;
    cudaGetDevice(&device);
    size_t& opted = opted_by_device[device & 63];
    if (opted < 48U * 1024U) opted = 48U * 1024U;
    if (smem_staged > opted) {
      rc = check_cuda(cudaFuncSetAttribute(moe_gate_up_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(110U * 1024U)), "expert kernel shared memory opt-in");
      if (rc) return rc;
      opted = 110U * 1024U;
    }
    // one wave: five CTAs per SM (148 SMs), shared evenly by the selections
    const uint32_t tiles = a.expert_ffn / kStagedRows;
    const uint32_t per_selection = std::max(1U, std::min(tiles, 740U / selections));
    rc = check_cuda(launch_pdl(moe_gate_up_staged_kernel, dim3(per_selection, selections), dim3(kStagedThreads),
                               smem_staged, stream, a, a.error), "moe_gate_up_staged");
  } else {
    rc = check_cuda(launch_pdl(moe_gate_up_kernel, dim3((a.expert_ffn + kGateUpRows - 1U) / kGateUpRows, selections),
                               dim3(256), smem_gu, stream, a), "moe_gate_up");
  }
  if (rc) return rc;
  count_launch(2);
  // 32 lanes per column only when that leaves no lane idle
  const bool wide = (a.expert_ffn / 16U) % 32U == 0U;
  const size_t smem_down_staged = static_cast<size_t>(kDownStages) * 8U * down_tile_bytes(a.expert_ffn) + smem_d;
  if (a.staged && a.expert_ffn % 32U == 0U && a.hidden % kDownTile == 0U && smem_down_staged <= 72U * 1024U) {
    static bool opted_by_device[64] = {};  // the opt-in belongs to the device
    int device = 0;
    cudaGetDevice(&device);
    bool& opted = opted_by_device[device & 63];
    if (!opted) {
      rc = check_cuda(cudaFuncSetAttribute(moe_down_staged_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(72U * 1024U)), "expert kernel shared memory opt-in");
      if (rc) return rc;
      rc = check_cuda(cudaFuncSetAttribute(moe_down_staged_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(72U * 1024U)), "expert kernel shared memory opt-in");
      if (rc) return rc;
      opted = true;
    }
    // one wave: four CTAs per SM, shared evenly by the rows
    const uint32_t per_row = std::max(1U, std::min(a.hidden / kDownTile, 592U / a.rows));
    const dim3 staged_grid(per_row, a.rows);
    if (wide)
      return check_cuda(launch_pdl(moe_down_staged_kernel<32>, staged_grid, dim3(256), smem_down_staged, stream, a,
                                   a.error), "moe_down_staged");
    return check_cuda(launch_pdl(moe_down_staged_kernel<16>, staged_grid, dim3(256), smem_down_staged, stream, a,
                                 a.error), "moe_down_staged");
  }
  const dim3 grid((a.hidden + kDownColumns - 1U) / kDownColumns, a.rows);
  if (wide)
    return check_cuda(launch_pdl(moe_down_kernel<32>, grid, dim3(256), smem_d, stream, a), "moe_down");
  return check_cuda(launch_pdl(moe_down_kernel<16>, grid, dim3(256), smem_d, stream, a), "moe_down");
}

}  // namespace qllm
