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

// ---- router: one warp per row -------------------------------------------------------------
__global__ void __launch_bounds__(32)
moe_router_select_kernel(GemvOut logits, uint32_t experts, uint32_t top_k, float route_scale, uint32_t* indices,
                         float* scores) {
  pdl_trigger();
  pdl_wait();
  const uint32_t row = blockIdx.x, lane = threadIdx.x;
  constexpr uint32_t kPerLane = 8;  // up to 256 experts
  float value[kPerLane];
#pragma unroll
  for (uint32_t i = 0; i < kPerLane; ++i) {
    const uint32_t e = lane + 32U * i;
    value[i] = e < experts ? bf16r(gemv_value(logits, row, e)) : kNegInf;
  }
  uint32_t taken = 0U;  // bit i: this lane's i-th expert is already selected
  float chosen_value[8];
  uint32_t chosen_index[8];
  for (uint32_t slot = 0; slot < top_k; ++slot) {
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
  if (lane == 0U) {
    float top = -INFINITY, sum = 0.0F, s[8];
    for (uint32_t slot = 0; slot < top_k; ++slot) top = fmaxf(top, chosen_value[slot]);
    for (uint32_t slot = 0; slot < top_k; ++slot) {
      // exp in double, rounded once: the same FP32 value on the device and in a host check
      s[slot] = static_cast<float>(exp(static_cast<double>(chosen_value[slot] - top)));
      sum += s[slot];
    }
    for (uint32_t slot = 0; slot < top_k; ++slot) {
      float v = s[slot] / sum;
      if (route_scale != 1.0F) v *= route_scale;
      scores[row * top_k + slot] = bf16r(v);
      indices[row * top_k + slot] = chosen_index[slot];
    }
  }
}

// ---- shared pieces of the two expert projections ---------------------------------------------
// Quantises `count` FP32 values (count % 16 == 0) into INT8 + block scales in shared memory.
__device__ __forceinline__ void quantize_row_to_shared(const float* __restrict__ x, uint32_t count, float g,
                                                       bool round_bf16, int8_t* xi8, float* xscale) {
  for (uint32_t blk = threadIdx.x; blk < count / 16U; blk += blockDim.x) {
    float v[16];
    const float4* in4 = reinterpret_cast<const float4*>(x + 16U * blk);
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
}

// Exact sum over the blocks of one weight row against the quantised activations (warp-wide).
__device__ __forceinline__ double row_dot(const ExpertMatrix& m, uint32_t row, uint32_t cols, const int8_t* xi8,
                                          const float* xscale, uint32_t lane) {
  const uint32_t blocks = cols / 16U;
  const uint2* w = reinterpret_cast<const uint2*>(m.codes + static_cast<size_t>(row) * (cols / 2U));
  const uint8_t* s = m.scales + static_cast<size_t>(row) * blocks;
  double acc = 0.0;
  for (uint32_t blk = lane; blk < blocks; blk += 32U) {
    const int d = block16_dot(__ldg(w + blk), reinterpret_cast<const uint4*>(xi8)[blk]);
    // exact: |d| < 2^12, the product of the two E4M3 scales has 8 significant bits
    acc += static_cast<double>(static_cast<float>(d) * (e4m3_value(__ldg(s + blk)) * xscale[blk]) * 0.25F);
  }
  return warp_sum_f64(acc);
}

// ---- gate / up / SiLU: grid (ceil(expert_ffn / 8), selections), 8 warps = 8 output rows --------
__global__ void __launch_bounds__(256)
moe_gate_up_kernel(MoeArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const uint32_t selection = blockIdx.y, row = selection / a.route_width;
  const uint32_t expert = a.indices[selection];
  if (expert >= a.experts) return;  // the router found no candidate (non-finite logits): contributes nothing
  const uint32_t H = a.hidden, blocks = H / 16U;
  int8_t* gi8 = reinterpret_cast<int8_t*>(smem);
  int8_t* ui8 = gi8 + H;
  float* gscale = reinterpret_cast<float*>(ui8 + H);
  float* uscale = gscale + blocks;
  const ExpertMatrix G = a.gate[expert], U = a.up[expert];
  const float* x = a.x + static_cast<size_t>(row) * a.x_stride;
  quantize_row_to_shared(x, H, G.input_scale, true, gi8, gscale);
  quantize_row_to_shared(x, H, U.input_scale, true, ui8, uscale);
  __syncthreads();
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t out_row = blockIdx.x * 8U + warp;
  if (out_row >= a.expert_ffn) return;
  const double g = row_dot(G, out_row, H, gi8, gscale, lane);
  const double u = row_dot(U, out_row, H, ui8, uscale, lane);
  if (lane == 0U) {
    const float gate = bf16r(static_cast<float>(g) * G.weight_scale / G.input_scale);
    const float up = bf16r(static_cast<float>(u) * U.weight_scale / U.input_scale);
    a.mid[static_cast<size_t>(selection) * a.expert_ffn + out_row] = bf16r((gate / (1.0F + expf(-gate))) * up);
  }
}

// ---- down: grid (ceil(hidden / 8), selections) ---------------------------------------------------
__global__ void __launch_bounds__(256)
moe_down_kernel(MoeArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_trigger();
  pdl_wait();
  const uint32_t selection = blockIdx.y;
  const uint32_t expert = a.indices[selection];
  const uint32_t W = a.expert_ffn, blocks = W / 16U;
  const uint32_t warp = threadIdx.x >> 5U, lane = threadIdx.x & 31U;
  const uint32_t out_row = blockIdx.x * 8U + warp;
  if (expert >= a.experts) {
    if (out_row < a.hidden && lane == 0U) a.out[static_cast<size_t>(selection) * a.hidden + out_row] = 0.0F;
    return;
  }
  int8_t* mi8 = reinterpret_cast<int8_t*>(smem);
  float* mscale = reinterpret_cast<float*>(mi8 + W);
  const ExpertMatrix D = a.down[expert];
  quantize_row_to_shared(a.mid + static_cast<size_t>(selection) * W, W, D.input_scale, false, mi8, mscale);
  __syncthreads();
  if (out_row >= a.hidden) return;
  const double t = row_dot(D, out_row, W, mi8, mscale, lane);
  if (lane == 0U)
    a.out[static_cast<size_t>(selection) * a.hidden + out_row] =
        bf16r(static_cast<float>(t) * D.weight_scale / D.input_scale);
}

// ---- ordered weighted sum over the slots -------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_aggregate_kernel(MoeArgs a) {
  pdl_trigger();
  pdl_wait();
  const uint32_t index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= a.rows * a.hidden) return;
  const uint32_t row = index / a.hidden, column = index % a.hidden;
  float total = 0.0F;
  for (uint32_t slot = 0; slot < a.route_width; ++slot) {
    const size_t selection = static_cast<size_t>(row) * a.route_width + slot;
    const float contribution = a.scores[selection] * a.out[selection * a.hidden + column];
    total = total + contribution;
  }
  a.moe[index] = bf16r(total);
}

}  // namespace

size_t moe_workspace_floats(uint32_t rows, uint32_t route_width, uint32_t hidden, uint32_t expert_ffn) {
  const size_t selections = static_cast<size_t>(rows) * route_width;
  // scores | mid | out | moe, and the indices (same width as a float) in front
  return 2U * selections + selections * expert_ffn + selections * hidden + static_cast<size_t>(rows) * hidden;
}

int launch_moe_router_select(const GemvOut& logits, const MoeArgs& a, cudaStream_t stream) {
  if (!a.rows || !a.route_width || a.route_width > 8U || a.route_width > a.experts || a.experts > 256U)
    return fail(QLLM_INVALID_ARGUMENT, "router needs 1..8 selections out of at most 256 experts");
  count_launch();
  return check_cuda(launch_pdl(moe_router_select_kernel, dim3(a.rows), dim3(32), 0, stream, logits, a.experts,
                               a.route_width, a.route_scale, a.indices, a.scores), "moe_router_select");
}

int launch_moe_experts(const MoeArgs& a, cudaStream_t stream) {
  if (a.hidden % 16U || a.expert_ffn % 16U || a.x_stride % 4U || a.hidden > 16384U || a.expert_ffn > 16384U)
    return fail(QLLM_INVALID_ARGUMENT, "expert widths must be multiples of 16 (at most 16384)");
  const uint32_t selections = a.rows * a.route_width;
  const size_t smem_gu = 2U * (static_cast<size_t>(a.hidden) + a.hidden / 16U * sizeof(float));
  const size_t smem_d = static_cast<size_t>(a.expert_ffn) + a.expert_ffn / 16U * sizeof(float);
  if (smem_gu > 48U * 1024U || smem_d > 48U * 1024U)
    return fail(QLLM_INVALID_ARGUMENT, "expert input row does not fit the shared-memory staging");
  int rc = check_cuda(launch_pdl(moe_gate_up_kernel, dim3((a.expert_ffn + 7U) / 8U, selections), dim3(256), smem_gu,
                                 stream, a), "moe_gate_up");
  if (rc) return rc;
  rc = check_cuda(launch_pdl(moe_down_kernel, dim3((a.hidden + 7U) / 8U, selections), dim3(256), smem_d, stream, a),
                  "moe_down");
  if (rc) return rc;
  count_launch(3);
  return check_cuda(launch_pdl(moe_aggregate_kernel, dim3((a.rows * a.hidden + 255U) / 256U), dim3(256), 0, stream, a),
                    "moe_aggregate");
}

}  // namespace qllm
