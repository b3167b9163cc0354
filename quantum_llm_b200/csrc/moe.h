// Routed-expert FFN of the decode step: device descriptors and launchers (kernels_moe.cu).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "quant.cuh"

namespace qllm {

// One expert projection on the device (NVFP4: codes [rows, cols/2], E4M3 scales [rows, cols/16]).
struct ExpertMatrix {
  const uint8_t* codes;
  const uint8_t* scales;
  float weight_scale;
  float input_scale;
};

struct MoeArgs {
  const float* x;          // [rows, x_stride] post-attention RMSNorm rows (rounded to BF16 on use)
  uint32_t x_stride;
  uint32_t rows, hidden, experts, route_width, expert_ffn;
  float route_scale;
  uint32_t* indices;       // [rows * route_width] selected expert per slot
  float* scores;           // [rows * route_width] BF16-rounded routing weights
  const ExpertMatrix* gate;  // [experts], each [expert_ffn, hidden]
  const ExpertMatrix* up;    // [experts], each [expert_ffn, hidden]
  const ExpertMatrix* down;  // [experts], each [hidden, expert_ffn]
  int8_t* mid_i8;          // [rows * route_width, expert_ffn] mid quantised for the down projection
  float* mid_scale;        // [rows * route_width, expert_ffn / 16] its block scales
  float* moe;              // [rows, hidden] BF16-rounded weighted sum (added to the residual by the next norm)
  float* router_logits;    // [rows, 256] BF16-rounded router logits (fused router kernel)
  uint32_t* router_tickets;  // [8] arrival counters of that kernel's CTAs per row, zero between launches
  bool staged;             // every expert tensor is 16-byte aligned: the gate/up weights may come in by bulk copies
  uint32_t* error;         // status word set when a bounded wait runs out
};

// floats of workspace for indices, scores, quantised mid and moe together (16-byte aligned parts)
size_t moe_workspace_floats(uint32_t rows, uint32_t route_width, uint32_t hidden, uint32_t expert_ffn);
// points indices, scores, mid_i8, mid_scale and moe of `a` (rows, route_width, expert_ffn set)
// into a workspace of that size
void moe_carve_workspace(float* base, MoeArgs& a);
// top-K selection + normalised scores from the router GEMV result
int launch_moe_router_select(const GemvOut& logits, const MoeArgs& a, cudaStream_t stream);
// router projection (exact CUDA-core arithmetic over the INT8 operand `operand`, kind 0) and
// selection in one launch
int launch_moe_router(const ExpertMatrix& router, const QuantSink& operand, const MoeArgs& a, cudaStream_t stream);
// gate/up/SiLU, then down with the ordered weighted sum (two launches)
int launch_moe_experts(const MoeArgs& a, cudaStream_t stream);

}  // namespace qllm
