// tcgen05 block-scaled NVFP4 GEMV: prepared weight view and launcher.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/qllm_b200.h"
#include "quant.cuh"

namespace qllm {

// Per-matrix state of the tensor-core path: a TMA descriptor over the packed
// codes and the block scales re-tiled into the layout tcgen05 reads from
// tensor memory.  Owned by the provider; released with it.
struct MmaWeights {
  alignas(64) CUtensorMap codes_map;
  uint8_t* tiled_scales = nullptr;  // [row_tiles, k_atoms, 512]
  uint32_t rows = 0, cols = 0;
  bool ready = false;
  int prepare(const qllm_matrix& device_matrix, cudaStream_t stream);
  void release();
  MmaWeights() = default;
  MmaWeights(const MmaWeights&) = delete;
  MmaWeights& operator=(const MmaWeights&) = delete;
  MmaWeights(MmaWeights&& o) noexcept { *this = static_cast<MmaWeights&&>(o); }
  MmaWeights& operator=(MmaWeights&& o) noexcept;
  ~MmaWeights() { release(); }
};

// Tensor-parallel exchange of a K-split projection: every CTA of the GEMV stores its partial
// sums into the same inbox slot of every rank (its own through the local pointer, the peers'
// through their mapped memory) as 8-byte pairs {FP32 bits, sequence number}, one store per
// value, so that a reader can tell a delivered value from a stale one without any flag or fence
// (8-byte stores are not torn).  The consumer sums all ranks' partials in rank order
// (gemv_value4, quant.cuh), so every rank computes the same values.  The last CTA of a launch
// (a ticket counter) advances this rank's sequence number for the kernels that follow.
// Passed by value to the exchange form of the kernel.
struct GemvExchange {
  uint32_t ranks, rank;
  uint2* inbox[8];      // the slot of this exchange in every rank's inbox
  uint32_t* words;      // local status words (GemvOut::exchange): error, sequence, tickets
  size_t capacity;      // pairs one slot holds
};

size_t gemv_mma_workspace_bytes(uint32_t batch, uint32_t rows, uint32_t cols);
// y[batch, row_count] = bf16(fakequant(x) . W[first_row .. first_row+row_count)^T)
int launch_gemv_mma(const MmaWeights& w, const qllm_matrix& m, uint32_t first_row,
                    uint32_t row_count, const float* x, float* y, uint32_t batch, void* workspace,
                    size_t workspace_bytes, cudaStream_t stream);
// The tensor-core kernel alone over the operand a launch_gemv_mma() call with the same
// workspace, matrix and batch left behind (split-K partials stay in the workspace).
int launch_gemv_mma_core_only(const MmaWeights& w, const qllm_matrix& m, uint32_t batch, void* workspace,
                              size_t workspace_bytes, cudaStream_t stream);

}  // namespace qllm
