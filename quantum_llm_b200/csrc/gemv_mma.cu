// placeholder until the tcgen05 kernel lands
#include "gemv_mma.h"
#include "common.cuh"
namespace qllm {
int MmaWeights::prepare(const qllm_matrix&, cudaStream_t) { ready = false; return 0; }
void MmaWeights::release() { if (tiled_scales) cudaFree(tiled_scales); tiled_scales = nullptr; ready = false; }
MmaWeights& MmaWeights::operator=(MmaWeights&& o) noexcept {
  if (this != &o) { release(); codes_map = o.codes_map; tiled_scales = o.tiled_scales; rows = o.rows; cols = o.cols; ready = o.ready; o.tiled_scales = nullptr; o.ready = false; }
  return *this;
}
size_t gemv_mma_workspace_bytes(uint32_t, uint32_t, uint32_t) { return 0; }
int launch_gemv_mma(const MmaWeights&, const qllm_matrix&, uint32_t, uint32_t, const float*, float*, uint32_t, void*, size_t, cudaStream_t) {
  return fail(QLLM_INVALID_ARGUMENT, "tcgen05 GEMV is not built");
}
}
