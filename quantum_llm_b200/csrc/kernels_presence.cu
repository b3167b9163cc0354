// Sampling presence penalty (apply_presence_penalty / presence_penalty_kernel,
// runtime/src/cuda/transformer_kernels.cu:7180-7186, :10784-10795) as the exact-decode path uses
// it (runtime/tools/dense_fp4_provider.cpp:8336-8347, :11182-11202, :11261-11270, :8822-8847):
// logits[token] -= penalty for every token the request has emitted, and -- inside a speculative
// step -- for the proposals that precede the row being judged.
//
// The reference keeps two byte masks per request (emitted, and a working copy that a verify pass
// or a rollout advances proposal by proposal, copied from the first before each use).  Here only
// the emitted mask exists; the working copy of a row is the mask plus the step's own draft tokens,
// which sit in the device-resident step state, so no 150 KB copy runs inside a step and every row
// of a verify pass is penalised by one launch.
#include "common.cuh"
#include "kernels.h"

namespace qllm {

namespace {

__global__ void __launch_bounds__(256)
presence_penalty_rows_kernel(PresenceArgs a) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  const uint32_t row = blockIdx.y;
  if (i >= a.count) return;
  bool hit = a.emitted[i] != 0U;
  if (!hit && a.mode != 0U) {
    const StepState* s = a.state;
    // verify row r sees the proposals before it; draft pass p the drafts of its own rollout so far
    const uint32_t seen = min(a.mode == 1U ? row : a.pass, min(s->draft_count, 4U));
    for (uint32_t j = 1U; j <= seen; ++j) hit = hit || s->verify_tokens[j] == i;
  }
  if (hit) a.logits[static_cast<size_t>(row) * a.stride + i] -= a.penalty;
}

// after the acceptance kernel: the accepted proposals and the selected next token become emitted
__global__ void presence_commit_step_kernel(const StepState* s, uint8_t* emitted, uint32_t vocab) {
  if (threadIdx.x != 0U || blockIdx.x != 0U || s->error != 0U) return;
  const uint32_t rows = min(s->mtp_rows, 8U);
  for (uint32_t i = 0; i < rows; ++i)
    if (s->mtp_tokens[i] < vocab) emitted[s->mtp_tokens[i]] = 1U;
}

// after the scalar head: the selected token becomes emitted
__global__ void presence_commit_token_kernel(const uint32_t* token, uint8_t* emitted, uint32_t vocab) {
  if (threadIdx.x != 0U || blockIdx.x != 0U) return;
  if (*token < vocab) emitted[*token] = 1U;
}

}  // namespace

int launch_presence_penalty(const PresenceArgs& a, cudaStream_t stream) {
  if (!a.logits || !a.emitted || !a.rows || !a.count || a.count > a.stride || (a.mode != 0U && !a.state) ||
      a.mode > 2U || !(a.penalty >= -2.0F && a.penalty <= 2.0F))
    return fail(QLLM_INVALID_ARGUMENT, "invalid presence penalty");
  presence_penalty_rows_kernel<<<dim3((a.count + 255U) / 256U, a.rows), 256, 0, stream>>>(a);
  count_launch();
  return check_launch("presence_penalty");
}

int launch_presence_commit_step(const StepState* state, uint8_t* emitted, uint32_t vocab, cudaStream_t stream) {
  presence_commit_step_kernel<<<1, 32, 0, stream>>>(state, emitted, vocab);
  count_launch();
  return check_launch("presence_commit_step");
}

int launch_presence_commit_token(const uint32_t* token, uint8_t* emitted, uint32_t vocab, cudaStream_t stream) {
  presence_commit_token_kernel<<<1, 32, 0, stream>>>(token, emitted, vocab);
  count_launch();
  return check_launch("presence_commit_token");
}

}  // namespace qllm
