// Stand-in for libqllm_b200.so in the CPU link-compatibility test of the reference-side adapter:
// the same entry points with the same signatures (include/qllm_b200.h), no GPU behind them.
// It records what the adapter passes and answers like a provider whose every first draft is
// accepted: emitted = {guaranteed, guaranteed + 1}, next = guaranteed + 2.
#include <cstdlib>
#include <cstring>
#include <string>

#include "qllm_b200.h"

struct qllm_provider {
  qllm_config config;
  unsigned states, synchronizations, executions;
  qllm_request last_request;
};
struct qllm_request_state {
  unsigned length;
  unsigned checkpoint;   // 0: none
};

namespace {
thread_local std::string g_error;
qllm_provider* g_last = nullptr;
int fail(int rc, const char* text) {
  g_error = text;
  return rc;
}
}  // namespace

extern "C" {
const char* qllm_last_error(void) { return g_error.c_str(); }
const char* qllm_capability_name(void) { return "decode.mtp.dense-full-attention.nvfp4-block16.exact.v1"; }
uint32_t qllm_capability_abi(void) { return 2U; }

int qllm_provider_create(const qllm_config* config, const qllm_weights* weights, int on_device, int, qllm_provider** out) {
  if (!config || !weights || !out || on_device) return fail(QLLM_INVALID_ARGUMENT, "stub: bad create");
  // touch every pointer the adapter bound: a wrong offset shows up as a wrong byte
  if (!weights->embedding || !weights->layers || !weights->final_norm || !weights->head.codes || !weights->head.scales ||
      !weights->mtp_fusion.codes || !weights->mtp_block.qkv.codes || weights->final_norm[0] != 1.0F ||
      weights->layers[0].qkv.codes[0] != 0x21 || !(weights->head.weight_scale > 0.0F) ||
      weights->head.input_scale != 336.0F)
    return fail(QLLM_INVALID_ARGUMENT, "stub: the adapter bound a tensor wrongly");
  auto* p = new qllm_provider{};
  p->config = *config;
  g_last = p;
  *out = p;
  return QLLM_OK;
}
void qllm_provider_destroy(qllm_provider* p) {
  if (g_last == p) g_last = nullptr;
  delete p;
}
int qllm_provider_create_request_state(qllm_provider* p, qllm_request_state** out) {
  if (!p || !out) return fail(QLLM_INVALID_ARGUMENT, "stub: bad state");
  ++p->states;
  *out = new qllm_request_state{};
  return QLLM_OK;
}
void qllm_provider_destroy_request_state(qllm_provider* p, qllm_request_state* s) {
  if (p && s) --p->states;
  delete s;
}
int qllm_provider_synchronize_exact_decode_batch(qllm_provider* p, qllm_request_state* s, const qllm_request* rq,
                                                 const uint32_t* tokens, uint32_t count, uint32_t first, int) {
  if (!p || !s || !rq || !tokens || !count) return fail(QLLM_INVALID_ARGUMENT, "stub: bad synchronization");
  if (rq->sampling_presence_penalty_biased_ppm > 4000000U)
    return fail(QLLM_INVALID_ARGUMENT, "sampling presence penalty is invalid");
  p->last_request = *rq;
  ++p->synchronizations;
  s->length = first + count;
  return QLLM_OK;
}
int qllm_provider_execute_exact_decode(qllm_provider* p, qllm_request_state* s, const qllm_request* rq, uint32_t token,
                                       uint32_t position, uint32_t limit, qllm_exact_result* out) {
  if (!p || !s || !rq || !out) return fail(QLLM_INVALID_ARGUMENT, "stub: bad step");
  if (rq->sampling_presence_penalty_biased_ppm > 4000000U)
    return fail(QLLM_INVALID_ARGUMENT, "sampling presence penalty is invalid");
  if (position + 2U >= limit) return fail(QLLM_INVALID_ARGUMENT, "exact MTP invocation stream is invalid");
  p->last_request = *rq;
  ++p->executions;
  std::memset(out, 0, sizeof(*out));
  out->emitted_tokens[0] = token;
  out->emitted_tokens[1] = token + 1U;
  out->emitted_count = 2U;
  out->next_token = token + 2U;
  out->positions_advanced = 2U;
  s->length = position + 2U;
  return QLLM_OK;
}

int qllm_provider_checkpoint_request_state(qllm_provider* p, qllm_request_state* s, uint32_t next_position) {
  if (!p || !s || !next_position || next_position != s->length)
    return fail(QLLM_INVALID_ARGUMENT, "retention checkpoint position is invalid");
  s->checkpoint = next_position;
  return QLLM_OK;
}
int qllm_provider_rewind_request_state(qllm_provider* p, qllm_request_state* s, uint32_t next_position) {
  if (!p || !s || !s->checkpoint || s->checkpoint != next_position)
    return fail(QLLM_INVALID_ARGUMENT, "retention rewind position is invalid");
  s->length = next_position;
  return QLLM_OK;
}

// what the test reads back
const qllm_provider* qllm_stub_last_provider(void) { return g_last; }
}
