// Acceptance sampling, draft sampling and rollback bookkeeping on the device.
// One kernel decides the whole verify batch (greedy or temperature rejection),
// emits the result record, and moves the request cursor, so the decode step
// never returns to the host between verify and the next draft passes.
// Arithmetic follows runtime/src/speculative_sampling.cpp (double precision,
// same operation order) and the call sequence of
// runtime/tools/dense_fp4_provider.cpp:11183-11304, 8809-8852.
#include "common.cuh"
#include "kernels.h"

namespace qllm {

struct DeviceDist {
  uint32_t count;
  uint32_t tokens[64];
  double probs[64];
};

__device__ unsigned long long splitmix64(unsigned long long v) {
  v += 0x9e3779b97f4a7c15ULL;
  v = (v ^ (v >> 30U)) * 0xbf58476d1ce4e5b9ULL;
  v = (v ^ (v >> 27U)) * 0x94d049bb133111ebULL;
  return v ^ (v >> 31U);
}

__device__ double counter_uniform(unsigned long long seed, uint32_t position, uint32_t stream,
                                  uint32_t index) {
  unsigned long long c = seed;
  c ^= static_cast<unsigned long long>(position) * 0xd2b74407b1ce6e93ULL;
  c ^= static_cast<unsigned long long>(stream) * 0xca5a826395121157ULL;
  c ^= static_cast<unsigned long long>(index) * 0x9e3779b185ebca87ULL;
  return static_cast<double>(splitmix64(c) >> 11U) * (1.0 / 9007199254740992.0);
}

// Returns false when the candidates are invalid (same conditions as the reference throws on).
__device__ bool make_distribution(const float* logits, const uint32_t* tokens, uint32_t count,
                                  uint32_t temperature_ppm, uint32_t top_p_ppm, uint32_t min_p_ppm,
                                  DeviceDist* out) {
  if (!count || count > 64U || temperature_ppm == 0U || temperature_ppm > 2000000U ||
      top_p_ppm == 0U || top_p_ppm > 1000000U || min_p_ppm > 1000000U || !isfinite(logits[0]))
    return false;
  for (uint32_t i = 1; i < count; ++i)
    if ((!isnan(logits[i]) && logits[i] > logits[i - 1]) ||
        (logits[i] == logits[i - 1] && tokens[i] < tokens[i - 1]))
      return false;
  const double inv_t = 1000000.0 / static_cast<double>(temperature_ppm);
  const double maximum = static_cast<double>(logits[0]);
  const double min_rel = static_cast<double>(min_p_ppm) / 1000000.0;
  double total = 0.0;
  uint32_t n = 0;
  for (uint32_t i = 0; i < count; ++i) {
    const double l = static_cast<double>(logits[i]);
    const double w = isfinite(l) ? exp((l - maximum) * inv_t) : 0.0;
    if (w < min_rel) continue;
    out->tokens[n] = tokens[i];
    out->probs[n] = w;
    total += w;
    ++n;
  }
  if (!n || !isfinite(total) || !(total > 0.0)) return false;
  const double top_p = static_cast<double>(top_p_ppm) / 1000000.0;
  double cumulative = 0.0;
  uint32_t nucleus = n;
  for (uint32_t i = 0; i < n; ++i) {
    cumulative += out->probs[i] / total;
    if (cumulative >= top_p) { nucleus = i + 1U; break; }
  }
  total = 0.0;
  for (uint32_t i = 0; i < nucleus; ++i) total += out->probs[i];
  for (uint32_t i = 0; i < nucleus; ++i) out->probs[i] = out->probs[i] / total;
  out->count = nucleus;
  return true;
}

__device__ double dist_probability(const uint32_t* tokens, const double* probs, uint32_t count,
                                   uint32_t token) {
  for (uint32_t i = 0; i < count; ++i)
    if (tokens[i] == token) return probs[i];
  return 0.0;
}

__device__ uint32_t sample_distribution(const uint32_t* tokens, const double* probs, uint32_t count,
                                        double u) {
  double cumulative = 0.0;
  for (uint32_t i = 0; i < count; ++i) {
    cumulative += probs[i];
    if (u < cumulative) return tokens[i];
  }
  return tokens[count - 1U];
}

// 1 accepted, 0 rejected (token = sample of normalised max(p-q,0) walked in ascending
// token id), -1 invalid.
__device__ int rejection_sample(uint32_t proposal, const uint32_t* tt, const double* tp, uint32_t tc,
                                const uint32_t* dt, const double* dp, uint32_t dc, double ua,
                                double uc, uint32_t* token) {
  const double p = dist_probability(tt, tp, tc, proposal);
  const double q = dist_probability(dt, dp, dc, proposal);
  if (!(q > 0.0)) return -1;
  if (ua < fmin(1.0, p / q)) { *token = proposal; return 1; }
  uint32_t rt[128];
  double rp[128];
  uint32_t n = 0;
  for (uint32_t i = 0; i < tc; ++i) { rt[n] = tt[i]; rp[n] = tp[i]; ++n; }
  for (uint32_t i = 0; i < dc; ++i) {
    uint32_t j = 0;
    while (j < n && rt[j] != dt[i]) ++j;
    if (j == n) { rt[n] = dt[i]; rp[n] = 0.0; ++n; }
    rp[j] = fmax(0.0, rp[j] - dp[i]);
  }
  for (uint32_t i = 1; i < n; ++i) {  // ascending token id
    const uint32_t t = rt[i];
    const double v = rp[i];
    uint32_t j = i;
    while (j > 0 && rt[j - 1] > t) { rt[j] = rt[j - 1]; rp[j] = rp[j - 1]; --j; }
    rt[j] = t;
    rp[j] = v;
  }
  double total = 0.0;
  for (uint32_t i = 0; i < n; ++i) total += rp[i];
  if (!isfinite(total) || !(total > 0.0)) return -1;
  const double threshold = uc * total;
  double cumulative = 0.0;
  uint32_t last_positive = 0;
  bool found = false;
  for (uint32_t i = 0; i < n; ++i) {
    if (rp[i] > 0.0) { last_positive = rt[i]; found = true; }
    cumulative += rp[i];
    if (threshold < cumulative) { *token = rt[i]; return 0; }
  }
  if (!found) return -1;
  *token = last_positive;
  return 0;
}

// Target distribution of verify row `row`: {argmax: 1} when greedy.
__device__ bool target_distribution(const StepState* s, const AcceptArgs& a, uint32_t row,
                                    DeviceDist* out) {
  if (s->temperature_ppm == 0U) {
    out->count = 1;
    out->tokens[0] = a.argmax_tokens[row];
    out->probs[0] = 1.0;
    return true;
  }
  return make_distribution(a.top_values + static_cast<size_t>(row) * s->top_k,
                           a.top_tokens + static_cast<size_t>(row) * s->top_k, s->top_k,
                           s->temperature_ppm, s->top_p_ppm, s->min_p_ppm, out);
}

__global__ void accept_kernel(AcceptArgs a) {
  if (threadIdx.x != 0U || blockIdx.x != 0U) return;
  StepState* s = a.state;
  const uint32_t proposals = s->draft_count;
  const uint32_t position = s->position;
  StepRecord* record = a.results + (s->step_index % a.results_capacity);
  qllm_exact_result* result = &record->result;
  record->draft_count = 0U;
  record->error = s->error;
  s->step_index += 1U;
  result->emitted_count = 0U;
  result->positions_advanced = 0U;
  if (s->error != 0U || proposals == 0U || proposals > 4U ||
      position + proposals >= s->context_limit) {
    if (s->error == 0U) s->error = 1U;  // invalid multi-draft state
    record->error = s->error;
    return;
  }
  DeviceDist target;
  uint32_t accepted = 0, next_token = 0;
  bool rejected = false;
  for (; accepted < proposals; ++accepted) {
    if (!target_distribution(s, a, accepted, &target)) { s->error = record->error = 2U; return; }
    const DraftDistribution& d = s->drafts[accepted];
    uint32_t token = 0;
    const int r = rejection_sample(s->verify_tokens[accepted + 1U], target.tokens, target.probs,
                                   target.count, d.tokens, d.probabilities, d.count,
                                   counter_uniform(s->seed, position + accepted, 100U, accepted),
                                   counter_uniform(s->seed, position + accepted, 200U, accepted),
                                   &token);
    if (r < 0) { s->error = record->error = 3U; return; }
    if (r == 0) { next_token = token; rejected = true; break; }
  }
  if (!rejected) {
    if (!target_distribution(s, a, accepted, &target)) { s->error = record->error = 2U; return; }
    next_token = sample_distribution(target.tokens, target.probs, target.count,
                                     counter_uniform(s->seed, position + accepted, 300U, 0U));
  }
  // result record: guaranteed token + accepted drafts; next_token stays unemitted
  for (uint32_t i = 0; i <= accepted; ++i) result->emitted_tokens[i] = s->verify_tokens[i];
  result->emitted_count = accepted + 1U;
  result->next_token = next_token;
  result->positions_advanced = accepted + 1U;
  result->rejected = rejected ? 1U : 0U;
  // rollback bookkeeping: the draft cache cursor stays at `position`; the rows the next
  // draft pass consumes are the accepted drafts followed by the selected token
  for (uint32_t i = 0; i < 8U; ++i)
    s->mtp_tokens[i] = i < accepted ? s->verify_tokens[i + 1U] : next_token;
  s->accepted = accepted;
  s->next_token = next_token;
  s->rejected = rejected ? 1U : 0U;
  s->mtp_rows = accepted + 1U;
  s->new_position = position + accepted + 1U;
  s->draft_count = 0U;
  s->exact_calls += 1ULL;
  s->accepted_drafts += accepted;
  s->accepted_depth_calls[accepted] += 1ULL;
}

int launch_accept(const AcceptArgs& a, cudaStream_t stream) {
  accept_kernel<<<1, 32, 0, stream>>>(a);
  count_launch();
  return check_launch("accept");
}

__global__ void draft_sample_kernel(DraftSampleArgs a, uint32_t commit) {
  if (threadIdx.x != 0U || blockIdx.x != 0U) return;
  StepState* s = a.state;
  if (s->error == 0U) {
    const uint32_t i = a.pass;
    // cache length before this pass ran: the committed length plus the chained rows so far
    const uint32_t length_before = s->new_position + (i == 0U ? 0U : i - 1U);
    bool produce;
    if (i == 0U) produce = s->new_position + 1U < s->context_limit;  // future_exact
    else produce = s->draft_count == i && s->draft_count < s->draft_depth &&
                   length_before + 2U < s->context_limit;
    if (produce) {
      DraftDistribution& d = s->drafts[i];
      uint32_t token;
      if (s->temperature_ppm == 0U) {
        token = a.argmax_token[0];
        d.count = 1U;
        d.tokens[0] = token;
        d.probabilities[0] = 1.0;
      } else {
        DeviceDist dist;
        if (!make_distribution(a.top_values, a.top_tokens, s->top_k, s->temperature_ppm,
                               s->top_p_ppm, s->min_p_ppm, &dist)) {
          s->error = 4U;
          return;
        }
        d.count = dist.count;
        for (uint32_t j = 0; j < dist.count; ++j) {
          d.tokens[j] = dist.tokens[j];
          d.probabilities[j] = dist.probs[j];
        }
        token = sample_distribution(dist.tokens, dist.probs, dist.count,
                                    counter_uniform(s->seed, length_before, 1U + i, 0U));
      }
      s->verify_tokens[i + 1U] = token;
      s->draft_count = i + 1U;
    }
  }
  if (commit) {
    if (a.kernel_error != nullptr && *a.kernel_error != 0U && s->error == 0U) s->error = *a.kernel_error;
    s->verify_tokens[0] = s->next_token;
    s->position = s->new_position;
    if (a.results != nullptr && !a.from_sync) {
      StepRecord* record = a.results + ((s->step_index - 1U) % a.results_capacity);
      record->draft_count = s->draft_count;
      record->error = s->error;
    }
  }
}

int launch_draft_sample(const DraftSampleArgs& a, cudaStream_t stream) {
  // the provider marks the last pass of a step by setting bit 31 of `pass`
  DraftSampleArgs b = a;
  const uint32_t commit = a.pass >> 31U;
  b.pass = a.pass & 0x7fffffffU;
  draft_sample_kernel<<<1, 32, 0, stream>>>(b, commit);
  count_launch();
  return check_launch("draft_sample");
}

__global__ void first_token_kernel(StepState* s, const uint32_t* argmax_token,
                                   const float* top_values, const uint32_t* top_tokens,
                                   uint32_t sample_position, uint32_t* out) {
  if (threadIdx.x != 0U || blockIdx.x != 0U) return;
  if (s->temperature_ppm == 0U) { *out = argmax_token[0]; return; }
  DeviceDist dist;
  if (!make_distribution(top_values, top_tokens, s->top_k, s->temperature_ppm, s->top_p_ppm,
                         s->min_p_ppm, &dist)) {
    s->error = 5U;
    *out = 0U;
    return;
  }
  *out = sample_distribution(dist.tokens, dist.probs, dist.count,
                             counter_uniform(s->seed, sample_position, 0U, 0U));
}

int launch_first_token(StepState* state, const uint32_t* argmax_token, const float* top_values,
                       const uint32_t* top_tokens, uint32_t sample_position, uint32_t* out,
                       cudaStream_t stream) {
  first_token_kernel<<<1, 32, 0, stream>>>(state, argmax_token, top_values, top_tokens,
                                           sample_position, out);
  count_launch();
  return check_launch("first_token");
}

// ---------------------------------------------------------------------------
// Host-pointer forms used by the parity tests of the sampler arithmetic.
struct HostProbe {
  uint32_t tt[64], dt[64];
  double tp[64], dp[64];
  float logits[64];
  uint32_t tc, dc, proposal, token;
  uint32_t temperature_ppm, top_p_ppm, min_p_ppm;
  double ua, uc, uniform;
  unsigned long long seed;
  uint32_t position, stream, index;
  int status;
};

__global__ void probe_kernel(HostProbe* p, int what) {
  if (threadIdx.x != 0U) return;
  if (what == 0) {
    p->status = rejection_sample(p->proposal, p->tt, p->tp, p->tc, p->dt, p->dp, p->dc, p->ua,
                                 p->uc, &p->token);
  } else if (what == 1) {
    DeviceDist d;
    if (make_distribution(p->logits, p->tt, p->tc, p->temperature_ppm, p->top_p_ppm, p->min_p_ppm,
                          &d)) {
      p->dc = d.count;
      for (uint32_t i = 0; i < d.count; ++i) { p->dt[i] = d.tokens[i]; p->dp[i] = d.probs[i]; }
      p->status = static_cast<int>(d.count);
    } else {
      p->status = -1;
    }
  } else {
    p->uniform = counter_uniform(p->seed, p->position, p->stream, p->index);
    p->status = 0;
  }
}

static int run_probe(HostProbe& h, int what) {
  HostProbe* d = nullptr;
  int rc = check_cuda(cudaMalloc(&d, sizeof(HostProbe)), "probe alloc");
  if (rc) return rc;
  rc = check_cuda(cudaMemcpy(d, &h, sizeof(HostProbe), cudaMemcpyHostToDevice), "probe upload");
  if (!rc) {
    probe_kernel<<<1, 32>>>(d, what);
    count_launch();
    rc = check_launch("sampler probe");
  }
  if (!rc) rc = check_cuda(cudaMemcpy(&h, d, sizeof(HostProbe), cudaMemcpyDeviceToHost), "probe download");
  cudaFree(d);
  return rc;
}

}  // namespace qllm

extern "C" {

int qllm_k_rejection_sample_host(uint32_t proposal, const uint32_t* tt, const double* tp,
                                 uint32_t tc, const uint32_t* dt, const double* dp, uint32_t dc,
                                 double ua, double uc, uint32_t* token) {
  if (!tc || tc > 64U || !dc || dc > 64U || !token)
    return qllm::fail(QLLM_INVALID_ARGUMENT, "invalid rejection probe");
  qllm::HostProbe h{};
  for (uint32_t i = 0; i < tc; ++i) { h.tt[i] = tt[i]; h.tp[i] = tp[i]; }
  for (uint32_t i = 0; i < dc; ++i) { h.dt[i] = dt[i]; h.dp[i] = dp[i]; }
  h.tc = tc; h.dc = dc; h.proposal = proposal; h.ua = ua; h.uc = uc;
  const int rc = qllm::run_probe(h, 0);
  if (rc) return rc;
  *token = h.token;
  return h.status < 0 ? qllm::fail(QLLM_INVALID_ARGUMENT, "rejection sample rejected its input")
                      : h.status;
}

int qllm_k_make_distribution_host(const float* logits, const uint32_t* tokens, uint32_t count,
                                  uint32_t temperature_ppm, uint32_t top_p_ppm,
                                  uint32_t min_p_ppm, uint32_t* out_tokens, double* out_probs) {
  if (!count || count > 64U) return qllm::fail(QLLM_INVALID_ARGUMENT, "invalid distribution probe");
  qllm::HostProbe h{};
  for (uint32_t i = 0; i < count; ++i) { h.logits[i] = logits[i]; h.tt[i] = tokens[i]; }
  h.tc = count; h.temperature_ppm = temperature_ppm; h.top_p_ppm = top_p_ppm; h.min_p_ppm = min_p_ppm;
  const int rc = qllm::run_probe(h, 1);
  if (rc) return rc;
  if (h.status < 0) return qllm::fail(QLLM_INVALID_ARGUMENT, "invalid sorted sampling candidates");
  for (int i = 0; i < h.status; ++i) { out_tokens[i] = h.dt[i]; out_probs[i] = h.dp[i]; }
  return h.status;
}

int qllm_k_counter_uniform_host(uint64_t seed, uint32_t position, uint32_t stream_id,
                                uint32_t index, double* out) {
  qllm::HostProbe h{};
  h.seed = seed; h.position = position; h.stream = stream_id; h.index = index;
  const int rc = qllm::run_probe(h, 2);
  if (rc) return rc;
  *out = h.uniform;
  return 0;
}

}  // extern "C"
