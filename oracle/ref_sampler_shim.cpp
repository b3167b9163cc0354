// C shim over the reference's own sampler (runtime/src/speculative_sampling.cpp),
// compiled from the reference tree where it lies.  TEST INFRASTRUCTURE ONLY: it
// is used to pin the oracle's sampler restatement and, optionally, as the CPU
// baseline for the acceptance loop.  No reference source is copied here.
#include <chrono>
#include <cstdint>
#include <exception>
#include <span>
#include <vector>

#include "expert/runtime/speculative_sampling.hpp"

namespace er = expert::runtime;

extern "C" {

double ref_counter_uniform(std::uint64_t seed, std::uint32_t position, std::uint32_t stream,
                           std::uint32_t index) {
  return er::counter_uniform(seed, position, stream, index);
}

int ref_make_distribution(const float* logits, const std::uint32_t* tokens, std::uint32_t count,
                          std::uint32_t temperature_ppm, std::uint32_t top_p_ppm,
                          std::uint32_t min_p_ppm, std::uint32_t* out_tokens,
                          double* out_probabilities) {
  try {
    const auto d = er::make_sampling_distribution(std::span(logits, count), std::span(tokens, count),
                                                  temperature_ppm, top_p_ppm, min_p_ppm);
    for (std::size_t i = 0; i < d.entries.size(); ++i) {
      out_tokens[i] = d.entries[i].token;
      out_probabilities[i] = d.entries[i].probability;
    }
    return static_cast<int>(d.entries.size());
  } catch (const std::exception&) {
    return -1;
  }
}

static er::SamplingDistribution build(const std::uint32_t* tokens, const double* probs,
                                      std::uint32_t count) {
  er::SamplingDistribution d;
  for (std::uint32_t i = 0; i < count; ++i) d.entries.push_back({tokens[i], probs[i]});
  return d;
}

int ref_sample_distribution(const std::uint32_t* tokens, const double* probs, std::uint32_t count,
                            double uniform, std::uint32_t* token) {
  try {
    *token = er::sample_distribution(build(tokens, probs, count), uniform);
    return 0;
  } catch (const std::exception&) {
    return -1;
  }
}

int ref_rejection_sample(std::uint32_t proposal, const std::uint32_t* tt, const double* tp,
                         std::uint32_t tc, const std::uint32_t* dt, const double* dp,
                         std::uint32_t dc, double ua, double uc, std::uint32_t* token) {
  try {
    const auto r = er::rejection_sample(proposal, build(tt, tp, tc), build(dt, dp, dc), ua, uc);
    *token = r.token;
    return r.accepted ? 1 : 0;
  } catch (const std::exception&) {
    return -1;
  }
}

// The acceptance decisions of `steps` speculative steps as the reference makes them on the host
// (dense_fp4_provider.cpp:11190-11234): per step 5 target and 4 draft distributions over `top_k`
// sorted candidates, up to 4 rejection decisions, one bonus sample.  Returns seconds per step
// (negative on error); *accepted = drafts accepted in total.  Benchmark's CPU leg only.
double ref_acceptance_seconds_per_step(std::uint32_t steps, std::uint32_t top_k, std::uint64_t seed,
                                       std::uint64_t* accepted) {
  try {
    std::vector<float> logits(top_k);
    std::vector<std::uint32_t> tokens(top_k);
    std::uint64_t total = 0;
    const auto begin = std::chrono::steady_clock::now();
    for (std::uint32_t step = 0; step < steps; ++step) {
      std::vector<er::SamplingDistribution> target, draft;
      for (std::uint32_t row = 0; row < 9U; ++row) {
        for (std::uint32_t i = 0; i < top_k; ++i) {
          // descending logits, the same candidate ids for target and draft so that p/q is not trivially 0
          logits[i] = 4.0F - 0.37F * static_cast<float>(i) -
                      0.01F * static_cast<float>((step * 9U + row + i) % 7U) * (row < 5U ? 1.0F : 0.5F);
          tokens[i] = 100U + i;
        }
        for (std::uint32_t i = 1; i < top_k; ++i)
          if (logits[i] > logits[i - 1U]) logits[i] = logits[i - 1U];
        auto d = er::make_sampling_distribution(logits, tokens, 700000U, 950000U, 0U);
        (row < 5U ? target : draft).push_back(std::move(d));
      }
      std::uint32_t a = 0;
      for (; a < 4U; ++a) {
        const auto proposal = er::sample_distribution(draft[a], er::counter_uniform(seed, step, 1U + a));
        const auto r = er::rejection_sample(proposal, target[a], draft[a], er::counter_uniform(seed, step + a, 100U, a),
                                            er::counter_uniform(seed, step + a, 200U, a));
        if (!r.accepted) break;
      }
      if (a == 4U) (void)er::sample_distribution(target[4], er::counter_uniform(seed, step + a, 300U));
      total += a;
    }
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - begin).count();
    if (accepted) *accepted = total;
    return seconds / (steps ? steps : 1U);
  } catch (const std::exception&) {
    return -1.0;
  }
}

}  // extern "C"
