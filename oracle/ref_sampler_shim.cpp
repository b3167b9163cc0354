// C shim over the reference's own sampler (runtime/src/speculative_sampling.cpp),
// compiled from the reference tree where it lies.  TEST INFRASTRUCTURE ONLY: it
// is used to pin the oracle's sampler restatement and, optionally, as the CPU
// baseline for the acceptance loop.  No reference source is copied here.
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

}  // extern "C"
