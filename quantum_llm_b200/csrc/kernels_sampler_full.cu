// Full-vocabulary sampler of the scalar decode fallback: top_k == 0 (no truncation) or
// top_k > 64, where the exact sorted top-k kernels do not apply.  Restates, on the device,
// sample_token (runtime/tools/dense_fp4_provider.cpp:771-802): order every token id by
// (logit descending, NaN last, id ascending), keep the first top_k (all when 0), then
// make_sampling_distribution / sample_distribution (runtime/src/speculative_sampling.cpp:52-128)
// over that list with counter_uniform(seed, position, 0).  The reference copies the whole
// logits row to the host and sorts it there; here the row never leaves the device.
//
// Order of operations that fixes the bits: the weights exp((l - max) / T) are independent and
// computed in parallel; every sum the reference makes front to back (total mass, the nucleus
// cumulative, the renormalising total, the sampling cumulative) is made front to back by one
// thread, fed from shared memory by the rest of the block.
#include "common.cuh"
#include "kernels.h"

namespace qllm {

namespace {

constexpr uint32_t kSortTile = 2048U;     // keys one CTA sorts in shared memory (1024 threads)
constexpr uint32_t kStage = 2048U;        // doubles staged per step of the sequential passes

// Ascending 64-bit key == the reference's comparator: high word falls as the logit rises, NaN is
// the largest high word, -0 and +0 share one, the id breaks ties upwards.
__device__ __forceinline__ unsigned long long sort_key(float v, uint32_t id) {
  uint32_t high;
  if (isnan(v)) {
    high = 0xFFFFFFFFU;
  } else {
    uint32_t u = __float_as_uint(v == 0.0F ? 0.0F : v);
    u = (u & 0x80000000U) ? ~u : (u | 0x80000000U);   // monotone in the value
    high = ~u;
  }
  return (static_cast<unsigned long long>(high) << 32U) | id;
}

__global__ void __launch_bounds__(1024)
full_sort_keys_kernel(const float* __restrict__ logits, uint32_t vocab, unsigned long long* __restrict__ keys) {
  __shared__ unsigned long long tile[kSortTile];
  const uint32_t base = blockIdx.x * kSortTile;
  for (uint32_t i = threadIdx.x; i < kSortTile; i += 1024U) {
    const uint32_t id = base + i;
    tile[i] = id < vocab ? sort_key(logits[id], id) : ~0ULL;   // padding sorts behind every token
  }
  __syncthreads();
  for (uint32_t k = 2U; k <= kSortTile; k <<= 1U)
    for (uint32_t j = k >> 1U; j; j >>= 1U) {
      const uint32_t t = threadIdx.x;
      const uint32_t i = ((t & ~(j - 1U)) << 1U) | (t & (j - 1U));
      const unsigned long long a = tile[i], b = tile[i | j];
      const bool up = ((base + i) & k) == 0U;
      if ((a > b) == up) { tile[i] = b; tile[i | j] = a; }
      __syncthreads();
    }
  for (uint32_t i = threadIdx.x; i < kSortTile; i += 1024U) keys[base + i] = tile[i];
}

// one compare-exchange distance j >= kSortTile of the merge of runs of length k
__global__ void __launch_bounds__(1024)
full_sort_global_kernel(unsigned long long* __restrict__ keys, uint32_t k, uint32_t j) {
  const uint32_t t = blockIdx.x * 1024U + threadIdx.x;
  const uint32_t i = ((t & ~(j - 1U)) << 1U) | (t & (j - 1U));
  const unsigned long long a = keys[i], b = keys[i | j];
  const bool up = (i & k) == 0U;
  if ((a > b) == up) { keys[i] = b; keys[i | j] = a; }
}

// the distances below kSortTile of that merge, in shared memory
__global__ void __launch_bounds__(1024)
full_sort_local_kernel(unsigned long long* __restrict__ keys, uint32_t k) {
  __shared__ unsigned long long tile[kSortTile];
  const uint32_t base = blockIdx.x * kSortTile;
  for (uint32_t i = threadIdx.x; i < kSortTile; i += 1024U) tile[i] = keys[base + i];
  __syncthreads();
  for (uint32_t j = kSortTile >> 1U; j; j >>= 1U) {
    const uint32_t t = threadIdx.x;
    const uint32_t i = ((t & ~(j - 1U)) << 1U) | (t & (j - 1U));
    const unsigned long long a = tile[i], b = tile[i | j];
    const bool up = ((base + i) & k) == 0U;
    if ((a > b) == up) { tile[i] = b; tile[i | j] = a; }
    __syncthreads();
  }
  for (uint32_t i = threadIdx.x; i < kSortTile; i += 1024U) keys[base + i] = tile[i];
}

__global__ void full_weights_kernel(const float* __restrict__ logits, const unsigned long long* __restrict__ keys,
                                    uint32_t count, uint32_t temperature_ppm, double* __restrict__ weights,
                                    uint32_t* __restrict__ ids) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const double inv_t = 1000000.0 / static_cast<double>(temperature_ppm);
  const double maximum = static_cast<double>(logits[static_cast<uint32_t>(keys[0])]);
  const uint32_t id = static_cast<uint32_t>(keys[i]);
  const double l = static_cast<double>(logits[id]);
  weights[i] = isfinite(l) ? exp((l - maximum) * inv_t) : 0.0;
  ids[i] = id;
}

// Walks `n` values front to back on thread 0, staged through shared memory by the whole block:
// `body(index, value)` returns false to stop.  Thread 0's accumulators live in its registers;
// the caller publishes them to the block afterwards.
template <typename Body>
__device__ void sequential_pass(const double* values, uint32_t n, double* stage, uint32_t* stop, Body body) {
  for (uint32_t base = 0; base < n; base += kStage) {
    const uint32_t m = min(kStage, n - base);
    for (uint32_t i = threadIdx.x; i < m; i += blockDim.x) stage[i] = values[base + i];
    __syncthreads();
    if (threadIdx.x == 0U)
      for (uint32_t i = 0; i < m; ++i)
        if (!body(base + i, stage[i])) { *stop = 1U; break; }
    __syncthreads();
    if (*stop) break;
  }
  __syncthreads();
  if (threadIdx.x == 0U) *stop = 0U;
  __syncthreads();
}

__global__ void __launch_bounds__(256)
full_sample_kernel(FullSampleParams q, const float* __restrict__ logits, const unsigned long long* __restrict__ keys,
                   uint32_t count, double* weights, uint32_t* ids, uint32_t* error, uint32_t* out) {
  __shared__ double stage[kStage];
  __shared__ uint32_t stop, shared_count;
  __shared__ double shared_sum;
  if (threadIdx.x == 0U) stop = 0U;
  __syncthreads();
  const uint32_t temperature_ppm = q.temperature_ppm, top_p_ppm = q.top_p_ppm, min_p_ppm = q.min_p_ppm;
  if (!count || temperature_ppm == 0U || temperature_ppm > 2000000U || top_p_ppm == 0U || top_p_ppm > 1000000U ||
      min_p_ppm > 1000000U || !isfinite(logits[static_cast<uint32_t>(keys[0])])) {
    if (threadIdx.x == 0U) { *error = 5U; *out = 0U; }
    return;
  }
  // candidates below the min-p floor drop out, the rest keep their order (compacted in place:
  // the write index never passes the read index, and a stage is read before it is overwritten)
  const double min_rel = static_cast<double>(min_p_ppm) / 1000000.0;
  double total = 0.0;
  uint32_t kept = 0U;
  sequential_pass(weights, count, stage, &stop, [&](uint32_t i, double w) {
    if (w < min_rel) return true;
    if (kept != i) { weights[kept] = w; ids[kept] = ids[i]; }
    total += w;
    ++kept;
    return true;
  });
  if (threadIdx.x == 0U) { shared_count = kept; shared_sum = total; }
  __syncthreads();
  kept = shared_count;
  total = shared_sum;
  __syncthreads();
  if (!kept || !isfinite(total) || !(total > 0.0)) {
    if (threadIdx.x == 0U) { *error = 5U; *out = 0U; }
    return;
  }
  const double top_p = static_cast<double>(top_p_ppm) / 1000000.0;
  double cumulative = 0.0;
  uint32_t nucleus = kept;
  sequential_pass(weights, kept, stage, &stop, [&](uint32_t i, double w) {
    cumulative += w / total;
    if (cumulative >= top_p) { nucleus = i + 1U; return false; }
    return true;
  });
  if (threadIdx.x == 0U) shared_count = nucleus;
  __syncthreads();
  nucleus = shared_count;
  __syncthreads();
  double mass = 0.0;
  sequential_pass(weights, nucleus, stage, &stop, [&](uint32_t, double w) { mass += w; return true; });
  if (threadIdx.x == 0U) shared_sum = mass;
  __syncthreads();
  mass = shared_sum;
  // counter_uniform(seed, position, stream 0, index 0) of speculative_sampling.cpp: the stream and
  // index terms vanish, the rest is the splitmix64 finaliser
  unsigned long long c = q.seed ^ (static_cast<unsigned long long>(q.sample_position) * 0xd2b74407b1ce6e93ULL);
  c += 0x9e3779b97f4a7c15ULL;
  c = (c ^ (c >> 30U)) * 0xbf58476d1ce4e5b9ULL;
  c = (c ^ (c >> 27U)) * 0x94d049bb133111ebULL;
  c ^= c >> 31U;
  const double uniform = static_cast<double>(c >> 11U) * (1.0 / 9007199254740992.0);
  cumulative = 0.0;
  uint32_t chosen = nucleus - 1U;     // the last entry when the cumulative never passes the uniform
  sequential_pass(weights, nucleus, stage, &stop, [&](uint32_t i, double w) {
    cumulative += w / mass;
    if (uniform < cumulative) { chosen = i; return false; }
    return true;
  });
  if (threadIdx.x == 0U) *out = ids[chosen];
}

}  // namespace

uint32_t full_sampler_padded(uint32_t vocab) {
  uint32_t n = kSortTile;
  while (n < vocab) n <<= 1U;
  return n;
}

size_t full_sampler_workspace_bytes(uint32_t vocab) {
  // keys [padded] u64, weights [vocab] f64, ids [vocab] u32
  return static_cast<size_t>(full_sampler_padded(vocab)) * 8U + static_cast<size_t>(vocab) * 12U + 64U;
}

int launch_full_vocabulary_sample(const FullSampleParams& q, const float* logits, uint32_t vocab, void* workspace,
                                  uint32_t* error, uint32_t* out, cudaStream_t stream) {
  const uint32_t top_k = q.top_k;
  if (!error || !logits || !workspace || !out || !vocab || top_k > vocab || vocab > (1U << 30U) ||
      q.temperature_ppm == 0U)
    return fail(QLLM_INVALID_ARGUMENT, "invalid full-vocabulary sampling arguments");
  const uint32_t padded = full_sampler_padded(vocab);
  auto* keys = static_cast<unsigned long long*>(workspace);
  auto* weights = reinterpret_cast<double*>(keys + padded);
  auto* ids = reinterpret_cast<uint32_t*>(weights + vocab);
  full_sort_keys_kernel<<<padded / kSortTile, 1024, 0, stream>>>(logits, vocab, keys);
  count_launch();
  for (uint32_t k = kSortTile << 1U; k <= padded; k <<= 1U) {
    for (uint32_t j = k >> 1U; j >= kSortTile; j >>= 1U) {
      full_sort_global_kernel<<<padded / 2048U, 1024, 0, stream>>>(keys, k, j);
      count_launch();
    }
    full_sort_local_kernel<<<padded / kSortTile, 1024, 0, stream>>>(keys, k);
    count_launch();
  }
  const uint32_t count = top_k == 0U ? vocab : top_k;
  full_weights_kernel<<<(count + 255U) / 256U, 256, 0, stream>>>(logits, keys, count, q.temperature_ppm, weights, ids);
  count_launch();
  full_sample_kernel<<<1, 256, 0, stream>>>(q, logits, keys, count, weights, ids, error, out);
  count_launch();
  return check_launch("full_vocabulary_sample");
}

}  // namespace qllm
