// C shim over the reference's own CPU FFN executor (runtime/src/cpu/fp4_host_executor.cpp,
// Fp4HostExecutor), compiled unmodified from the reference tree into oracle/_ref/ by
// `make ref_fp4_host`.  TEST / BENCHMARK INFRASTRUCTURE ONLY: it gives the CPU-baseline leg of the
// benchmark a figure produced by the reference's own host code.  The executor runs SwiGLU experts
// stored as FP4-E2M1 with UE8M0 scales per 32 values against Q8 activations -- the reference's CPU
// lane format, not the NVFP4 block-16 format of the GPU path -- so the figure is a throughput
// reference (bytes of an FFN layer per second on this host), not a parity anchor.
#include <chrono>
#include <cstdint>
#include <cstring>
#include <vector>

#include "expert/runtime/cpu/fp4_host_executor.hpp"

namespace er = expert::runtime;

extern "C" {

// One dense FFN layer seen as a single expert selected by every row: gate/up [intermediate, hidden],
// down [hidden, intermediate], seeded bytes.  Returns the mean seconds of `repeats` executions after
// one untimed run, or a negative value on error; *checksum = sum of the last outputs.
double ref_fp4_host_ffn_seconds(uint32_t hidden, uint32_t intermediate, uint32_t rows, uint32_t threads,
                                uint32_t repeats, uint64_t seed, double* checksum) {
  try {
    const uint64_t wide = static_cast<uint64_t>(intermediate) * hidden;
    er::SplitExpertSections s{};
    uint64_t offset = 0;
    const auto place = [&](uint64_t& at, uint64_t& bytes, uint64_t size) {
      at = offset;
      bytes = size;
      offset += (size + 255U) & ~static_cast<uint64_t>(255U);
    };
    place(s.w1_weight_offset, s.w1_weight_bytes, wide / 2U);
    place(s.w1_scale_offset, s.w1_scale_bytes, wide / 32U);
    place(s.w3_weight_offset, s.w3_weight_bytes, wide / 2U);
    place(s.w3_scale_offset, s.w3_scale_bytes, wide / 32U);
    place(s.w2_weight_offset, s.w2_weight_bytes, wide / 2U);
    place(s.w2_scale_offset, s.w2_scale_bytes, wide / 32U);
    std::vector<std::byte> record(offset);
    uint64_t state = seed * 0x9e3779b97f4a7c15ULL + 1U;
    const auto next = [&] {
      state ^= state << 13U;
      state ^= state >> 7U;
      state ^= state << 17U;
      return state;
    };
    for (uint64_t i = 0; i + 8U <= record.size(); i += 8U) {
      const uint64_t v = next();
      std::memcpy(record.data() + i, &v, 8U);
    }
    // block scales: UE8M0 exponents around 2^-6 so that the sums stay finite
    const auto scales = [&](uint64_t at, uint64_t bytes) {
      for (uint64_t i = 0; i < bytes; ++i) record[at + i] = static_cast<std::byte>(119U + (next() & 3U));
    };
    scales(s.w1_scale_offset, s.w1_scale_bytes);
    scales(s.w3_scale_offset, s.w3_scale_bytes);
    scales(s.w2_scale_offset, s.w2_scale_bytes);
    er::cpu::Fp4HostWorkGroup group{};
    group.record_bytes = record;
    group.sections = s;
    group.hidden = hidden;
    group.intermediate = intermediate;
    for (uint32_t r = 0; r < rows; ++r) {
      group.selections.push_back(r);     // top_k = 1: selection r is row r
      group.output_slots.push_back(r);
    }
    std::vector<float> inputs(static_cast<size_t>(rows) * hidden), outputs(static_cast<size_t>(rows) * hidden);
    for (auto& v : inputs) v = static_cast<float>(static_cast<int64_t>(next() >> 40U) - (1 << 23)) * (1.0F / (1 << 23));
    er::cpu::Fp4HostExecutorConfig config{};
    config.maximum_threads = threads;
    er::cpu::Fp4HostExecutor executor(config);
    const std::vector<er::cpu::Fp4HostWorkGroup> groups{group};
    const auto run = [&] { return executor.execute(groups, inputs, rows, 1U, outputs); };
    if (!run().ok()) return -1.0;
    const auto begin = std::chrono::steady_clock::now();
    for (uint32_t i = 0; i < repeats; ++i)
      if (!run().ok()) return -1.0;
    const double seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - begin).count();
    double sum = 0.0;
    for (const float v : outputs) sum += v;
    if (checksum) *checksum = sum;
    return seconds / (repeats ? repeats : 1U);
  } catch (...) {
    return -2.0;
  }
}

}  // extern "C"
