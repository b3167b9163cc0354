// Reference-side adapter: quantum-llm's IOperationProvider over the C ABI of include/qllm_b200.h.
//
// A maintainer adds integration/b200_nvfp4_mtp_provider.{hpp,cpp} to the runner target next to
// runtime/tools/dense_fp4_provider.cpp and links libqllm_b200.so.  The adapter implements the
// exact-decode service of expert::runtime::IOperationProvider
// (runtime/include/expert/runtime/program_executor.hpp:244-370) and exports a factory of the shape the
// runner uses for every provider module (runtime/tools/dense_fp4_provider.cpp:11398-11499,
// runtime/tools/moe_vm_runner.cpp:39-53).
#pragma once

#include <cstdint>
#include <string>

#include "expert/runtime/execution_provider.hpp"
#include "expert/runtime/program_executor.hpp"

namespace expert::runtime {

struct B200Nvfp4MtpOptions final {
  std::uint32_t max_context{};        // admitted context (tokens); 0 = the artifact's
  std::uint32_t kv_page_tokens{256};
  std::string kv_dtype{"q4-f16-per-head"};   // or "f16"
  std::uint32_t attention_split_tokens{512};
  std::uint32_t mtp_draft_depth{4};   // must equal the artifact's draft_depth
  int device{0};
  std::uint32_t priority{50};
};

// One module = one provider bound to one GPU.  The artifact selects it by declaring
//   kernel        decode.mtp.dense-full-attention.nvfp4-block16.exact.v1  2
//   exact_decode  decode.mtp.dense-full-attention.nvfp4-block16.exact.v1  2  <draft_depth + 1>
// with the exact_decode_parameter keys of runtime/tools/dense_fp4_provider.cpp:2937-2966 and one
// exact_decode_tensor record per role listed in b200_nvfp4_mtp_provider.cpp.
[[nodiscard]] CreateExecutionProviderModuleResult make_b200_nvfp4_mtp_callable_provider(
    const B200Nvfp4MtpOptions& options);

}  // namespace expert::runtime
