// Reference-side adapter: quantum-llm's IOperationProvider over the C ABI of include/qllm_b200.h.
// See b200_nvfp4_mtp_provider.hpp.  Everything here runs at start-up or forwards one call; the
// decode step itself is one C call (qllm_provider_execute_exact_decode).
//
// Tensor roles this provider asks the artifact to bind with exact_decode_tensor records
// (provider-owned names, like the roles of runtime/tools/dense_fp4_provider.cpp:4733-4786):
//   token_embedding (BF16 [vocab, hidden]), final_norm, output_head,
//   embedding_norm, hidden_norm, draft_norm, fusion_projection,
//   layer.<l>.{input_norm, qkv_projection, output_projection, post_attention_norm,
//              gate_up_projection, down_projection}          for every target layer l,
//   mtp.{input_norm, qkv_projection, output_projection, post_attention_norm, gate_up_projection,
//        down_projection}                                    for the draft block.
// Projections are native NVFP4 records (quant ABI 5: packed E2M1 codes, E4M3 block scales, then
// the FP32 weight divisor and the FP32 or BF16 activation divisor, decoded as
// runtime/tools/dense_fp4_provider.cpp:3534-3568 does); q/k/v and gate/up are fused row-wise by
// the artifact compiler because a fused projection has one per-tensor scale.
#include "b200_nvfp4_mtp_provider.hpp"

#include <bit>
#include <cmath>
#include <cstring>
#include <map>
#include <mutex>
#include <optional>
#include <vector>

#include "qllm_b200.h"

namespace expert::runtime {
namespace {

constexpr std::uint32_t kNvfp4QuantAbi = 5U;   // kExpertRecordAbiNvfp4Block16W4A4

Status to_status(int rc) {
  if (rc == QLLM_OK) return Status::success();
  // the library's status codes are the negated ErrorCode values that can occur on this path
  return {static_cast<ErrorCode>(static_cast<std::uint8_t>(-rc)), qllm_last_error()};
}

std::optional<std::uint64_t> find(const std::map<std::string, std::uint64_t, std::less<>>& m, std::string_view key) {
  const auto it = m.find(key);
  if (it == m.end()) return std::nullopt;
  return it->second;
}

// Request parameters read on this path (runtime/tools/moe_vm_runner.cpp:318-347).  A request that
// asks for something this provider does not implement is refused, never decoded without it.
Status request_of(const ProgramRequestContext& context, qllm_request* out) {
  auto get = [&](std::string_view key, std::uint64_t fallback) { return find(context.parameters, key).value_or(fallback); };
  qllm_request r{};
  r.sampling_seed = get("sampling_seed", 0U);
  r.sampling_temperature_ppm = static_cast<std::uint32_t>(get("sampling_temperature_ppm", 0U));
  r.sampling_top_p_ppm = static_cast<std::uint32_t>(get("sampling_top_p_ppm", 1'000'000U));
  r.sampling_top_k = static_cast<std::uint32_t>(get("sampling_top_k", 0U));
  r.sampling_min_p_ppm = static_cast<std::uint32_t>(get("sampling_min_p_ppm", 0U));
  r.reserved_context_tokens = static_cast<std::uint32_t>(get("reserved_context_tokens", 0U));
  // value + 2 000 000 (runtime/tools/dense_fp4_provider.cpp:8336-8341); absent = neutral
  r.sampling_presence_penalty_biased_ppm =
      static_cast<std::uint32_t>(get("sampling_presence_penalty_biased_ppm", 2'000'000U));
  r.sampling_first_output_position = static_cast<std::uint32_t>(get("sampling_first_output_position", 0U));
  if (get("sampling_presence_penalty_biased_ppm", 2'000'000U) > 4'000'000U)
    return {ErrorCode::invalid_argument, "sampling presence penalty is invalid"};
  *out = r;
  return Status::success();
}

struct PreparedExactDecode final : IPreparedOperation {};

struct RequestState final : IOperationProviderRequestState {
  qllm_provider* provider{};
  qllm_request_state* state{};
  ~RequestState() override {
    if (state) qllm_provider_destroy_request_state(provider, state);
  }
};

class B200Nvfp4MtpProvider final : public IOperationProvider {
 public:
  explicit B200Nvfp4MtpProvider(B200Nvfp4MtpOptions options) : options_(std::move(options)) {}
  ~B200Nvfp4MtpProvider() override {
    if (provider_) qllm_provider_destroy(provider_);
  }

  // Ordinary SSA operations are other providers' business: this one implements the
  // artifact-declared exact decode service only.
  PrepareOperationResult prepare(const OperationPreparationContext&) override {
    return {{ErrorCode::invalid_argument, "the B200 NVFP4 MTP provider implements the exact decode service only"}, {}};
  }
  OperationExecutionHandle execute(const IPreparedOperation&, const std::shared_ptr<IOperationProviderRequestState>&,
                                   const OperationInvocation&) override {
    return {};
  }

  CreateOperationRequestStateResult create_request_state(const ProgramRequestContext&) override {
    std::lock_guard lock(mutex_);
    if (!provider_) return {{ErrorCode::invalid_argument, "exact decode was not prepared"}, {}};
    auto state = std::make_shared<RequestState>();
    state->provider = provider_;
    const int rc = qllm_provider_create_request_state(provider_, &state->state);
    if (rc != QLLM_OK) return {to_status(rc), {}};
    return {Status::success(), std::move(state)};
  }

  // Binds geometry and tensors once (the work of DenseFp4Provider::prepare_exact_decode,
  // runtime/tools/dense_fp4_provider.cpp:2865-2984) and creates the library's provider object,
  // which uploads the weights and builds its TMA descriptors and re-tiled scales.
  PrepareOperationResult prepare_exact_decode(const ExactDecodePreparationContext& context) override {
    std::lock_guard lock(mutex_);
    try {
      if (provider_) return {{ErrorCode::invalid_argument, "exact decode is prepared already"}, {}};
      if (context.program.capability != qllm_capability_name() || context.program.abi_version != qllm_capability_abi())
        return {{ErrorCode::invalid_argument, "the artifact's exact decode program is another provider's"}, {}};
      qllm_config c{};
      const auto& p = context.compiled.parameters;
      const auto& a = context.model.attributes;
      auto need = [](const auto& map, std::string_view key) -> std::uint32_t {
        const auto v = find(map, key);
        if (!v) throw std::runtime_error("the artifact lacks '" + std::string(key) + "'");
        return static_cast<std::uint32_t>(*v);
      };
      c.draft_depth = need(p, "draft_depth");
      c.draft_vocab = need(p, "draft_vocabulary_size");
      if (need(p, "source_mtp_layers") != 1U || need(p, "mtp_kv_encoding") != 1U || need(p, "embedding_first") != 1U ||
          need(p, "post_norm") != 1U || !c.draft_depth || c.draft_depth > 4U ||
          c.draft_depth != options_.mtp_draft_depth || context.compiled.maximum_emitted_tokens != c.draft_depth + 1U)
        return {{ErrorCode::invalid_argument, "unsupported exact-decode artifact contract"}, {}};
      c.layers = static_cast<std::uint32_t>(context.model.layer_program.size());
      c.hidden = context.model.hidden_size;
      c.vocab = context.model.vocab_size;
      c.q_heads = need(a, "attention_heads");
      c.kv_heads = need(a, "kv_heads");
      c.head_dim = need(a, "head_dim");
      c.rotary_dim = need(a, "rotary_dimension");
      c.eps = std::bit_cast<float>(need(a, "norm_epsilon_f32_bits"));
      c.rope_theta = std::bit_cast<float>(need(a, "rope_theta_f32_bits"));
      c.ffn = need(a, "intermediate_size");
      c.activation_bf16 = find(a, "activation_bf16").value_or(0U) == 1U ? 1U : 0U;
      c.page_tokens = options_.kv_page_tokens;
      c.split_tokens = options_.attention_split_tokens;
      c.kv_encoding = options_.kv_dtype == "f16" ? QLLM_KV_F16 : QLLM_KV_Q4H;
      c.mtp_kv_encoding = QLLM_KV_Q8;
      c.max_context = options_.max_context ? std::min(options_.max_context, context.model.max_context_tokens)
                                           : context.model.max_context_tokens;

      std::map<std::string, const ImmutableModelTensor*, std::less<>> roles;
      for (const auto& binding : context.tensors) {
        if (!binding.tensor || !binding.tensor->value.valid() || !roles.emplace(binding.role, binding.tensor.get()).second)
          return {{ErrorCode::invalid_argument, "exact decode tensor binding '" + binding.role + "' is invalid"}, {}};
        retained_.push_back(binding.tensor);   // the mapping outlives the upload
      }
      auto tensor = [&](const std::string& role) -> const ImmutableModelTensor& {
        const auto it = roles.find(role);
        if (it == roles.end()) throw std::runtime_error("the artifact binds no tensor to role '" + role + "'");
        return *it->second;
      };
      auto vector_f32 = [&](const std::string& role, std::uint32_t count) {
        const auto& t = tensor(role);
        if (t.data_bytes != static_cast<std::uint64_t>(count) * sizeof(float))
          throw std::runtime_error("tensor of role '" + role + "' is not an FP32 vector of the model's width");
        return reinterpret_cast<const float*>(t.value.data + t.data_offset);
      };
      auto matrix = [&](const std::string& role, std::uint32_t rows, std::uint32_t cols) {
        const auto& t = tensor(role);
        const std::uint64_t local = static_cast<std::uint64_t>(rows) * cols / 16U;
        if (t.quant_abi != kNvfp4QuantAbi || t.shape.size() != 2U || t.shape[0] != rows || t.shape[1] != cols ||
            cols % 16U || t.data_bytes != static_cast<std::uint64_t>(rows) * cols / 2U ||
            (t.scale_bytes != local + 2U * sizeof(float) && t.scale_bytes != local + sizeof(float) + sizeof(std::uint16_t)))
          throw std::runtime_error("tensor of role '" + role + "' is not a native NVFP4 matrix of the expected shape");
        const auto* base = reinterpret_cast<const std::uint8_t*>(t.value.data);
        float weight_divisor{}, input_divisor{};
        std::memcpy(&weight_divisor, base + t.scale_offset + local, sizeof(float));
        if (t.scale_bytes == local + 2U * sizeof(float)) {
          std::memcpy(&input_divisor, base + t.scale_offset + local + sizeof(float), sizeof(float));
        } else {
          std::uint16_t bits{};
          std::memcpy(&bits, base + t.scale_offset + local + sizeof(float), sizeof(bits));
          input_divisor = std::bit_cast<float>(static_cast<std::uint32_t>(bits) << 16U);
        }
        if (!std::isfinite(weight_divisor) || !(weight_divisor > 0.0F) || !std::isfinite(input_divisor) ||
            !(input_divisor > 0.0F))
          throw std::runtime_error("native NVFP4 global divisor is invalid");
        qllm_matrix m{};
        m.codes = base + t.data_offset;
        m.scales = base + t.scale_offset;
        m.weight_scale = 1.0F / weight_divisor;
        m.input_scale = input_divisor;
        m.rows = rows;
        m.cols = cols;
        return m;
      };
      auto block = [&](const std::string& prefix) {
        qllm_block b{};
        b.input_norm = vector_f32(prefix + "input_norm", c.hidden);
        b.qkv = matrix(prefix + "qkv_projection", (c.q_heads + 2U * c.kv_heads) * c.head_dim, c.hidden);
        b.o = matrix(prefix + "output_projection", c.hidden, c.q_heads * c.head_dim);
        b.post_norm = vector_f32(prefix + "post_attention_norm", c.hidden);
        b.gate_up = matrix(prefix + "gate_up_projection", 2U * c.ffn, c.hidden);
        b.down = matrix(prefix + "down_projection", c.hidden, c.ffn);
        return b;
      };
      std::vector<qllm_block> layers;
      for (std::uint32_t l = 0; l < c.layers; ++l) layers.push_back(block("layer." + std::to_string(l) + "."));
      qllm_weights w{};
      const auto& embedding = tensor("token_embedding");
      if (embedding.data_bytes != static_cast<std::uint64_t>(c.vocab) * c.hidden * 2U)
        throw std::runtime_error("token_embedding is not a BF16 [vocab, hidden] table");
      w.embedding = reinterpret_cast<const std::uint16_t*>(embedding.value.data + embedding.data_offset);
      w.layers = layers.data();
      w.final_norm = vector_f32("final_norm", c.hidden);
      w.head = matrix("output_head", c.vocab, c.hidden);
      w.mtp_embedding_norm = vector_f32("embedding_norm", c.hidden);
      w.mtp_hidden_norm = vector_f32("hidden_norm", c.hidden);
      w.mtp_fusion = matrix("fusion_projection", c.hidden, 2U * c.hidden);
      w.mtp_block = block("mtp.");
      w.mtp_draft_norm = vector_f32("draft_norm", c.hidden);
      const int rc = qllm_provider_create(&c, &w, /*weights_on_device=*/0, options_.device, &provider_);
      if (rc != QLLM_OK) return {to_status(rc), {}};
      config_ = c;
      return {Status::success(), std::make_shared<PreparedExactDecode>()};
    } catch (const std::exception& e) {
      return {{ErrorCode::invalid_argument, e.what()}, {}};
    }
  }

  Status synchronize_exact_decode(const IPreparedOperation& operation,
                                  const std::shared_ptr<IOperationProviderRequestState>& state,
                                  const ExactDecodeSynchronization& s) override {
    const std::uint32_t token = s.next_token;
    return synchronize_exact_decode_batch(
        operation, state, {s.request, std::span<const std::uint32_t>(&token, 1U), s.target_position, s.produce_draft});
  }

  Status synchronize_exact_decode_batch(const IPreparedOperation& operation,
                                        const std::shared_ptr<IOperationProviderRequestState>& state,
                                        const ExactDecodeSynchronizationBatch& batch) override {
    std::lock_guard lock(mutex_);   // one driver thread at a time, runtime/tools/dense_fp4_provider.cpp:11144
    auto* st = dynamic_cast<RequestState*>(state.get());
    if (dynamic_cast<const PreparedExactDecode*>(&operation) == nullptr || st == nullptr || batch.next_tokens.empty())
      return {ErrorCode::invalid_argument, "MTP synchronization stream is invalid"};
    qllm_request rq{};
    if (auto status = request_of(batch.request, &rq); !status.ok()) return status;
    return to_status(qllm_provider_synchronize_exact_decode_batch(
        provider_, st->state, &rq, batch.next_tokens.data(), static_cast<std::uint32_t>(batch.next_tokens.size()),
        batch.first_target_position, batch.produce_final_draft ? 1 : 0));
  }

  ExactDecodeExecutionHandle execute_exact_decode(const IPreparedOperation& operation,
                                                  const std::shared_ptr<IOperationProviderRequestState>& state,
                                                  const ExactDecodeInvocation& invocation) override {
    std::lock_guard lock(mutex_);
    auto* st = dynamic_cast<RequestState*>(state.get());
    if (dynamic_cast<const PreparedExactDecode*>(&operation) == nullptr || st == nullptr) return {};
    ExactDecodeExecutionResult out;
    qllm_request rq{};
    out.status = request_of(invocation.request, &rq);
    if (out.status.ok()) {
      qllm_exact_result r{};
      const int rc = qllm_provider_execute_exact_decode(provider_, st->state, &rq, invocation.guaranteed_token,
                                                        invocation.position, invocation.context_limit, &r);
      out.status = to_status(rc);
      if (rc == QLLM_OK) {
        out.emitted_tokens.assign(r.emitted_tokens, r.emitted_tokens + r.emitted_count);
        out.next_token = r.next_token;
        out.positions_advanced = r.positions_advanced;
      }
    }
    // the call above returns when the step's record has reached the host: the handle is complete
    // at once, like the reference's (completed_exact)
    struct Done final {
      ExactDecodeExecutionResult result;
      bool taken{};
    };
    auto done = std::make_shared<Done>();
    done->result = std::move(out);
    return ExactDecodeExecutionHandle::from_callbacks(
        [done]() -> std::optional<ExactDecodeExecutionResult> {
          if (done->taken) return std::nullopt;
          done->taken = true;
          return std::move(done->result);
        },
        [done] { done->taken = true; });
  }

  // Session retention (runtime/tools/dense_fp4_provider.cpp:9209-9338): the library keeps the
  // checkpointed position per request state and applies the reference's admission conditions.
  bool supports_request_state_retention() const noexcept override { return true; }
  Status checkpoint_request_state(const std::shared_ptr<IOperationProviderRequestState>& state,
                                  std::uint32_t next_position) override {
    std::lock_guard lock(mutex_);
    auto* st = dynamic_cast<RequestState*>(state.get());
    if (st == nullptr || provider_ == nullptr)
      return {ErrorCode::invalid_argument, "retention checkpoint position is invalid"};
    return to_status(qllm_provider_checkpoint_request_state(provider_, st->state, next_position));
  }
  Status rewind_request_state(const std::shared_ptr<IOperationProviderRequestState>& state,
                              std::uint32_t next_position) override {
    std::lock_guard lock(mutex_);
    auto* st = dynamic_cast<RequestState*>(state.get());
    if (st == nullptr || provider_ == nullptr)
      return {ErrorCode::invalid_argument, "retention rewind position is invalid"};
    return to_status(qllm_provider_rewind_request_state(provider_, st->state, next_position));
  }

  // exact_calls, accepted_drafts, accepted_depth_calls (runtime/tools/dense_fp4_provider.cpp:11313-11316)
  // are kept per request by the library (qllm_provider_telemetry); the module publishes the
  // geometry it bound.
  std::map<std::string, std::uint64_t, std::less<>> telemetry() const {
    return {{"b200_prepared", provider_ ? 1U : 0U}, {"b200_layers", config_.layers}, {"b200_draft_depth", config_.draft_depth}};
  }

 private:
  B200Nvfp4MtpOptions options_;
  std::mutex mutex_;
  qllm_provider* provider_{};
  qllm_config config_{};
  std::vector<std::shared_ptr<const ImmutableModelTensor>> retained_;
};

}  // namespace

CreateExecutionProviderModuleResult make_b200_nvfp4_mtp_callable_provider(const B200Nvfp4MtpOptions& options) {
  CreateExecutionProviderModuleResult result;
  if (!options.kv_page_tokens || options.kv_page_tokens % 128U || !options.mtp_draft_depth || options.mtp_draft_depth > 4U ||
      (options.kv_dtype != "q4-f16-per-head" && options.kv_dtype != "f16")) {
    result.status = {ErrorCode::invalid_argument, "unsupported B200 NVFP4 MTP provider options"};
    return result;
  }
  auto provider = std::make_shared<B200Nvfp4MtpProvider>(options);
  // startup validation of what the ABI range cannot express (KernelCapability::validate)
  auto validate = [depth = options.mtp_draft_depth](const ModelDescriptor& model) -> Status {
    const auto head_dim = find(model.attributes, "head_dim");
    if (!head_dim || *head_dim % 32U || *head_dim > 256U)
      return {ErrorCode::invalid_argument, "head_dim must be a multiple of 32 up to 256"};
    if (!model.routed_components.empty())
      return {ErrorCode::invalid_argument, "this adapter binds dense FFN artifacts"};
    if (!model.exact_decode_program || model.exact_decode_program->maximum_emitted_tokens != depth + 1U)
      return {ErrorCode::invalid_argument, "the artifact's exact decode depth differs from the provider's"};
    return Status::success();
  };
  const std::uint32_t abi = qllm_capability_abi();
  result.module.definition = ExecutionProviderDefinition(
      "b200-nvfp4-mtp", options.priority, {KernelCapability{qllm_capability_name(), abi, abi, validate}}, provider);
  auto& service = result.module.service;
  service.prefill_mode = "provider-chunks";
  service.prefill_chunk_tokens = 128U;
  service.session_retention = false;
  service.kv_dtype = options.kv_dtype;
  service.kv_allocation = "preallocated";
  service.kv_page_tokens = options.kv_page_tokens;
  service.mtp_resource_available = service.mtp_runtime_ready = service.mtp_enabled = true;
  service.sampling_supported = true;
  result.module.telemetry = [provider] { return provider->telemetry(); };
  result.status = Status::success();
  return result;
}

}  // namespace expert::runtime
