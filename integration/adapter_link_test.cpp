// CPU check that the reference-side adapter is real code: compiled against the reference's own
// headers, linked with the reference's registry / executor and a stub of the C ABI, and driven the
// way runtime/tests/cache_state_test.cpp:574-857 drives its fixture provider: parse an artifact that
// declares this provider's capability, register the module, bind, create the executor (which calls
// prepare_exact_decode with the artifact's tensors), open a session, synchronise, step.  The
// executor re-validates every result (runtime/src/program_executor.cpp:835-851).
#include <array>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <map>
#include <string>
#include <vector>

#include "b200_nvfp4_mtp_provider.hpp"
#include "expert/runtime/model_descriptor.hpp"
#include "qllm_b200.h"

namespace er = expert::runtime;

struct qllm_provider {   // layout of integration/stub_qllm_abi.cpp
  qllm_config config;
  unsigned states, synchronizations, executions;
  qllm_request last_request;
};
extern "C" const qllm_provider* qllm_stub_last_provider(void);

namespace {

void require(bool condition, const char* what) {
  if (!condition) {
    std::cerr << "FAIL: " << what << "\n";
    std::exit(1);
  }
}

constexpr std::uint32_t H = 64, V = 128, QH = 2, KV = 1, HD = 32, F = 64, L = 2, DV = 96;

// One host buffer per tensor: NVFP4 matrices as codes | scales | f32 weight divisor | f32 input divisor
struct Store final : er::IModelTensorStore {
  std::map<std::string, std::shared_ptr<er::ImmutableModelTensor>, std::less<>> tensors;
  unsigned resolves{};

  void add_vector(const std::string& name, std::uint32_t count) {
    auto bytes = std::make_shared<std::vector<std::byte>>(count * sizeof(float));
    const float one = 1.0F;
    for (std::uint32_t i = 0; i < count; ++i) std::memcpy(bytes->data() + i * sizeof(float), &one, sizeof(float));
    auto t = std::make_shared<er::ImmutableModelTensor>();
    t->name = name;
    t->encoding = "f32";
    t->shape = {count};
    t->data_bytes = bytes->size();
    t->value = {"tensor.f32.v1", "host", bytes, bytes->data(), bytes->size()};
    tensors[name] = std::move(t);
  }
  void add_table(const std::string& name, std::uint32_t rows, std::uint32_t cols) {
    auto bytes = std::make_shared<std::vector<std::byte>>(static_cast<std::size_t>(rows) * cols * 2U, std::byte{0x3c});
    auto t = std::make_shared<er::ImmutableModelTensor>();
    t->name = name;
    t->encoding = "bf16";
    t->shape = {rows, cols};
    t->data_bytes = bytes->size();
    t->value = {"tensor.bf16.v1", "host", bytes, bytes->data(), bytes->size()};
    tensors[name] = std::move(t);
  }
  void add_matrix(const std::string& name, std::uint32_t rows, std::uint32_t cols, bool bf16_input_divisor) {
    const std::size_t codes = static_cast<std::size_t>(rows) * cols / 2U, local = static_cast<std::size_t>(rows) * cols / 16U;
    const std::size_t tail = sizeof(float) + (bf16_input_divisor ? 2U : sizeof(float));
    auto bytes = std::make_shared<std::vector<std::byte>>(codes + local + tail, std::byte{0x21});
    std::memset(bytes->data() + codes, 0x38, local);
    const float weight_divisor = 512.0F, input_divisor = 336.0F;
    std::memcpy(bytes->data() + codes + local, &weight_divisor, sizeof(float));
    if (bf16_input_divisor) {
      std::uint32_t bits;
      std::memcpy(&bits, &input_divisor, 4);
      const std::uint16_t high = static_cast<std::uint16_t>(bits >> 16U);
      std::memcpy(bytes->data() + codes + local + sizeof(float), &high, 2);
    } else {
      std::memcpy(bytes->data() + codes + local + sizeof(float), &input_divisor, sizeof(float));
    }
    auto t = std::make_shared<er::ImmutableModelTensor>();
    t->name = name;
    t->encoding = "nvfp4-block16";
    t->quant_abi = 5U;
    t->shape = {rows, cols};
    t->data_offset = 0U;
    t->data_bytes = codes;
    t->scale_offset = codes;
    t->scale_bytes = local + tail;
    t->value = {"tensor.nvfp4.v1", "host", bytes, bytes->data(), bytes->size()};
    tensors[name] = std::move(t);
  }
  er::ResolveModelTensorResult resolve(std::string_view name) override {
    ++resolves;
    const auto it = tensors.find(name);
    if (it == tensors.end()) return {{er::ErrorCode::invalid_argument, "unknown tensor"}, {}};
    return {er::Status::success(), it->second};
  }
};

std::string u32_bits(float v) {
  std::uint32_t bits;
  std::memcpy(&bits, &v, 4);
  return std::to_string(bits);
}

}  // namespace

int main() {
  Store store;
  const std::string capability = qllm_capability_name();
  std::string artifact =
      "expert-runtime-model-v1\n"
      "model\t3\tb200.link.test\t" + std::to_string(V) + "\t4096\t" + std::to_string(H) + "\n"
      "attribute\tattention_heads\t" + std::to_string(QH) + "\n"
      "attribute\tkv_heads\t" + std::to_string(KV) + "\n"
      "attribute\thead_dim\t" + std::to_string(HD) + "\n"
      "attribute\trotary_dimension\t" + std::to_string(HD) + "\n"
      "attribute\tnorm_epsilon_f32_bits\t" + u32_bits(1e-6F) + "\n"
      "attribute\trope_theta_f32_bits\t" + u32_bits(1e6F) + "\n"
      "attribute\tintermediate_size\t" + std::to_string(F) + "\n"
      "attribute\tmtp_layers\t1\n"
      "program_input\ttoken\trequest.token\tfixture.scalar.u64.v1\n"
      "program_output\tnext_token\tresponse.token\tfixture.scalar.u64.v1\n"
      "kernel\tfixture.block.v1\t1\n"
      "kernel\t" + capability + "\t2\n"
      "exact_decode\t" + capability + "\t2\t5\n"
      "exact_decode_parameter\tdraft_depth\t4\n"
      "exact_decode_parameter\tdraft_vocabulary_size\t" + std::to_string(DV) + "\n"
      "exact_decode_parameter\tsource_mtp_layers\t1\n"
      "exact_decode_parameter\tmtp_kv_encoding\t1\n"
      "exact_decode_parameter\tembedding_first\t1\n"
      "exact_decode_parameter\tpost_norm\t1\n";
  auto bind = [&](const std::string& role, const std::string& name) {
    artifact += "model_tensor\t" + role + "\t" + name + "\n";
    return "exact_decode_tensor\t" + role + "\t" + name + "\n";
  };
  std::string exact_tensors;
  store.add_table("tok.embedding", V, H);
  exact_tensors += bind("token_embedding", "tok.embedding");
  for (const char* role : {"final_norm", "embedding_norm", "hidden_norm", "draft_norm"}) {
    store.add_vector(std::string("model.") + role, H);
    exact_tensors += bind(role, std::string("model.") + role);
  }
  store.add_matrix("model.head", V, H, false);
  exact_tensors += bind("output_head", "model.head");
  store.add_matrix("mtp.fusion", H, 2U * H, true);
  exact_tensors += bind("fusion_projection", "mtp.fusion");
  std::vector<std::string> prefixes;
  for (std::uint32_t l = 0; l < L; ++l) prefixes.push_back("layer." + std::to_string(l) + ".");
  prefixes.push_back("mtp.");
  for (const auto& prefix : prefixes) {
    store.add_vector(prefix + "input_norm", H);
    store.add_vector(prefix + "post_attention_norm", H);
    store.add_matrix(prefix + "qkv_projection", (QH + 2U * KV) * HD, H, false);
    store.add_matrix(prefix + "output_projection", H, QH * HD, true);
    store.add_matrix(prefix + "gate_up_projection", 2U * F, H, false);
    store.add_matrix(prefix + "down_projection", H, F, false);
    for (const char* role : {"input_norm", "post_attention_norm", "qkv_projection", "output_projection",
                             "gate_up_projection", "down_projection"})
      exact_tensors += bind(prefix + role, prefix + role);
  }
  // the tensor records of the exact decode program follow the model-level ones
  artifact += exact_tensors;
  for (std::uint32_t l = 0; l < L; ++l)
    artifact += "layer\t" + std::to_string(l) + "\tfixture.block.v1\t1\t-\t0\n";
  // a minimal SSA program (one model-level operation in, one per layer, one out) so that the
  // artifact is a valid schema v3 program; the fixture block provider below serves it
  {
    std::uint32_t index = 0;
    std::string value = "request.token";
    auto operation = [&](const std::string& layer, const std::string& out) {
      artifact += "operation\t" + std::to_string(index) + "\t" + layer + "\tfixture.block.v1\t1\t-\t0\n";
      artifact += "operation_input\t" + std::to_string(index) + "\tx\t" + value + "\tfixture.scalar.u64.v1\n";
      artifact += "operation_output\t" + std::to_string(index) + "\ty\t" + out + "\tfixture.scalar.u64.v1\n";
      value = out;
      ++index;
    };
    operation("-", "embedded.hidden");
    for (std::uint32_t l = 0; l < L; ++l) operation(std::to_string(l), "layer" + std::to_string(l) + ".hidden");
    operation("-", "response.token");
  }

  er::Sha256Digest hash{};
  auto parsed = er::parse_model_descriptor_artifact(artifact, hash, 1U);
  if (!parsed.status.ok()) std::cerr << parsed.status.message() << "\n";
  require(parsed.status.ok() && parsed.descriptor.exact_decode_program.has_value(), "the artifact did not parse");

  er::B200Nvfp4MtpOptions options;
  options.max_context = 2048U;
  auto wrong = options;
  wrong.kv_dtype = "fp8";
  require(!er::make_b200_nvfp4_mtp_callable_provider(wrong).status.ok(), "unsupported options were accepted");
  auto created = er::make_b200_nvfp4_mtp_callable_provider(options);
  require(created.status.ok() && created.module.definition.implementation, "the factory failed");

  // a second provider serves the ordinary operation; ours serves the exact decode service only
  struct BlockProvider final : er::IOperationProvider {
    struct Prepared final : er::IPreparedOperation {};
    struct State final : er::IOperationProviderRequestState {};
    er::PrepareOperationResult prepare(const er::OperationPreparationContext&) override {
      return {er::Status::success(), std::make_shared<Prepared>()};
    }
    er::CreateOperationRequestStateResult create_request_state(const er::ProgramRequestContext&) override {
      return {er::Status::success(), std::make_shared<State>()};
    }
    er::OperationExecutionHandle execute(const er::IPreparedOperation&,
                                         const std::shared_ptr<er::IOperationProviderRequestState>&,
                                         const er::OperationInvocation&) override {
      return {};
    }
    // stateless fixture: nothing to checkpoint
    er::Status checkpoint_request_state(const std::shared_ptr<er::IOperationProviderRequestState>&,
                                        std::uint32_t) override {
      return er::Status::success();
    }
    er::Status rewind_request_state(const std::shared_ptr<er::IOperationProviderRequestState>&, std::uint32_t) override {
      return er::Status::success();
    }
  };
  er::ExecutionProviderRegistry registry;
  require(registry.add(created.module.definition).ok(), "registering the module failed");
  require(registry.add({"fixture-blocks", 10U, {er::KernelCapability{"fixture.block.v1", 1U, 1U}},
                        std::make_shared<BlockProvider>()}).ok(), "registering the block provider failed");
  const auto bound = registry.bind(parsed.descriptor, er::ExecutionProviderBindingMode::executable);
  if (!bound.status.ok()) std::cerr << bound.status.message() << "\n";
  require(bound.status.ok() && bound.provider.program.exact_decode.has_value(), "capability negotiation failed");

  er::MoeProgramExecutor executor;
  const auto status = er::MoeProgramExecutor::create(parsed.descriptor, bound.provider, &store, executor);
  if (!status.ok()) std::cerr << status.message() << "\n";
  require(status.ok() && executor.valid(), "the executor did not prepare the exact decode program");
  const qllm_provider* stub = qllm_stub_last_provider();
  require(stub != nullptr && stub->config.layers == L && stub->config.hidden == H && stub->config.q_heads == QH &&
              stub->config.kv_heads == KV && stub->config.head_dim == HD && stub->config.ffn == F &&
              stub->config.vocab == V && stub->config.draft_vocab == DV && stub->config.draft_depth == 4U &&
              stub->config.kv_encoding == QLLM_KV_Q4H && stub->config.max_context == 2048U,
          "the adapter filled qllm_config wrongly");

  er::ProgramRequestContext context;
  context.request_id = 1U;
  context.parameters.emplace("reserved_context_tokens", 128U);
  context.parameters.emplace("sampling_seed", 77U);
  auto begun = executor.begin_session(std::move(context));
  require(begun.status.ok() && begun.session.valid() && begun.session.exact_decode_available() && stub->states == 1U,
          "the session did not create the provider's request state");
  require(begun.session.synchronize_exact_decode(110U, 1U, true).ok() && stub->synchronizations == 1U &&
              stub->last_request.sampling_seed == 77U && stub->last_request.reserved_context_tokens == 128U &&
              stub->last_request.sampling_presence_penalty_biased_ppm == 2000000U,
          "synchronisation did not reach the C ABI with the request's parameters");
  // retention through the executor's session: a checkpoint at the end of the cached stream
  // (position 2 after the one-row synchronisation at position 1), none anywhere else
  require(!begun.session.checkpoint_retention(7U).ok(), "a checkpoint away from the end of the stream was accepted");
  require(begun.session.checkpoint_retention(2U).ok(), "the retention checkpoint did not reach the C ABI");
  auto exact = begun.session.execute_exact_decode(110U, 2U, 128U);
  const auto result = exact.handle.poll();
  require(exact.status.ok() && result && result->status.ok() &&
              result->emitted_tokens == std::vector<std::uint32_t>({110U, 111U}) && result->next_token == 112U &&
              result->positions_advanced == 2U && stub->executions == 1U,
          "the step's result did not survive the executor's re-validation");
  require(!begun.session.rewind_retention(3U).ok(), "a rewind to a position that was not checkpointed was accepted");
  require(begun.session.rewind_retention(2U).ok(), "the retention rewind did not reach the C ABI");
  begun.session.cancel();
  require(stub->states == 0U, "closing the session leaked the request state");

  // a request's presence penalty and first output position reach the C ABI; an invalid one is refused
  er::ProgramRequestContext penalised;
  penalised.request_id = 2U;
  penalised.parameters.emplace("reserved_context_tokens", 128U);
  penalised.parameters.emplace("sampling_presence_penalty_biased_ppm", 2500000U);
  penalised.parameters.emplace("sampling_first_output_position", 9U);
  auto second = executor.begin_session(std::move(penalised));
  require(second.status.ok(), "second session");
  require(second.session.synchronize_exact_decode(5U, 1U, true).ok() &&
              stub->last_request.sampling_presence_penalty_biased_ppm == 2500000U &&
              stub->last_request.sampling_first_output_position == 9U,
          "the presence penalty did not reach the C ABI");
  second.session.cancel();
  er::ProgramRequestContext invalid;
  invalid.request_id = 3U;
  invalid.parameters.emplace("reserved_context_tokens", 128U);
  invalid.parameters.emplace("sampling_presence_penalty_biased_ppm", 4000001U);
  auto third = executor.begin_session(std::move(invalid));
  require(third.status.ok(), "third session");
  require(!third.session.synchronize_exact_decode(5U, 1U, true).ok(), "an invalid presence penalty was accepted");
  third.session.cancel();
  std::cout << "PASS adapter link test\n";
  return 0;
}
