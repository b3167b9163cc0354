// Test infrastructure: C entry point around the reference's own model-descriptor parser
// (runtime/src/model_descriptor.cpp, compiled unmodified from the reference tree by
// `make ref`).  It parses a runtime-model.tsv text and prints what the reference understood in
// a canonical one-line-per-section form, which tests/golden/make_descriptor_golden.py stores
// next to each input as the expected answer for the library's own parser.
#include <cstring>
#include <sstream>
#include <string>

#include "expert/runtime/model_descriptor.hpp"

namespace {

template <class Map>
void dump_map(std::ostringstream& out, const Map& map) {
  bool first = true;
  for (const auto& [key, value] : map) {
    out << (first ? "" : ",") << key << "=" << value;
    first = false;
  }
}

}  // namespace

extern "C" {

// Returns 0 and the dump (NUL-terminated, truncated to capacity) when the reference accepts the
// text, 1 and the reference's message when it rejects it.
int qref_descriptor_parse(const char* text, unsigned long bytes, char* out, unsigned long capacity) {
  namespace er = expert::runtime;
  const er::Sha256Digest digest{};
  const auto parsed = er::parse_model_descriptor_artifact(std::string_view(text, bytes), digest, 1U);
  std::ostringstream s;
  if (!parsed.status.ok()) {
    s << parsed.status.message();
  } else {
    const auto& d = parsed.descriptor;
    s << "model schema=" << d.schema_version << " architecture=" << d.architecture_id << " vocab=" << d.vocab_size
      << " context=" << d.max_context_tokens << " hidden=" << d.hidden_size << "\n";
    s << "attributes ";
    dump_map(s, d.attributes);
    s << "\ntensors ";
    dump_map(s, d.tensor_bindings);
    s << "\nkernels ";
    for (std::size_t i = 0; i < d.required_kernels.size(); ++i)
      s << (i ? "," : "") << d.required_kernels[i].capability << "@" << d.required_kernels[i].abi_version;
    s << "\nexact ";
    if (d.exact_decode_program) {
      const auto& e = *d.exact_decode_program;
      s << e.capability << "@" << e.abi_version << " emitted=" << e.maximum_emitted_tokens << " parameters ";
      dump_map(s, e.parameters);
      s << " tensors ";
      dump_map(s, e.tensor_bindings);
    } else {
      s << "none";
    }
    s << "\nlayers " << d.layer_program.size() << " operations " << d.operation_program.size() << "\ncomponents ";
    for (std::size_t i = 0; i < d.routed_components.size(); ++i) {
      const auto& c = d.routed_components[i];
      s << (i ? ";" : "") << c.name << " layers=" << c.layer_count << " experts=" << c.experts_per_layer
        << " route=" << c.route_width << " shared=" << c.shared_experts_per_layer << " hidden=" << c.hidden_size
        << " intermediate=" << c.intermediate_size << " execution=" << c.execution_capability << "@"
        << c.execution_abi << " router=" << c.router.capability << "@" << c.router.abi_version;
    }
    s << "\n";
  }
  const std::string text_out = s.str();
  if (out && capacity) {
    const std::size_t n = text_out.size() < capacity - 1U ? text_out.size() : capacity - 1U;
    std::memcpy(out, text_out.data(), n);
    out[n] = '\0';
  }
  return parsed.status.ok() ? 0 : 1;
}

}  // extern "C"
