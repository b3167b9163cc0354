// runtime-model.tsv: the artifact's model descriptor, and the negotiation of this library's
// exact-decode capability against it.  Host code only (no CUDA).
//
// Grammar and validity rules follow the reference's parser and validator
// (runtime/src/model_descriptor.cpp:492-746 records, :107-324 validate_model_descriptor,
// :326-341 routed components); the provider-side contract of the exact-decode program follows
// runtime/tools/dense_fp4_provider.cpp:2367-2470 (geometry attributes, ABI-2 parameters) and
// :2935-2966 (prepare_exact_decode).  The text is a header line followed by tab-separated
// records; every record kind has a fixed field count, numbers are plain decimal without sign,
// names ("atoms") are non-empty and free of tab / CR / LF, and maps reject duplicate keys.
#include <algorithm>
#include <charconv>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <optional>
#include <set>
#include <sstream>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

#include "../../include/qllm_b200.h"

namespace qllm {
int fail(int code, const std::string& message);  // sets qllm_last_error()
}

namespace {

using Fields = std::vector<std::string_view>;
constexpr uint32_t kModelLevel = std::numeric_limits<uint32_t>::max();  // operation without a layer ("-")

struct Endpoint { std::string value, abi; };

struct Router {
  std::string capability;
  uint32_t abi = 1;
  std::map<std::string, uint64_t> parameters;
};

struct Component {
  std::string name, execution, encoding;
  uint64_t namespace_id = 0;
  uint32_t layers = 0, experts = 0, route_width = 0, shared = 0, hidden = 0, intermediate = 0;
  uint32_t execution_abi = 1, source_abi = 0, encoding_abi = 0;
  std::map<std::string, uint64_t> attributes;
  Router router;
};

struct Layer {
  uint32_t index = 0, abi = 1, component_layer = 0;
  std::string block, component;
  std::map<std::string, uint64_t> parameters;
};

struct Operation {
  uint32_t index = 0, layer = 0, abi = 1, component_layer = 0;
  std::string capability, component;
  std::map<std::string, uint64_t> parameters;
  std::map<std::string, std::string> tensors;
  std::map<std::string, Endpoint> inputs, outputs;
};

struct ExactDecode {
  std::string capability;
  uint32_t abi = 1, emitted = 0;
  std::map<std::string, uint64_t> parameters;
  std::map<std::string, std::string> tensors;
};

}  // namespace

struct qllm_descriptor {
  uint32_t schema = 1, vocab = 0, context = 0, hidden = 0;
  std::string architecture;
  std::map<std::string, uint64_t> attributes;
  std::map<std::string, std::string> tensors;
  std::vector<Component> components;
  std::vector<std::pair<std::string, uint32_t>> kernels;
  std::vector<Layer> layers;
  std::vector<Operation> operations;
  std::map<std::string, Endpoint> inputs, outputs;
  std::optional<ExactDecode> exact;
};

namespace {

// ---- lexical level ------------------------------------------------------------------------------
bool number(std::string_view text, uint64_t& value) {
  if (text.empty()) return false;
  const auto r = std::from_chars(text.data(), text.data() + text.size(), value);
  return r.ec == std::errc{} && r.ptr == text.data() + text.size();
}
bool number(std::string_view text, uint32_t& value) {
  uint64_t wide = 0;
  if (!number(text, wide) || wide > std::numeric_limits<uint32_t>::max()) return false;
  value = static_cast<uint32_t>(wide);
  return true;
}
bool atom(std::string_view text) { return !text.empty() && text.find_first_of("\t\r\n") == std::string_view::npos; }

Fields split(std::string_view line) {
  Fields out;
  for (;;) {
    const size_t tab = line.find('\t');
    out.push_back(line.substr(0, tab));
    if (tab == std::string_view::npos) return out;
    line.remove_prefix(tab + 1);
  }
}

template <class Map, class Value>
bool insert_new(Map& map, std::string_view key, Value&& value) {
  return map.emplace(std::string(key), std::forward<Value>(value)).second;
}

// ---- record level: one handler per record kind, false = malformed line ------------------------
struct Reader {
  qllm_descriptor& d;
  bool have_model = false;

  Component* component(std::string_view name) {
    for (auto& c : d.components) if (c.name == name) return &c;
    return nullptr;
  }
  Layer* layer(uint32_t index) {
    for (auto& l : d.layers) if (l.index == index) return &l;
    return nullptr;
  }
  Operation* operation(uint32_t index) {
    for (auto& o : d.operations) if (o.index == index) return &o;
    return nullptr;
  }

  bool model(const Fields& f) {
    if (have_model || f.size() != 6 || !atom(f[2]) || !number(f[1], d.schema) || !number(f[3], d.vocab) ||
        !number(f[4], d.context) || !number(f[5], d.hidden))
      return false;
    d.architecture = f[2];
    return have_model = true;
  }
  bool attribute(const Fields& f) {
    uint64_t v = 0;
    return have_model && f.size() == 3 && atom(f[1]) && number(f[2], v) && insert_new(d.attributes, f[1], v);
  }
  bool model_tensor(const Fields& f) {
    return have_model && f.size() == 3 && atom(f[1]) && atom(f[2]) && insert_new(d.tensors, f[1], std::string(f[2]));
  }
  bool endpoint(const Fields& f) {
    if (!have_model || f.size() != 4 || !atom(f[1]) || !atom(f[2]) || !atom(f[3])) return false;
    auto& map = f[0] == "program_input" ? d.inputs : d.outputs;
    return insert_new(map, f[1], Endpoint{std::string(f[2]), std::string(f[3])});
  }
  bool kernel(const Fields& f) {
    uint32_t abi = 0;
    if (!have_model || f.size() != 3 || !atom(f[1]) || !number(f[2], abi)) return false;
    d.kernels.emplace_back(std::string(f[1]), abi);
    return true;
  }
  bool exact_decode(const Fields& f) {
    ExactDecode e;
    if (!have_model || d.exact || f.size() != 4 || !atom(f[1]) || !number(f[2], e.abi) || !number(f[3], e.emitted))
      return false;
    e.capability = f[1];
    d.exact = std::move(e);
    return true;
  }
  bool exact_parameter(const Fields& f) {
    uint64_t v = 0;
    return d.exact && f.size() == 3 && atom(f[1]) && number(f[2], v) && insert_new(d.exact->parameters, f[1], v);
  }
  bool exact_tensor(const Fields& f) {
    return d.exact && f.size() == 3 && atom(f[1]) && atom(f[2]) &&
           insert_new(d.exact->tensors, f[1], std::string(f[2]));
  }
  bool component_record(const Fields& f, uint64_t namespace_base) {
    Component c;
    uint64_t offset = 0;
    if (!have_model || f.size() != 14 || !atom(f[1]) || !atom(f[9]) || !atom(f[13]) || !number(f[2], offset) ||
        offset > std::numeric_limits<uint64_t>::max() - namespace_base || !number(f[3], c.layers) ||
        !number(f[4], c.experts) || !number(f[5], c.route_width) || !number(f[6], c.shared) ||
        !number(f[7], c.hidden) || !number(f[8], c.intermediate) || !number(f[10], c.execution_abi) ||
        !number(f[11], c.source_abi) || !number(f[12], c.encoding_abi))
      return false;
    c.name = f[1];
    c.namespace_id = namespace_base + offset;
    c.execution = f[9];
    c.encoding = f[13];
    d.components.push_back(std::move(c));
    return true;
  }
  bool component_attribute(const Fields& f) {
    uint64_t v = 0;
    Component* c = f.size() == 4 ? component(f[1]) : nullptr;
    return c && atom(f[2]) && number(f[3], v) && insert_new(c->attributes, f[2], v);
  }
  bool router(const Fields& f) {
    Component* c = f.size() == 4 ? component(f[1]) : nullptr;
    if (!c || !atom(f[2]) || !c->router.capability.empty() || !number(f[3], c->router.abi)) return false;
    c->router.capability = f[2];
    return true;
  }
  bool router_parameter(const Fields& f) {
    uint64_t v = 0;
    Component* c = f.size() == 4 ? component(f[1]) : nullptr;
    return c && !c->router.capability.empty() && atom(f[2]) && number(f[3], v) &&
           insert_new(c->router.parameters, f[2], v);
  }
  bool layer_record(const Fields& f) {
    Layer l;
    if (!have_model || f.size() != 6 || !atom(f[2]) || !number(f[1], l.index) || !number(f[3], l.abi) ||
        !number(f[5], l.component_layer))
      return false;
    l.block = f[2];
    if (f[4] != "-") {
      if (!atom(f[4])) return false;
      l.component = f[4];
    }
    d.layers.push_back(std::move(l));
    return true;
  }
  bool layer_parameter(const Fields& f) {
    uint32_t index = 0;
    uint64_t v = 0;
    Layer* l = f.size() == 4 && number(f[1], index) ? layer(index) : nullptr;
    return l && atom(f[2]) && number(f[3], v) && insert_new(l->parameters, f[2], v);
  }
  bool operation_record(const Fields& f) {
    Operation o;
    if (!have_model || f.size() != 7 || !atom(f[3]) || !number(f[1], o.index) ||
        (f[2] != "-" && !number(f[2], o.layer)) || !number(f[4], o.abi) || !number(f[6], o.component_layer))
      return false;
    if (f[2] == "-") o.layer = kModelLevel;
    o.capability = f[3];
    if (f[5] != "-") {
      if (!atom(f[5])) return false;
      o.component = f[5];
    }
    d.operations.push_back(std::move(o));
    return true;
  }
  Operation* operation_of(const Fields& f, size_t count) {
    uint32_t index = 0;
    return f.size() == count && number(f[1], index) ? operation(index) : nullptr;
  }
  bool operation_parameter(const Fields& f) {
    uint64_t v = 0;
    Operation* o = operation_of(f, 4);
    return o && atom(f[2]) && number(f[3], v) && insert_new(o->parameters, f[2], v);
  }
  bool operation_tensor(const Fields& f) {
    Operation* o = operation_of(f, 4);
    return o && atom(f[2]) && atom(f[3]) && insert_new(o->tensors, f[2], std::string(f[3]));
  }
  bool operation_port(const Fields& f) {
    Operation* o = operation_of(f, 5);
    if (!o || !atom(f[2]) || !atom(f[3]) || !atom(f[4])) return false;
    auto& map = f[0] == "operation_input" ? o->inputs : o->outputs;
    return insert_new(map, f[2], Endpoint{std::string(f[3]), std::string(f[4])});
  }

  bool record(const Fields& f, uint64_t namespace_base) {
    const std::string_view kind = f[0];
    if (kind == "model") return model(f);
    if (kind == "attribute") return attribute(f);
    if (kind == "model_tensor") return model_tensor(f);
    if (kind == "program_input" || kind == "program_output") return endpoint(f);
    if (kind == "kernel") return kernel(f);
    if (kind == "exact_decode") return exact_decode(f);
    if (kind == "exact_decode_parameter") return exact_parameter(f);
    if (kind == "exact_decode_tensor") return exact_tensor(f);
    if (kind == "component") return component_record(f, namespace_base);
    if (kind == "component_attribute") return component_attribute(f);
    if (kind == "router") return router(f);
    if (kind == "router_parameter") return router_parameter(f);
    if (kind == "layer") return layer_record(f);
    if (kind == "layer_parameter") return layer_parameter(f);
    if (kind == "operation") return operation_record(f);
    if (kind == "operation_parameter") return operation_parameter(f);
    if (kind == "operation_tensor") return operation_tensor(f);
    if (kind == "operation_input" || kind == "operation_output") return operation_port(f);
    return false;
  }
};

// ---- validity of the whole descriptor: empty string = valid ------------------------------------
const Component* find_component(const qllm_descriptor& d, std::string_view name) {
  for (const auto& c : d.components) if (c.name == name) return &c;
  return nullptr;
}

std::string check(const qllm_descriptor& d) {
  if (d.schema < 1 || d.schema > 3 || d.architecture.empty() || !d.vocab || !d.context || !d.hidden ||
      d.layers.empty() || d.kernels.empty())
    return "model descriptor architecture is incomplete";

  std::set<std::string> names;
  std::set<uint64_t> namespaces;
  for (const auto& c : d.components) {
    if (c.name.empty() || !c.namespace_id || !c.layers || !c.experts || !c.route_width || c.route_width > c.experts ||
        !c.hidden || !c.intermediate || !c.source_abi || !c.encoding_abi || c.execution.empty() || !c.execution_abi ||
        c.encoding.empty() || c.hidden != d.hidden)
      return "routed expert component geometry or identity is invalid";
    if (static_cast<uint64_t>(c.layers) * c.experts > std::numeric_limits<size_t>::max() / 128U)
      return "routed expert table exceeds addressable metadata";
    if (!names.insert(c.name).second || !namespaces.insert(c.namespace_id).second)
      return "routed expert component geometry or identity is invalid";
  }

  std::set<std::pair<std::string, uint32_t>> required;
  for (const auto& [capability, abi] : d.kernels)
    if (capability.empty() || !abi || !required.emplace(capability, abi).second)
      return "kernel requirement is invalid or duplicated";
  const auto requires_kernel = [&](const std::string& capability, uint32_t abi) {
    return required.count({capability, abi}) != 0;
  };

  if (d.exact) {
    const ExactDecode& e = *d.exact;
    if (d.schema < 3 || !e.abi || e.emitted < 2 || !requires_kernel(e.capability, e.abi))
      return "exact decode program is invalid or unsupported";
  }
  for (const auto& c : d.components) {
    if (!requires_kernel(c.execution, c.execution_abi)) return "routed component lacks its execution kernel requirement";
    const bool has_router = !c.router.capability.empty();
    if ((d.schema >= 2 && !has_router) || (has_router && (!c.router.abi || !requires_kernel(c.router.capability, c.router.abi))))
      return "routed component lacks its routing kernel requirement";
  }

  // layers: 0, 1, 2, ... in file order
  std::set<uint32_t> layer_indices;
  for (const auto& l : d.layers) {
    if (l.block.empty() || !l.abi || l.index != layer_indices.size() || !layer_indices.insert(l.index).second ||
        !requires_kernel(l.block, l.abi))
      return "layer program is invalid or lacks a kernel requirement";
    if (!l.component.empty()) {
      const Component* c = find_component(d, l.component);
      if (!c || l.component_layer >= c->layers) return "layer program references an unavailable expert component";
    } else if (l.component_layer != 0) {
      return "dense layer program has a routed component index";
    }
  }

  if (d.schema >= 2 && d.operations.empty()) return "schema v2 model descriptor lacks its operation program";
  if (!d.operations.empty()) {
    std::set<uint32_t> operation_indices, covered;
    uint32_t previous_layer = 0;
    bool first = true;
    for (const auto& o : d.operations) {
      const bool model_level = o.layer == kModelLevel;
      if (o.capability.empty() || !o.abi || o.index != operation_indices.size() ||
          !operation_indices.insert(o.index).second || (!model_level && !layer_indices.count(o.layer)) ||
          (model_level && d.schema < 3) || (!model_level && !first && o.layer < previous_layer) ||
          !requires_kernel(o.capability, o.abi))
        return "operation program is invalid or unsupported";
      if (!model_level) {
        previous_layer = o.layer;
        first = false;
        covered.insert(o.layer);
      }
      if (!o.component.empty()) {
        if (model_level) return "model-level operation references an expert component";
        const Component* c = find_component(d, o.component);
        if (!c || o.component_layer >= c->layers) return "operation program references an unavailable expert component";
      } else if (o.component_layer != 0) {
        return "model-level operation has a component-local index";
      }
    }
    if (covered != layer_indices) return "operation program indices or layer coverage are invalid";
    if (d.schema >= 2) {
      // a routed layer names its router and its expert execution as operations of that layer
      for (const auto& l : d.layers) {
        if (l.component.empty()) continue;
        const Component* c = find_component(d, l.component);
        const auto has = [&](const std::string& capability, uint32_t abi) {
          return std::any_of(d.operations.begin(), d.operations.end(), [&](const Operation& o) {
            return o.layer == l.index && o.component == l.component && o.component_layer == l.component_layer &&
                   o.capability == capability && o.abi == abi;
          });
        };
        if (!c || !has(c->router.capability, c->router.abi) || !has(c->execution, c->execution_abi))
          return "routed layer lacks explicit router or expert operations";
      }
    }
  }

  if (d.schema < 3) {
    const bool flows = std::any_of(d.operations.begin(), d.operations.end(),
                                   [](const Operation& o) { return !o.inputs.empty() || !o.outputs.empty(); });
    if (!d.inputs.empty() || !d.outputs.empty() || d.exact || flows)
      return "legacy model descriptor contains schema v3 data flow";
    return {};
  }
  // schema 3: single-assignment data flow from the program inputs to the program outputs
  if (d.inputs.empty() || d.outputs.empty()) return "schema v3 model descriptor lacks program endpoints";
  std::map<std::string, std::string> values;  // value name -> ABI
  for (const auto& [role, e] : d.inputs)
    if (!values.emplace(e.value, e.abi).second) return "schema v3 program input is invalid or duplicated";
  for (const auto& o : d.operations) {
    if (o.inputs.empty() && o.outputs.empty()) return "schema v3 operation lacks explicit data flow";
    for (const auto& [port, e] : o.inputs) {
      const auto v = values.find(e.value);
      if (v == values.end() || v->second != e.abi) return "schema v3 operation input is unavailable or has the wrong ABI";
    }
    for (const auto& [port, e] : o.outputs)
      if (!values.emplace(e.value, e.abi).second) return "schema v3 operation output has multiple producers";
  }
  for (const auto& [role, e] : d.outputs) {
    const auto v = values.find(e.value);
    if (v == values.end() || v->second != e.abi) return "schema v3 program output is unavailable or invalid";
  }
  return {};
}

template <class Map>
void dump_map(std::ostringstream& out, const Map& map) {
  bool first = true;
  for (const auto& [key, value] : map) {
    out << (first ? "" : ",") << key << "=" << value;
    first = false;
  }
}

uint32_t parameter(const std::map<std::string, uint64_t>& map, const char* key, bool* missing) {
  const auto it = map.find(key);
  if (it == map.end() || it->second > std::numeric_limits<uint32_t>::max()) {
    *missing = true;
    return 0;
  }
  return static_cast<uint32_t>(it->second);
}

float float_bits(uint32_t bits) {
  float f;
  std::memcpy(&f, &bits, sizeof(f));
  return f;
}

}  // namespace

extern "C" {

int qllm_descriptor_parse(const char* text, size_t bytes, qllm_descriptor** out) {
  if (!text || !out) return qllm::fail(QLLM_INVALID_ARGUMENT, "null descriptor text");
  *out = nullptr;
  try {
    auto d = std::make_unique<qllm_descriptor>();
    Reader reader{*d};
    std::string_view rest(text, bytes);
    bool header = false;
    size_t line_number = 0;
    while (!rest.empty()) {
      ++line_number;
      const size_t end = rest.find('\n');
      std::string_view line = rest.substr(0, end);
      rest = end == std::string_view::npos ? std::string_view{} : rest.substr(end + 1);
      if (!line.empty() && line.back() == '\r') line.remove_suffix(1);
      if (line.empty()) continue;
      if (!header) {
        if (line != "expert-runtime-model-v1")
          return qllm::fail(QLLM_INVALID_ARGUMENT, "unknown model descriptor artifact header");
        header = true;
        continue;
      }
      if (!reader.record(split(line), 1U))
        return qllm::fail(QLLM_INVALID_ARGUMENT, "malformed model descriptor line " + std::to_string(line_number));
    }
    if (!header || !reader.have_model)
      return qllm::fail(QLLM_INVALID_ARGUMENT, "model descriptor artifact is incomplete");
    const std::string problem = check(*d);
    if (!problem.empty()) return qllm::fail(QLLM_INVALID_ARGUMENT, problem);
    *out = d.release();
    return QLLM_OK;
  } catch (const std::exception& e) {
    return qllm::fail(QLLM_INTERNAL, std::string("model descriptor parsing failed: ") + e.what());
  }
}

void qllm_descriptor_destroy(qllm_descriptor* d) { delete d; }

size_t qllm_descriptor_dump(const qllm_descriptor* d, char* out, size_t capacity) {
  if (!d) return 0;
  std::ostringstream s;
  s << "model schema=" << d->schema << " architecture=" << d->architecture << " vocab=" << d->vocab
    << " context=" << d->context << " hidden=" << d->hidden << "\nattributes ";
  dump_map(s, d->attributes);
  s << "\ntensors ";
  dump_map(s, d->tensors);
  s << "\nkernels ";
  for (size_t i = 0; i < d->kernels.size(); ++i) s << (i ? "," : "") << d->kernels[i].first << "@" << d->kernels[i].second;
  s << "\nexact ";
  if (d->exact) {
    s << d->exact->capability << "@" << d->exact->abi << " emitted=" << d->exact->emitted << " parameters ";
    dump_map(s, d->exact->parameters);
    s << " tensors ";
    dump_map(s, d->exact->tensors);
  } else {
    s << "none";
  }
  s << "\nlayers " << d->layers.size() << " operations " << d->operations.size() << "\ncomponents ";
  for (size_t i = 0; i < d->components.size(); ++i) {
    const Component& c = d->components[i];
    s << (i ? ";" : "") << c.name << " layers=" << c.layers << " experts=" << c.experts << " route=" << c.route_width
      << " shared=" << c.shared << " hidden=" << c.hidden << " intermediate=" << c.intermediate
      << " execution=" << c.execution << "@" << c.execution_abi << " router=" << c.router.capability << "@"
      << c.router.abi;
  }
  s << "\n";
  const std::string text = s.str();
  if (out && capacity) {
    const size_t n = std::min(text.size(), capacity - 1);
    std::memcpy(out, text.data(), n);
    out[n] = '\0';
  }
  return text.size();
}

const char* qllm_descriptor_tensor(const qllm_descriptor* d, const char* role) {
  if (!d || !role) return nullptr;
  if (d->exact) {
    const auto it = d->exact->tensors.find(role);
    if (it != d->exact->tensors.end()) return it->second.c_str();
  }
  const auto it = d->tensors.find(role);
  return it == d->tensors.end() ? nullptr : it->second.c_str();
}

int qllm_descriptor_negotiate(const qllm_descriptor* d, qllm_config* config) {
  if (!d || !config) return qllm::fail(QLLM_INVALID_ARGUMENT, "null descriptor or configuration");
  const std::string name = qllm_capability_name();
  const uint32_t abi = qllm_capability_abi();
  // the runner admits a provider only if the artifact lists its capability with this ABI, and
  // the exact-decode program must be that capability
  const bool listed = std::any_of(d->kernels.begin(), d->kernels.end(),
                                  [&](const auto& k) { return k.first == name && k.second == abi; });
  if (!listed || !d->exact || d->exact->capability != name || d->exact->abi != abi)
    return qllm::fail(QLLM_INVALID_ARGUMENT, "the artifact does not declare " + name + " ABI " + std::to_string(abi));
  bool missing = false;
  const auto& p = d->exact->parameters;
  const uint32_t depth = parameter(p, "draft_depth", &missing);
  const uint32_t draft_vocab = parameter(p, "draft_vocabulary_size", &missing);
  const uint32_t source_layers = parameter(p, "source_mtp_layers", &missing);
  const uint32_t mtp_kv = parameter(p, "mtp_kv_encoding", &missing);
  const uint32_t embedding_first = parameter(p, "embedding_first", &missing);
  const uint32_t post_norm = parameter(p, "post_norm", &missing);
  if (missing || source_layers != 1U || !depth || depth > 4U || d->exact->emitted != depth + 1U || !draft_vocab ||
      draft_vocab > d->vocab || mtp_kv != 1U || embedding_first != 1U || post_norm != 1U)
    return qllm::fail(QLLM_INVALID_ARGUMENT, "unsupported exact-decode artifact contract");
  const auto& a = d->attributes;
  qllm_config c = *config;  // cache encoding, page size, split size and context stay the caller's
  c.layers = static_cast<uint32_t>(d->layers.size());
  c.hidden = d->hidden;
  c.vocab = d->vocab;
  c.draft_vocab = draft_vocab;
  c.draft_depth = depth;
  c.q_heads = parameter(a, "attention_heads", &missing);
  c.kv_heads = parameter(a, "kv_heads", &missing);
  c.head_dim = parameter(a, "head_dim", &missing);
  c.rotary_dim = parameter(a, "rotary_dimension", &missing);
  c.eps = float_bits(parameter(a, "norm_epsilon_f32_bits", &missing));
  c.rope_theta = float_bits(parameter(a, "rope_theta_f32_bits", &missing));
  if (missing || parameter(a, "mtp_layers", &missing) != 1U || missing)
    return qllm::fail(QLLM_INVALID_ARGUMENT, "the artifact lacks a geometry attribute of the dense attention model");
  const auto bf16 = a.find("activation_bf16");
  c.activation_bf16 = bf16 != a.end() && bf16->second == 1U ? 1U : 0U;
  c.mtp_kv_encoding = QLLM_KV_Q8;
  const auto zero_centered = a.find("zero_centered_norm");
  if (zero_centered != a.end() && zero_centered->second == 1U)
    return qllm::fail(QLLM_INVALID_ARGUMENT, "zero-centred norm weights are not supported");
  bool absent = false;
  const uint32_t ffn = parameter(a, "intermediate_size", &absent);
  if (!absent) c.ffn = ffn;  // otherwise the caller takes it from the gate projection's rows
  if (!d->components.empty()) {
    const Component& e = d->components.front();
    if (e.shared != 0U) return qllm::fail(QLLM_INVALID_ARGUMENT, "shared experts are not supported");
    c.experts = e.experts;
    c.route_width = e.route_width;
    c.expert_ffn = e.intermediate;
    if (c.route_scale == 0.0F) c.route_scale = 1.0F;
  } else {
    c.experts = c.route_width = c.expert_ffn = 0U;
  }
  if (d->context < c.max_context) c.max_context = d->context;
  *config = c;
  return QLLM_OK;
}

}  // extern "C"
