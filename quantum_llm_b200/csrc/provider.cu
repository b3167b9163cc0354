// Host side of the B200 provider: the exact-decode subset of
// expert::runtime::IOperationProvider (runtime/include/expert/runtime/program_executor.hpp:244-370)
// over the kernel layer.  Control flow follows DenseFp4Provider::execute_exact_decode,
// run_target, run_mtp, extend_mtp_rollout and synchronize_exact_decode_batch
// (runtime/tools/dense_fp4_provider.cpp:11139-11318, 8529-8635, 8681-8852, 11011-11137),
// re-arranged so that one step is a fixed launch sequence driven by device-resident
// state: verify -> accept/rollback kernel -> draft passes, with one host read at the end.
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "common.cuh"
#include "gemv_mma.h"
#include "fused.h"
#include "kernels.h"
#include "moe.h"
#include "rope_tail.cuh"

namespace qllm {

namespace {
thread_local std::string g_error;
unsigned long long g_launches = 0;
}  // namespace

void set_error(const std::string& message) { g_error = message; }
int fail(int status, const std::string& message) {
  g_error = message;
  return status;
}
int check_cuda(cudaError_t error, const char* what) {
  if (error == cudaSuccess) return 0;
  return fail(QLLM_INTERNAL, std::string(what) + ": " + cudaGetErrorString(error));
}
int check_launch(const char* what) { return check_cuda(cudaPeekAtLastError(), what); }
namespace {
int g_pdl = -1;
}
bool pdl_enabled() {
  if (g_pdl < 0) {
    const char* env = std::getenv("QLLM_PDL");  // QLLM_PDL=0: ordinary launches only
    g_pdl = (env && env[0] == '0') ? 0 : 1;
  }
  return g_pdl == 1;
}
void set_pdl_enabled(bool enabled) { g_pdl = enabled ? 1 : 0; }
void count_launch(unsigned launches) { g_launches += launches; }
unsigned long long launches_counted() { return g_launches; }

struct Error : std::runtime_error {
  int status;
  Error(int s, const std::string& m) : std::runtime_error(m), status(s) {}
};
static void ok(int rc) {
  if (rc) throw Error(rc, g_error);
}
static void cu(cudaError_t e, const char* what) { ok(check_cuda(e, what)); }

template <typename T>
struct DeviceBuffer {
  T* p = nullptr;
  size_t n = 0;
  void alloc(size_t count, const char* what) {
    release();
    if (!count) return;
    cu(cudaMalloc(&p, count * sizeof(T)), what);
    n = count;
  }
  void release() {
    if (p) cudaFree(p);
    p = nullptr;
    n = 0;
  }
  ~DeviceBuffer() { release(); }
};

struct Matrix {
  qllm_matrix m{};           // device pointers
  MmaWeights mma;            // tensor map + re-tiled scales for the tcgen05 kernel
};
struct Block {
  const float* input_norm = nullptr;
  const float* post_norm = nullptr;
  Matrix qkv, o, gate_up, down;
  // routed experts (cfg.experts != 0) replace gate_up/down: router + device arrays of descriptors
  Matrix router;
  const ExpertMatrix* expert_gate = nullptr;
  const ExpertMatrix* expert_up = nullptr;
  const ExpertMatrix* expert_down = nullptr;
};

}  // namespace qllm

using namespace qllm;

struct qllm_request_state {
  uint8_t* slab = nullptr;          // page storage
  uint8_t** page_table = nullptr;   // device array of page pointers
  uint32_t pages = 0;
  StepState* state = nullptr;       // device
  StepRecord* results = nullptr;    // device ring
  StepRecord* host_records = nullptr;  // pinned landing area of the ring
  float* retained_hidden = nullptr; // [kChunkRows, hidden] rows of the last prefill chunk
  uint32_t retained_logits_row = 0; // row of the logits buffer that holds the chunk's last position
  float* mtp_last_hidden = nullptr; // [hidden]
  // host mirror of the invocation stream invariants
  uint32_t mtp_length = 0;
  uint32_t synchronized_token = 0;
  bool draft_valid = false;
  uint32_t draft_count = 0;
  uint32_t retained_rows = 0;
  uint32_t retained_first = 0;
  uint32_t ring_cursor = 0;  // host mirror of StepState::step_index
  uint32_t retention_position = 0;  // checkpoint_request_state / rewind_request_state
  bool retention_valid = false;
  uint8_t* emitted = nullptr;       // [vocab] sampling presence: tokens this request has emitted
  float presence_penalty = 0.0F;    // of the bound request; 0 = none (no presence kernel is launched)
  bool request_bound = false;
  qllm_request request{};
  cudaGraphExec_t step_graph = nullptr;
  uint32_t graph_splits = 0, graph_mtp_splits = 0;
  int graph_sampled = -1, graph_gemv = -1;
  float graph_presence = 0.0F;      // penalty baked into the captured step
};

struct qllm_provider {
  static constexpr uint32_t kMaxRows = 8;      // kMaximumWorkspaceRows of the microbatch paths
  // widest prompt chunk: the projections see it as one operand (one pass over the weights),
  // attention takes it in tiles of kMaxRows rows, and only its last row goes through the head
  static constexpr uint32_t kChunkRows = 128;  // one activation tile of the tensor-core kernel
  uint32_t chunk_limit() const { return tp_ranks ? kMaxRows : kChunkRows; }  // exchange slots hold kMaxRows rows
  static constexpr uint32_t kResultRing = 64;
  qllm_config cfg{};
  int device = 0;
  bool borrowed = false;
  cudaStream_t stream = nullptr;
  std::recursive_mutex mutex;   // recursive: the scalar decode step is composed of the chunk, token and synchronisation calls
  std::vector<void*> owned;          // uploads
  const uint16_t* embedding = nullptr;
  std::vector<Block> layers;
  const float* final_norm = nullptr;
  Matrix head;
  const float* mtp_embedding_norm = nullptr;
  const float* mtp_hidden_norm = nullptr;
  const float* mtp_draft_norm = nullptr;
  Matrix mtp_fusion;
  Block mtp_block;
  DeviceBuffer<float> inv_freq;
  std::vector<size_t> layer_off;
  size_t page_bytes = 0;
  // workspaces (rows <= kMaxRows)
  DeviceBuffer<float> hidden, mtp_hidden, qkv, logits, mtp_emb, draft_logits, q8_scale;
  DeviceBuffer<int8_t> q8;  // INT8 copy of the rotated queries for the Q4H attention
  DeviceBuffer<float> partial_buf, gemv_out;   // tensor-core split-K partials / CUDA-core results
  DeviceBuffer<float> moe_x, moe_ws;           // routed experts: normalised input rows, selection workspace
  bool experts_aligned = true;                 // all expert tensors start on 16-byte boundaries
  // Tensor parallelism (qllm_provider_tp_export / _attach): this provider holds one rank's shard
  // (local head and FFN counts in cfg); the K-split projections (o, down) exchange partial sums.
  // Shared area of a rank: [slot 0][slot 1], slot = ranks x tp_slot_pairs {value, sequence} pairs.
  uint32_t tp_ranks = 0, tp_rank = 0;
  uint8_t* tp_area = nullptr;                  // this rank's area (cudaMalloc, exported to the peers)
  uint8_t* tp_peer[8] = {};                    // every rank's area as mapped here (own = tp_area)
  bool tp_attached = false;
  bool tp_local = false;                       // peers' areas are plain device pointers (not IPC mappings)
  size_t tp_slot_pairs = 0;
  GemvExchange tp_exchange[2] = {};            // per inbox slot (o, down)
  DeviceBuffer<uint8_t> attn_ws, topk_ws, quant_buf, full_sampler_ws;
  DeviceBuffer<uint32_t> tile_tickets;         // per-tile arrival counters of the fused RoPE tail (zero between launches)
  // QLLM_ROPE_TAIL=1: the q/k/v projection finishes every head itself (rope_tail.cuh).  Off by default:
  // measured on the 27B step it saves a launch per block but costs what the separate kernel costs
  // (qkv GEMV 10.4 -> 18.6 us against a 7.9 us RoPE kernel that overlaps its launch), 7.36 vs 7.00 ms per step.
  bool rope_tail_enabled = false;
  DeviceBuffer<uint32_t> kernel_error;         // set by a kernel whose pipeline wait ran out
  DeviceBuffer<uint32_t> argmax_out, top_tokens, tokens_dev, first_token_dev;
  DeviceBuffer<float> top_values;
  uint32_t max_splits = 0;
  int graph_mode = 0;
  int gemv_impl = 0;
  int attention_impl = 1;
  uint32_t last_rows = 0;

  // ---------------------------------------------------------------- weights
  template <typename T>
  const T* bring(const T* src, size_t count, bool on_device) {
    if (!src) throw Error(QLLM_INVALID_ARGUMENT, "missing tensor");
    if (on_device) return src;
    void* d = nullptr;
    cu(cudaMalloc(&d, count * sizeof(T)), "tensor upload allocation");
    owned.push_back(d);
    cu(cudaMemcpy(d, src, count * sizeof(T), cudaMemcpyHostToDevice), "tensor upload");
    return static_cast<const T*>(d);
  }
  Matrix bring(const qllm_matrix& m, bool on_device, uint32_t rows, uint32_t cols, const char* name) {
    if (m.rows != rows || m.cols != cols || cols % 16U || !(m.weight_scale > 0.0F) ||
        !(m.input_scale > 0.0F))
      throw Error(QLLM_INVALID_ARGUMENT, std::string("native NVFP4 matrix geometry is invalid: ") + name);
    Matrix out;
    out.m = m;
    out.m.codes = bring(m.codes, static_cast<size_t>(rows) * cols / 2U, on_device);
    out.m.scales = bring(m.scales, static_cast<size_t>(rows) * cols / 16U, on_device);
    ok(out.mma.prepare(out.m, stream));
    return out;
  }
  Block bring(const qllm_block& b, bool on_device) {
    const auto& c = cfg;
    Block out;
    out.input_norm = bring(b.input_norm, c.hidden, on_device);
    out.post_norm = bring(b.post_norm, c.hidden, on_device);
    out.qkv = bring(b.qkv, on_device, (c.q_heads + 2U * c.kv_heads) * c.head_dim, c.hidden, "qkv");
    out.o = bring(b.o, on_device, c.hidden, c.q_heads * c.head_dim, "o");
    if (!c.experts) {
      out.gate_up = bring(b.gate_up, on_device, 2U * c.ffn, c.hidden, "gate_up");
      out.down = bring(b.down, on_device, c.hidden, c.ffn, "down");
      return out;
    }
    if (!b.expert_gate || !b.expert_up || !b.expert_down) throw Error(QLLM_INVALID_ARGUMENT, "missing expert tensors");
    out.router = bring(b.router, on_device, c.experts, c.hidden, "router");
    out.router.mma.release();  // consumed by moe_router_kernel (CUDA cores) whatever the GEMV implementation
    out.expert_gate = bring_experts(b.expert_gate, on_device, c.expert_ffn, c.hidden, "expert gate");
    out.expert_up = bring_experts(b.expert_up, on_device, c.expert_ffn, c.hidden, "expert up");
    out.expert_down = bring_experts(b.expert_down, on_device, c.hidden, c.expert_ffn, "expert down");
    return out;
  }
  // Host array of `experts` descriptors -> device array of (device) descriptors.
  const ExpertMatrix* bring_experts(const qllm_matrix* src, bool on_device, uint32_t rows, uint32_t cols,
                                    const char* name) {
    std::vector<ExpertMatrix> host(cfg.experts);
    for (uint32_t e = 0; e < cfg.experts; ++e) {
      const qllm_matrix& m = src[e];
      if (m.rows != rows || m.cols != cols || cols % 16U || !(m.weight_scale > 0.0F) || !(m.input_scale > 0.0F))
        throw Error(QLLM_INVALID_ARGUMENT, std::string("native NVFP4 matrix geometry is invalid: ") + name);
      host[e].codes = bring(m.codes, static_cast<size_t>(rows) * cols / 2U, on_device);
      host[e].scales = bring(m.scales, static_cast<size_t>(rows) * cols / 16U, on_device);
      if ((reinterpret_cast<uintptr_t>(host[e].codes) | reinterpret_cast<uintptr_t>(host[e].scales)) & 15U)
        experts_aligned = false;
      host[e].weight_scale = m.weight_scale;
      host[e].input_scale = m.input_scale;
    }
    return bring(host.data(), host.size(), false);
  }

  void create(const qllm_config& config, const qllm_weights& w, bool on_device, int dev) {
    cfg = config;
    const auto& c = cfg;
    if (!c.layers || !c.hidden || !c.kv_heads || !c.q_heads || c.q_heads % c.kv_heads ||
        c.head_dim % 32U || c.head_dim > 256U || c.hidden % 16U || c.ffn % 16U || !c.page_tokens ||
        c.page_tokens % 32U || !c.draft_depth || c.draft_depth > 4U || !c.split_tokens ||
        c.split_tokens % 32U || c.draft_vocab > c.vocab || !c.draft_vocab || !c.max_context ||
        c.kv_encoding > 2U || c.mtp_kv_encoding > 2U || c.rotary_dim > c.head_dim || c.rotary_dim % 2U ||
        kMaxRows * (c.q_heads / c.kv_heads) > 64U)
      throw Error(QLLM_INVALID_ARGUMENT, "provider does not support this model geometry");
    if (c.experts && (!c.route_width || c.route_width > 8U || c.route_width > c.experts || c.experts > 256U ||
                      !c.expert_ffn || c.expert_ffn % 16U || !(c.route_scale > 0.0F)))
      throw Error(QLLM_INVALID_ARGUMENT, "provider does not support this routed-expert geometry");
    device = dev;
    borrowed = on_device;
    cu(cudaSetDevice(device), "select device");
    cu(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "create stream");
    embedding = bring(w.embedding, static_cast<size_t>(c.vocab) * c.hidden, on_device);
    for (uint32_t l = 0; l < c.layers; ++l) layers.push_back(bring(w.layers[l], on_device));
    final_norm = bring(w.final_norm, c.hidden, on_device);
    head = bring(w.head, on_device, c.vocab, c.hidden, "head");
    mtp_embedding_norm = bring(w.mtp_embedding_norm, c.hidden, on_device);
    mtp_hidden_norm = bring(w.mtp_hidden_norm, c.hidden, on_device);
    mtp_draft_norm = bring(w.mtp_draft_norm, c.hidden, on_device);
    mtp_fusion = bring(w.mtp_fusion, on_device, c.hidden, 2U * c.hidden, "fusion");
    mtp_block = bring(w.mtp_block, on_device);

    std::vector<float> inv(c.rotary_dim / 2U);
    for (uint32_t p = 0; p < inv.size(); ++p)
      inv[p] = std::pow(c.rope_theta, -2.0F * static_cast<float>(p) / static_cast<float>(c.rotary_dim));
    inv_freq.alloc(inv.size() ? inv.size() : 1, "rope table");
    if (!inv.empty())
      cu(cudaMemcpy(inv_freq.p, inv.data(), inv.size() * sizeof(float), cudaMemcpyHostToDevice), "rope table");

    size_t off = 0;
    for (uint32_t l = 0; l < c.layers; ++l) {
      layer_off.push_back(off);
      off += kv_layer_bytes(c.kv_encoding, c.page_tokens, c.kv_heads, c.head_dim);
    }
    layer_off.push_back(off);
    off += kv_layer_bytes(c.mtp_kv_encoding, c.page_tokens, c.kv_heads, c.head_dim);
    page_bytes = (off + 255U) & ~static_cast<size_t>(255U);

    const uint32_t R = kChunkRows, H = kMaxRows;  // rows of a pass; rows that reach the head and the sampler
    const uint32_t qkv_w = (c.q_heads + 2U * c.kv_heads) * c.head_dim;
    hidden.alloc(static_cast<size_t>(R) * c.hidden, "hidden");
    mtp_hidden.alloc(static_cast<size_t>(R) * c.hidden, "draft residual stream");
    qkv.alloc(static_cast<size_t>(R) * qkv_w, "rotated queries");
    q8.alloc(static_cast<size_t>(R) * c.q_heads * c.head_dim, "INT8 queries");
    q8_scale.alloc(static_cast<size_t>(R) * c.q_heads, "INT8 query scales");
    logits.alloc(static_cast<size_t>(H) * c.vocab, "logits");
    const uint32_t widest = std::max(std::max(2U * c.hidden, c.ffn), c.q_heads * c.head_dim);
    quant_buf.alloc(quant_buffer_bytes(R, widest), "quantised GEMV operand");
    size_t partial_floats = 0;
    const uint32_t shapes[7][2] = {{qkv_w, c.hidden}, {c.hidden, c.q_heads * c.head_dim}, {2U * c.ffn, c.hidden},
                                   {c.hidden, c.ffn}, {c.vocab, c.hidden}, {c.hidden, 2U * c.hidden},
                                   {c.experts ? c.experts : 16U, c.hidden}};
    uint32_t most_outputs = 0;
    for (const auto& s : shapes) {
      partial_floats = std::max(partial_floats, gemv_partial_floats(s[0] == c.vocab ? H : R, s[0], s[1]));
      most_outputs = std::max(most_outputs, s[0] == c.vocab ? 0U : s[0]);
    }
    partial_buf.alloc(partial_floats, "split-K partial sums");
    gemv_out.alloc(static_cast<size_t>(R) * most_outputs, "GEMV results");
    // [0] status, [1] [2] the tensor-parallel exchange's sequence and ticket counters
    tile_tickets.alloc(4096, "tile tickets");
    cu(cudaMemsetAsync(tile_tickets.p, 0, 4096U * sizeof(uint32_t), stream), "tile tickets");
    if (const char* env = std::getenv("QLLM_ROPE_TAIL")) rope_tail_enabled = env[0] == '1';
    kernel_error.alloc(4, "kernel status word");
    cu(cudaMemsetAsync(kernel_error.p, 0, 4U * sizeof(uint32_t), stream), "kernel status word");
    if (c.experts) {
      moe_x.alloc(static_cast<size_t>(R) * c.hidden, "routed-expert input rows");
      const size_t moe_floats = moe_workspace_floats(R, c.route_width, c.hidden, c.expert_ffn);
      moe_ws.alloc(moe_floats, "routed-expert workspace");
      // the router kernel's arrival counters at its start count from zero
      cu(cudaMemsetAsync(moe_ws.p, 0, moe_floats * sizeof(float), stream), "routed-expert workspace");
    }
    mtp_emb.alloc(static_cast<size_t>(R) * c.hidden, "draft embedding");
    draft_logits.alloc(c.draft_vocab, "draft logits");
    // the page pool keeps a few slots of slack past max_context for speculative rows
    max_splits = (c.max_context + 2U * kMaxRows + c.split_tokens - 1U) / c.split_tokens;
    attn_ws.alloc(attention_workspace_bytes(R, c.q_heads, c.head_dim, max_splits), "attention partials");
    topk_ws.alloc(topk_workspace_bytes(H, c.vocab, 64), "top-k partials");
    full_sampler_ws.alloc(full_sampler_workspace_bytes(c.vocab), "full-vocabulary sampler workspace");
    argmax_out.alloc(H, "argmax");
    top_tokens.alloc(static_cast<size_t>(H) * 64U, "top-k tokens");
    top_values.alloc(static_cast<size_t>(H) * 64U, "top-k values");
    tokens_dev.alloc(R, "token upload");
    first_token_dev.alloc(1, "first token");
    cu(cudaStreamSynchronize(stream), "provider set-up");
  }

  ~qllm_provider() {
    for (uint32_t r = 0; r < tp_ranks; ++r)
      if (tp_peer[r] && tp_peer[r] != tp_area && !tp_local) cudaIpcCloseMemHandle(tp_peer[r]);
    if (tp_area) cudaFree(tp_area);
    for (void* p : owned) cudaFree(p);
    if (stream) cudaStreamDestroy(stream);
  }

  // ------------------------------------------------------------------ ops
  // Every GEMV reads its operand from quant_buf (written by the producer kernel before it)
  // and leaves its result either as final values (CUDA-core kernel) or as split-K partials
  // (tensor-core kernel) that the consumer kernel sums and scales.
  int impl_for(const Matrix& w) const { return gemv_impl == 1 && w.mma.ready ? 1 : 0; }
  QuantSink sink_for(const Matrix& w, uint32_t rows) {
    return make_sink(impl_for(w), quant_buf.p, rows, w.m.cols, w.m.input_scale);
  }
  // `exchange_slot` (0 or 1) marks a K-split projection of a tensor-parallel rank: its partial
  // sums are exchanged with the peers.  o uses slot 0 and down slot 1, so that a rank that runs
  // ahead never writes the slot a slower peer is still reading (it cannot get two exchanges ahead:
  // every exchange is consumed, which needs the peers' parts, before the next but one is produced).
  GemvOut gemv(const Matrix& w, uint32_t rows, uint32_t row_count = 0, float* final_out = nullptr,
               int exchange_slot = -1, const RopeTail* rope_tail = nullptr) {
    if (!row_count) row_count = w.m.rows;
    GemvOut o{};
    const bool exchange = tp_ranks != 0U && exchange_slot >= 0;
    if (exchange && !tp_attached)
      throw Error(QLLM_INVALID_ARGUMENT, "tensor-parallel provider used before qllm_provider_tp_attach");
    ok(launch_gemv_core(impl_for(w), w.mma, w.m, 0U, row_count, rows, quant_buf.p, partial_buf.p,
                        final_out ? final_out : gemv_out.p, kernel_error.p, &o, stream,
                        exchange ? &tp_exchange[exchange_slot] : nullptr, rope_tail));
    return o;
  }
  // Fills the two per-slot exchange descriptors once all areas are mapped.
  void tp_describe() {
    for (uint32_t slot = 0; slot < 2U; ++slot) {
      GemvExchange x{};
      x.ranks = tp_ranks;
      x.rank = tp_rank;
      for (uint32_t r = 0; r < tp_ranks; ++r)
        x.inbox[r] = reinterpret_cast<uint2*>(tp_peer[r]) + static_cast<size_t>(slot) * tp_ranks * tp_slot_pairs;
      x.words = kernel_error.p;  // error word, then the exchange counter and the ticket counter
      x.capacity = static_cast<size_t>(tp_ranks) * tp_slot_pairs;
      tp_exchange[slot] = x;
    }
    tp_attached = true;
  }

  // x' = act(x + delta) stored to `store`; operand of `next` = quantised rmsnorm(x') * weight
  void norm_quant(const float* x, uint32_t x_stride, const GemvOut* delta, float* store, const float* weight,
                  const Matrix* next, uint32_t rows, uint32_t sink_block_offset = 0,
                  const uint32_t* row_select = nullptr, float* normalized = nullptr, bool round_normalized = false) {
    const auto& c = cfg;
    NormQuantArgs a{};
    a.x = x;
    a.x_stride = x_stride;
    a.cols = c.hidden;
    a.has_delta = delta != nullptr;
    if (delta) a.delta = *delta;
    a.bf16 = c.activation_bf16 != 0U;
    a.store = store;
    a.store_stride = c.hidden;
    a.weight = weight;
    a.eps = c.eps;
    a.sink = next ? sink_for(*next, rows) : no_sink();
    a.sink_block_offset = sink_block_offset;
    a.row_select = row_select;
    a.normalized = normalized;
    a.normalized_stride = c.hidden;
    a.round_normalized = round_normalized;
    ok(launch_residual_norm_quant(a, rows, stream));
  }

  // Routed experts in place of the dense FFN (run_router + run_routed_moe, NVFP4 branch,
  // dense_fp4_provider.cpp:8128-8166, 8207-8248).  `attention_out` is the o-projection result still
  // to be added to the residual stream `h`; the weighted expert sum becomes the new `pending`.
  void routed_experts(const Block& b, float* h, const GemvOut& attention_out, uint32_t rows, GemvOut* pending) {
    const auto& c = cfg;
    norm_quant(h, c.hidden, &attention_out, h, b.post_norm, &b.router, rows, 0U, nullptr, moe_x.p, true);
    MoeArgs a{};
    a.x = moe_x.p;
    a.x_stride = c.hidden;
    a.rows = rows;
    a.hidden = c.hidden;
    a.experts = c.experts;
    a.route_width = c.route_width;
    a.expert_ffn = c.expert_ffn;
    a.route_scale = c.route_scale;
    moe_carve_workspace(moe_ws.p, a);
    a.staged = experts_aligned;
    a.error = kernel_error.p;
    a.gate = b.expert_gate;
    a.up = b.expert_up;
    a.down = b.expert_down;
    // router projection + selection in one launch over the INT8 operand the norm kernel left
    // (the router always takes the CUDA-core operand form: its matrix has no tensor-core view)
    ok(launch_moe_router(ExpertMatrix{b.router.m.codes, b.router.m.scales, b.router.m.weight_scale, b.router.m.input_scale},
                         sink_for(b.router, rows), a, stream));
    ok(launch_moe_experts(a, stream));
    GemvOut result{};
    result.data = a.moe;  // final values: the next norm kernel adds them to the residual stream
    result.split = 0U;
    result.n = c.hidden;
    result.batch = rows;
    result.weight_scale = 1.0F;
    result.input_scale = 1.0F;
    *pending = result;
  }

  // One transformer block over `rows` rows held in hidden: attention sub-block
  // (run_full_attention + residual add) then FFN (run_ffn), pre-norm / ABI 1.
  // `h` holds the residual stream of the rows; `pending` is the GEMV result still to be added
  // to it (null for the first block of a pass) and is replaced by this block's down projection.
  void block(const Block& b, float* h, bool h_valid, GemvOut* pending, bool has_pending, uint32_t rows,
             uint32_t enc, size_t layer_offset, qllm_request_state& st, const uint32_t* first_position,
             uint32_t position_offset, uint32_t rotary_offset, uint32_t splits) {
    const auto& c = cfg;
    const bool bf = c.activation_bf16 != 0U;
    norm_quant(h_valid ? h : nullptr, c.hidden, has_pending ? pending : nullptr, h, b.input_norm, &b.qkv, rows);
    RopeStoreFusedArgs rs{};
    // decode steps on the tensor-core GEMV: every head is rotated and stored by the GEMV CTA that
    // finishes it; otherwise a RoPE / KV-store kernel consumes the projection
    const bool fused_tail = rope_tail_enabled && rows <= kMaxRows &&
                            gemv_rope_tail_supported(impl_for(b.qkv), b.qkv.mma, b.qkv.m, rows, c.head_dim, c.rotary_dim);
    if (!fused_tail) rs.qkv = gemv(b.qkv, rows);
    rs.q_out = qkv.p;
    rs.base = RopeStoreArgs{nullptr, rows, c.q_heads, c.kv_heads, c.head_dim, c.rotary_dim, inv_freq.p,
                            first_position, position_offset, rotary_offset, st.page_table, layer_offset,
                            c.page_tokens, enc, bf, gemv_impl == 0};
    // a chunk wider than kMaxRows rows goes through attention in row tiles: every row sees the
    // cache up to its own position, and the records of the whole chunk are stored before the first tile
    const uint32_t tile_rows = std::min(rows, kMaxRows);
    const bool tensor_attention = attention_impl >= 1 && enc == QLLM_KV_Q4H && c.head_dim == 128U &&
                                  tile_rows * (c.q_heads / c.kv_heads) <= 64U;
    rs.q8_out = tensor_attention ? q8.p : nullptr;
    rs.q8_scale = tensor_attention ? q8_scale.p : nullptr;
    if (fused_tail) {
      const RopeTail tail{rs.base, rs.q_out, rs.q8_out, rs.q8_scale, tile_tickets.p};
      gemv(b.qkv, rows, 0U, nullptr, -1, &tail);
    } else {
      ok(launch_rope_kv_store_fused(rs, stream));
    }
    const uint32_t qkv_w = c.q_heads * c.head_dim;  // rotated queries only
    // the full tiles go out as one launch (grid z = tile), a ragged last tile as a second one
    const uint32_t full_tiles = rows / tile_rows;
    for (uint32_t pass = 0; pass < 2U; ++pass) {
      const uint32_t r0 = pass ? full_tiles * tile_rows : 0U;
      const uint32_t n = pass ? rows - r0 : tile_rows;
      const uint32_t tiles = pass ? 1U : full_tiles;
      if (!n) continue;
      AttentionArgs at{};
      at.encoding = enc;
      at.page_table = st.page_table;
      at.layer_offset = layer_offset;
      at.page_tokens = c.page_tokens;
      at.query = qkv.p + static_cast<size_t>(r0) * qkv_w;
      at.query_row_stride = qkv_w;
      at.rows = n;
      at.first_position = first_position;
      at.position_offset = position_offset + r0;
      at.q_heads = c.q_heads;
      at.kv_heads = c.kv_heads;
      at.head_dim = c.head_dim;
      at.split_tokens = c.split_tokens;
      at.max_splits = splits;
      at.bf16 = bf;
      at.workspace = attn_ws.p;
      at.out = nullptr;  // the splits are merged by the combine + quantise kernel below
      at.impl = tensor_attention ? 1 : 0;
      if (attention_impl >= 1 && enc == QLLM_KV_Q8 && attention_q8_mma_supported(at)) at.impl = 1;
      if (attention_impl >= 1 && enc == QLLM_KV_F16 && attention_f16_mma_supported(at)) at.impl = 1;
      // tensor-memory kernel (one row tile, at most 32 matrix rows); checked below once the INT8 queries are set
      const bool want_tc = attention_impl == 2 && tensor_attention && tiles == 1U;
      at.query_q8 = rs.q8_out ? rs.q8_out + static_cast<size_t>(r0) * qkv_w : nullptr;
      at.query_q8_scale = rs.q8_scale ? rs.q8_scale + static_cast<size_t>(r0) * c.q_heads : nullptr;
      at.error = kernel_error.p;
      at.skip_combine = true;
      at.tiles = tiles;
      if (want_tc && attention_q4h_tc_supported(at)) at.impl = 2;
      ok(launch_attention(at, stream));
      CombineArgs cb{};
      const size_t items = attention_partial_items(n, splits, c.q_heads);
      cb.maxima = reinterpret_cast<const float*>(attn_ws.p);
      cb.sums = cb.maxima + items;
      cb.outputs = cb.maxima + 2U * items;
      cb.first_position = first_position;
      cb.position_offset = position_offset + r0;
      cb.q_heads = c.q_heads;
      cb.head_dim = c.head_dim;
      cb.split_tokens = c.split_tokens;
      cb.max_splits = splits;
      cb.bf16 = bf;
      cb.out = nullptr;
      cb.exact = attention_impl == 0;
      cb.sink = sink_for(b.o, rows);
      cb.sink_row_offset = r0;
      cb.tiles = tiles;
      ok(launch_combine_quant(cb, n, stream));
    }
    const GemvOut o_out = gemv(b.o, rows, 0U, nullptr, 0);
    if (c.experts) {
      routed_experts(b, h, o_out, rows, pending);
      return;
    }
    norm_quant(h, c.hidden, &o_out, h, b.post_norm, &b.gate_up, rows);
    const GemvOut gu = gemv(b.gate_up, rows);
    ok(launch_silu_quant(gu, c.ffn, bf, sink_for(b.down, rows), nullptr, stream));
    *pending = gemv(b.down, rows, 0U, nullptr, 1);
  }

  uint32_t splits_for(uint32_t tokens) const {
    return std::min(max_splits, (tokens + cfg.split_tokens - 1U) / cfg.split_tokens);
  }

  // run_target: tokens (device) at positions *first_position + r.
  void run_target(qllm_request_state& st, const uint32_t* tokens, uint32_t rows,
                  const uint32_t* first_position, uint32_t splits, bool with_head) {
    const auto& c = cfg;
    ok(launch_embedding(embedding, tokens, hidden.p, rows, c.hidden, c.vocab, stream));
    GemvOut pending{};
    for (uint32_t l = 0; l < c.layers; ++l)
      block(layers[l], hidden.p, true, &pending, l > 0U, rows, c.kv_encoding, layer_off[l], st, first_position,
            0U, 0U, splits);
    last_rows = rows;
    // last residual add (+ final norm and the head's operand)
    if (with_head && rows > kMaxRows) {
      // a wide prompt chunk: residual add of every row, then the norm and the head of the last
      // row alone (the only logits the caller can ask for); they land in row 0 of the buffer
      norm_quant(hidden.p, c.hidden, &pending, hidden.p, nullptr, nullptr, rows);
      norm_quant(hidden.p + static_cast<size_t>(rows - 1U) * c.hidden, c.hidden, nullptr, nullptr, final_norm, &head, 1U);
      const GemvOut lg = gemv(head, 1U, 0U, logits.p);
      ok(launch_gemv_finalize(lg, logits.p, stream));
      return;
    }
    norm_quant(hidden.p, c.hidden, &pending, hidden.p, with_head ? final_norm : nullptr, with_head ? &head : nullptr,
               rows);
    if (with_head) {
      const GemvOut lg = gemv(head, rows, 0U, logits.p);
      ok(launch_gemv_finalize(lg, logits.p, stream));
    }
  }

  // Candidate selection of `rows` logit rows for the sampler.
  void select_candidates(const float* values, uint32_t rows, uint32_t count, uint32_t stride,
                         bool sampled, uint32_t top_k) {
    if (sampled)
      ok(launch_topk(values, rows, count, stride, top_k, top_values.p, top_tokens.p, topk_ws.p, stream));
    else
      ok(launch_argmax(values, rows, count, stride, argmax_out.p, stream));
  }

  // run_mtp over `rows` rows: tokens (device), previous hidden rows (device),
  // cache position of row r = *first_position + position_offset + r.
  // When `select_row` is set the draft head runs on that row (device index).
  void run_mtp(qllm_request_state& st, const uint32_t* tokens, const float* previous_hidden,
               uint32_t rows, const uint32_t* first_position, uint32_t position_offset,
               uint32_t splits, bool produce, const uint32_t* select_row, bool sampled,
               uint32_t top_k, uint32_t draft_pass = 0U) {
    const auto& c = cfg;
    ok(launch_embedding(embedding, tokens, mtp_emb.p, rows, c.hidden, c.vocab, stream));
    // [norm(embedding) | norm(previous hidden)] quantised straight into the two halves of
    // the fusion projection's operand
    norm_quant(mtp_emb.p, c.hidden, nullptr, nullptr, mtp_embedding_norm, &mtp_fusion, rows, 0U);
    norm_quant(previous_hidden, c.hidden, nullptr, nullptr, mtp_hidden_norm, &mtp_fusion, rows, c.hidden / 16U);
    GemvOut pending = gemv(mtp_fusion, rows);
    // the draft block runs in its own residual buffer, so the target's rows stay readable
    block(mtp_block, mtp_hidden.p, false, &pending, true, rows, c.mtp_kv_encoding, layer_off[c.layers], st,
          first_position, position_offset, 1U, splits);
    if (!produce) {
      // a tensor-parallel rank still takes delivery of the last exchange (see gemv())
      if (tp_ranks > 1U) norm_quant(mtp_hidden.p, c.hidden, &pending, mtp_hidden.p, nullptr, nullptr, rows);
      return;
    }
    // residual add of the selected row, kept as the chained passes' previous hidden, then the
    // draft norm and the head over the draft vocabulary
    norm_quant(mtp_hidden.p, c.hidden, &pending, st.mtp_last_hidden, mtp_draft_norm, &head, 1U, 0U, select_row);
    const GemvOut lg = gemv(head, 1U, c.draft_vocab, draft_logits.p);
    ok(launch_gemv_finalize(lg, draft_logits.p, stream));
    // the draft is drawn from logits penalised by what was emitted and by the rollout's own drafts so far
    if (st.presence_penalty != 0.0F)
      ok(launch_presence_penalty(PresenceArgs{draft_logits.p, 1U, c.draft_vocab, c.draft_vocab, st.emitted, st.state,
                                              2U, draft_pass, st.presence_penalty}, stream));
    select_candidates(draft_logits.p, 1, c.draft_vocab, c.draft_vocab, sampled, top_k);
  }

  // Draft passes after the first: chained on the draft block's own last hidden.
  void rollout(qllm_request_state& st, uint32_t splits, bool sampled, uint32_t top_k,
               bool from_sync = false) {
    const auto& c = cfg;
    for (uint32_t i = 1; i < c.draft_depth; ++i) {
      run_mtp(st, &st.state->verify_tokens[i], st.mtp_last_hidden, 1, &st.state->new_position,
              i - 1U, splits, true, nullptr, sampled, top_k, i);
      DraftSampleArgs ds{st.state, argmax_out.p, top_values.p, top_tokens.p,
                         i | (i + 1U == c.draft_depth ? 0x80000000U : 0U), from_sync ? 1U : 0U,
                         st.results, kResultRing, kernel_error.p};
      ok(launch_draft_sample(ds, stream));
    }
  }

  // The launch sequence of one speculative step (captured into a graph when enabled).
  void enqueue_step(qllm_request_state& st, uint32_t splits, uint32_t mtp_splits, bool sampled,
                    uint32_t top_k) {
    const auto& c = cfg;
    const uint32_t R = c.draft_depth + 1U;
    StepState* s = st.state;
    run_target(st, s->verify_tokens, R, &s->position, splits, true);
    // presence penalty: row r is judged against the emitted tokens plus the proposals before it
    if (st.presence_penalty != 0.0F)
      ok(launch_presence_penalty(PresenceArgs{logits.p, R, c.vocab, c.vocab, st.emitted, s, 1U, 0U,
                                              st.presence_penalty}, stream));
    select_candidates(logits.p, R, c.vocab, c.vocab, sampled, top_k);
    AcceptArgs aa{s, argmax_out.p, top_values.p, top_tokens.p, st.results, kResultRing};
    ok(launch_accept(aa, stream));
    // the accepted proposals and the selected token are emitted from here on
    if (st.presence_penalty != 0.0F) ok(launch_presence_commit_step(s, st.emitted, c.vocab, stream));
    // first draft pass: accepted drafts + selected token against the target's hidden rows;
    // rows past accepted+1 are padding whose cache records are overwritten before any read
    run_mtp(st, s->mtp_tokens, hidden.p, R, &s->position, 0U, mtp_splits, true,
            &s->accepted, sampled, top_k);
    DraftSampleArgs ds{s, argmax_out.p, top_values.p, top_tokens.p,
                       0U | (c.draft_depth == 1U ? 0x80000000U : 0U), 0U, st.results, kResultRing,
                       kernel_error.p};
    ok(launch_draft_sample(ds, stream));
    rollout(st, mtp_splits, sampled, top_k);
  }

  // `bounded_top_k`: the speculative path (acceptance over sorted top-k lists) needs 0 < top_k <= 64;
  // the scalar decode fallback samples from the whole vocabulary and takes any top_k <= vocab.
  void bind_request(qllm_request_state& st, const qllm_request& rq, bool bounded_top_k = true) {
    if (rq.sampling_temperature_ppm > 2000000U ||
        (rq.sampling_temperature_ppm != 0U &&
         (rq.sampling_top_p_ppm == 0U || rq.sampling_top_p_ppm > 1000000U || rq.sampling_min_p_ppm > 1000000U)))
      throw Error(QLLM_INVALID_ARGUMENT, "invalid token sampling contract");
    if (rq.sampling_temperature_ppm != 0U && bounded_top_k &&
        (rq.sampling_top_k == 0U || rq.sampling_top_k > 64U || rq.sampling_top_k > cfg.draft_vocab))
      throw Error(QLLM_INVALID_ARGUMENT, "sampled exact decode requires bounded nonzero top-k");
    if (rq.sampling_temperature_ppm != 0U && rq.sampling_top_k > cfg.vocab)
      throw Error(QLLM_INVALID_ARGUMENT, "invalid token sampling contract");
    if (rq.reserved_context_tokens > cfg.max_context)
      throw Error(QLLM_INVALID_ARGUMENT, "request context exceeds the provider's max_context");
    if (rq.sampling_presence_penalty_biased_ppm > 4000000U)
      throw Error(QLLM_INVALID_ARGUMENT, "sampling presence penalty is invalid");
    if (rq.sampling_first_output_position >= cfg.max_context)
      throw Error(QLLM_INVALID_ARGUMENT, "request has an invalid sampling profile");
    // (biased - 2 000 000) / 1 000 000 (dense_fp4_provider.cpp:8340-8341)
    st.presence_penalty =
        static_cast<float>((static_cast<double>(rq.sampling_presence_penalty_biased_ppm) - 2000000.0) / 1000000.0);
    if (st.request_bound && !std::memcmp(&st.request, &rq, sizeof(rq))) return;
    StepState head{};
    head.seed = rq.sampling_seed;
    head.temperature_ppm = rq.sampling_temperature_ppm;
    head.top_p_ppm = rq.sampling_top_p_ppm;
    head.top_k = rq.sampling_top_k;
    head.min_p_ppm = rq.sampling_min_p_ppm;
    head.context_limit = rq.reserved_context_tokens;
    head.draft_depth = cfg.draft_depth;
    cu(cudaMemcpyAsync(st.state, &head, offsetof(StepState, position), cudaMemcpyHostToDevice, stream),
       "bind request parameters");
    st.request = rq;
    st.request_bound = true;
  }

  // Inspection calls read on the default stream, which does not order with this one.
  void settle() { cu(cudaStreamSynchronize(stream), "wait for the provider's stream"); }
  template <typename T>
  void poke(T* device_field, const T& value) {
    cu(cudaMemcpyAsync(device_field, &value, sizeof(T), cudaMemcpyHostToDevice, stream), "state update");
  }
};

// ------------------------------------------------------------------- C ABI
namespace {

template <typename F>
int guarded(F&& body) {
  try {
    body();
    return QLLM_OK;
  } catch (const Error& e) {
    return fail(e.status, e.what());
  } catch (const std::exception& e) {
    return fail(QLLM_INTERNAL, e.what());
  }
}

void check_device_error(qllm_provider& p, qllm_request_state& st) {
  uint32_t error = 0;
  cu(cudaMemcpyAsync(&error, &st.state->error, sizeof(error), cudaMemcpyDeviceToHost, p.stream), "read step status");
  cu(cudaStreamSynchronize(p.stream), "step");
  if (error) throw Error(QLLM_INTERNAL, "exact MTP step failed on the device (code " + std::to_string(error) + ")");
}

}  // namespace

extern "C" {

const char* qllm_last_error(void) { return g_error.c_str(); }
const char* qllm_capability_name(void) { return "decode.mtp.dense-full-attention.nvfp4-block16.exact.v1"; }
uint32_t qllm_capability_abi(void) { return 2U; }

int qllm_provider_create(const qllm_config* config, const qllm_weights* weights,
                         int weights_on_device, int device, qllm_provider** out) {
  if (!config || !weights || !out) return fail(QLLM_INVALID_ARGUMENT, "null provider argument");
  *out = nullptr;
  auto p = std::make_unique<qllm_provider>();
  const int rc = guarded([&] { p->create(*config, *weights, weights_on_device != 0, device); });
  if (rc) return rc;
  *out = p.release();
  return QLLM_OK;
}

void qllm_provider_destroy(qllm_provider* p) { delete p; }

int qllm_provider_create_request_state(qllm_provider* p, qllm_request_state** out) {
  if (!p || !out) return fail(QLLM_INVALID_ARGUMENT, "null request-state argument");
  *out = nullptr;
  auto st = std::make_unique<qllm_request_state>();
  const int rc = guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    st->pages = (c.max_context + 2U * qllm_provider::kMaxRows + c.page_tokens - 1U) / c.page_tokens;
    cu(cudaMalloc(&st->slab, static_cast<size_t>(st->pages) * p->page_bytes), "KV page pool");
    cu(cudaMemsetAsync(st->slab, 0, static_cast<size_t>(st->pages) * p->page_bytes, p->stream), "clear KV pages");
    std::vector<uint8_t*> table(st->pages);
    for (uint32_t i = 0; i < st->pages; ++i) table[i] = st->slab + static_cast<size_t>(i) * p->page_bytes;
    cu(cudaMalloc(&st->page_table, st->pages * sizeof(uint8_t*)), "page table");
    cu(cudaMemcpyAsync(st->page_table, table.data(), st->pages * sizeof(uint8_t*), cudaMemcpyHostToDevice, p->stream), "page table");
    cu(cudaMalloc(&st->state, sizeof(StepState)), "step state");
    cu(cudaMemsetAsync(st->state, 0, sizeof(StepState), p->stream), "step state");
    cu(cudaMalloc(&st->results, qllm_provider::kResultRing * sizeof(StepRecord)), "result ring");
    cu(cudaMemsetAsync(st->results, 0, qllm_provider::kResultRing * sizeof(StepRecord), p->stream), "result ring");
    cu(cudaMallocHost(&st->host_records, qllm_provider::kResultRing * sizeof(StepRecord)), "pinned result ring");
    cu(cudaMalloc(&st->retained_hidden, static_cast<size_t>(qllm_provider::kChunkRows) * c.hidden * sizeof(float)), "retained hidden");
    cu(cudaMalloc(&st->mtp_last_hidden, c.hidden * sizeof(float)), "draft hidden");
    // sampling presence of the request, all clear (dense_fp4_provider.cpp:5519-5525)
    cu(cudaMalloc(&st->emitted, c.vocab), "sampling presence");
    cu(cudaMemsetAsync(st->emitted, 0, c.vocab, p->stream), "sampling presence");
    cu(cudaStreamSynchronize(p->stream), "request state set-up");
  });
  if (rc) {
    qllm_provider_destroy_request_state(p, st.release());
    return rc;
  }
  *out = st.release();
  return QLLM_OK;
}

void qllm_provider_destroy_request_state(qllm_provider* p, qllm_request_state* st) {
  if (!st) return;
  if (p) cudaSetDevice(p->device);
  if (p) cudaStreamSynchronize(p->stream);  // chunks may still be in flight
  if (st->step_graph) cudaGraphExecDestroy(st->step_graph);
  cudaFree(st->slab);
  cudaFree(st->page_table);
  cudaFree(st->state);
  cudaFree(st->results);
  if (st->host_records) cudaFreeHost(st->host_records);
  cudaFree(st->retained_hidden);
  cudaFree(st->mtp_last_hidden);
  cudaFree(st->emitted);
  delete st;
}

int qllm_provider_prefill_chunk(qllm_provider* p, qllm_request_state* st, const uint32_t* tokens,
                                uint32_t count, uint32_t first_position) {
  if (!p || !st || !tokens) return fail(QLLM_INVALID_ARGUMENT, "null prefill argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    if (!count || count > p->chunk_limit() || first_position + count > c.max_context)
      throw Error(QLLM_INVALID_ARGUMENT, "invalid target-model microbatch");
    for (uint32_t r = 0; r < count; ++r)
      if (tokens[r] >= c.vocab) throw Error(QLLM_INVALID_ARGUMENT, "target token exceeds vocabulary");
    cu(cudaMemcpyAsync(p->tokens_dev.p, tokens, count * sizeof(uint32_t), cudaMemcpyHostToDevice, p->stream), "upload embedding token batch");
    p->poke(&st->state->position, first_position);
    p->run_target(*st, p->tokens_dev.p, count, &st->state->position, p->splits_for(first_position + count), true);
    cu(cudaMemcpyAsync(st->retained_hidden, p->hidden.p, static_cast<size_t>(count) * c.hidden * sizeof(float),
                       cudaMemcpyDeviceToDevice, p->stream), "retain target hidden rows");
    // no wait here: the next chunk is enqueued while this one runs; the call that returns a
    // token or a draft (first_token, the producing synchronisation batch) waits and reports
    st->retained_rows = count;
    st->retained_first = first_position;
    st->retained_logits_row = count > qllm_provider::kMaxRows ? 0U : count - 1U;
  });
}

int qllm_provider_first_token(qllm_provider* p, qllm_request_state* st, const qllm_request* rq,
                              uint32_t sample_position, uint32_t* token) {
  if (!p || !st || !rq || !token) return fail(QLLM_INVALID_ARGUMENT, "null first-token argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    if (!st->retained_rows) throw Error(QLLM_INVALID_ARGUMENT, "no prefill rows retained");
    p->bind_request(*st, *rq, false);
    const bool sampled = rq->sampling_temperature_ppm != 0U;
    float* row = p->logits.p + static_cast<size_t>(st->retained_logits_row) * c.vocab;
    // the scalar head penalises and marks output positions only (dense_fp4_provider.cpp:8440-8453, :8514-8516)
    const bool penalised = st->presence_penalty != 0.0F && sample_position >= rq->sampling_first_output_position;
    if (penalised)
      ok(launch_presence_penalty(PresenceArgs{row, 1U, c.vocab, c.vocab, st->emitted, nullptr, 0U, 0U,
                                              st->presence_penalty}, p->stream));
    if (sampled && (rq->sampling_top_k == 0U || rq->sampling_top_k > 64U)) {
      // no truncation, or more candidates than the sorted top-k kernels hold: order the whole row
      const FullSampleParams q{rq->sampling_seed, rq->sampling_temperature_ppm, rq->sampling_top_p_ppm,
                               rq->sampling_top_k, rq->sampling_min_p_ppm, sample_position};
      ok(launch_full_vocabulary_sample(q, row, c.vocab, p->full_sampler_ws.p, &st->state->error,
                                       p->first_token_dev.p, p->stream));
    } else {
      p->select_candidates(row, 1, c.vocab, c.vocab, sampled, rq->sampling_top_k);
      ok(launch_first_token(st->state, p->argmax_out.p, p->top_values.p, p->top_tokens.p, sample_position,
                            p->first_token_dev.p, p->stream));
    }
    if (penalised) ok(launch_presence_commit_token(p->first_token_dev.p, st->emitted, c.vocab, p->stream));
    cu(cudaMemcpyAsync(token, p->first_token_dev.p, sizeof(uint32_t), cudaMemcpyDeviceToHost, p->stream), "copy first token");
    check_device_error(*p, *st);
  });
}

int qllm_provider_synchronize_exact_decode_batch(qllm_provider* p, qllm_request_state* st,
                                                 const qllm_request* rq, const uint32_t* next_tokens,
                                                 uint32_t count, uint32_t first_target_position,
                                                 int produce_final_draft) {
  if (!p || !st || !rq || !next_tokens) return fail(QLLM_INVALID_ARGUMENT, "null synchronization argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    if (!count || count > p->chunk_limit() || count != st->retained_rows ||
        first_target_position != st->retained_first || st->mtp_length != first_target_position ||
        first_target_position + count + 1U > c.max_context)
      throw Error(QLLM_INVALID_ARGUMENT, "MTP synchronization stream is invalid");
    for (uint32_t r = 0; r < count; ++r)
      if (next_tokens[r] >= c.vocab) throw Error(QLLM_INVALID_ARGUMENT, "MTP synchronization stream is invalid");
    const bool produce = produce_final_draft != 0;
    p->bind_request(*st, *rq, produce);
    const bool sampled = rq->sampling_temperature_ppm != 0U;
    if (produce && (rq->reserved_context_tokens > c.max_context ||
                    first_target_position + count + 1U >= rq->reserved_context_tokens))
      throw Error(QLLM_INVALID_ARGUMENT, "MTP rollout root exceeds context");
    st->draft_valid = false;
    st->synchronized_token = next_tokens[count - 1U];
    cu(cudaMemcpyAsync(p->tokens_dev.p, next_tokens, count * sizeof(uint32_t), cudaMemcpyHostToDevice, p->stream), "upload MTP token batch");
    StepState* s = st->state;
    p->poke(&s->position, first_target_position);
    p->poke(&s->new_position, first_target_position + count);
    p->poke(&s->accepted, count - 1U);
    p->poke(&s->next_token, st->synchronized_token);
    p->poke(&s->draft_count, 0U);
    const uint32_t splits = p->splits_for(first_target_position + count + c.draft_depth);
    p->run_mtp(*st, p->tokens_dev.p, st->retained_hidden, count, &s->position, 0U, splits, produce,
               &s->accepted, sampled, rq->sampling_top_k);
    if (produce) {
      DraftSampleArgs ds{s, p->argmax_out.p, p->top_values.p, p->top_tokens.p,
                         0U | (c.draft_depth == 1U ? 0x80000000U : 0U), 1U, st->results,
                         qllm_provider::kResultRing, p->kernel_error.p};
      ok(launch_draft_sample(ds, p->stream));
      p->rollout(*st, splits, sampled, rq->sampling_top_k, true);
      uint32_t drafts = 0;
      cu(cudaMemcpyAsync(&drafts, &s->draft_count, sizeof(drafts), cudaMemcpyDeviceToHost, p->stream), "read draft count");
      check_device_error(*p, *st);
      st->draft_count = drafts;
      st->draft_valid = drafts != 0U;
    } else {
      p->poke(&s->position, first_target_position + count);  // stream-ordered, like the pass itself
    }
    st->mtp_length = first_target_position + count;
    st->retained_rows = 0;
  });
}

static void run_steps(qllm_provider* p, qllm_request_state* st, const qllm_request* rq,
                      uint32_t context_limit, uint32_t steps, qllm_exact_result* results) {
  const auto& c = p->cfg;
  const uint32_t R = c.draft_depth + 1U;
  if (!steps || steps > qllm_provider::kResultRing)
    throw Error(QLLM_INVALID_ARGUMENT, "step count exceeds the result ring");
  // every enqueued step may advance by up to R positions and writes R speculative rows
  const uint32_t reach = st->mtp_length + steps * R + 2U * c.draft_depth + 2U;
  if (reach >= context_limit)
    throw Error(QLLM_INVALID_ARGUMENT, "multi-draft MTP state is invalid: too close to the context limit");
  const bool sampled = rq->sampling_temperature_ppm != 0U;
  // the split count is part of the captured graph: size it for a fixed horizon so that
  // single-step and batched calls share one graph until the context crosses a split
  const uint32_t horizon = std::max(steps, 32U);
  const uint32_t splits = p->splits_for(st->mtp_length + horizon * R + R);
  const uint32_t mtp_splits = splits;
  StepState* s = st->state;
  const uint32_t ring_start = st->ring_cursor;
  if (p->graph_mode) {
    if (!st->step_graph || st->graph_splits != splits || st->graph_sampled != static_cast<int>(sampled) ||
        st->graph_gemv != p->gemv_impl + 2 * p->attention_impl || st->graph_presence != st->presence_penalty) {
      if (st->step_graph) { cudaGraphExecDestroy(st->step_graph); st->step_graph = nullptr; }
      cudaGraph_t graph = nullptr;
      cu(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal), "begin step capture");
      try {
        p->enqueue_step(*st, splits, mtp_splits, sampled, rq->sampling_top_k);
      } catch (...) {
        cudaStreamEndCapture(p->stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        throw;
      }
      cu(cudaStreamEndCapture(p->stream, &graph), "end step capture");
      const cudaError_t e = cudaGraphInstantiate(&st->step_graph, graph, 0);
      cudaGraphDestroy(graph);
      cu(e, "instantiate step graph");
      st->graph_splits = splits;
      st->graph_sampled = sampled;
      st->graph_gemv = p->gemv_impl + 2 * p->attention_impl;  // kernel selection baked into the graph
      st->graph_presence = st->presence_penalty;
    }
    for (uint32_t i = 0; i < steps; ++i) cu(cudaGraphLaunch(st->step_graph, p->stream), "launch step graph");
  } else {
    for (uint32_t i = 0; i < steps; ++i) p->enqueue_step(*st, splits, mtp_splits, sampled, rq->sampling_top_k);
  }
  // one copy when the records are contiguous in the ring, two when they wrap
  const uint32_t cap = qllm_provider::kResultRing;
  const uint32_t begin = ring_start % cap;
  const uint32_t head_count = std::min(steps, cap - begin);
  cu(cudaMemcpyAsync(st->host_records + begin, st->results + begin, head_count * sizeof(StepRecord),
                     cudaMemcpyDeviceToHost, p->stream), "read step results");
  if (head_count < steps)
    cu(cudaMemcpyAsync(st->host_records, st->results, (steps - head_count) * sizeof(StepRecord),
                       cudaMemcpyDeviceToHost, p->stream), "read step results");
  cu(cudaStreamSynchronize(p->stream), "step");
  const StepRecord& last = st->host_records[(ring_start + steps - 1U) % cap];
  if (last.error)
    throw Error(QLLM_INTERNAL, "exact MTP step failed on the device (code " + std::to_string(last.error) + ")");
  const uint32_t drafts = last.draft_count;
  st->ring_cursor += steps;
  for (uint32_t i = 0; i < steps; ++i) {
    results[i] = st->host_records[(ring_start + i) % cap].result;
    st->mtp_length += results[i].positions_advanced;
    st->synchronized_token = results[i].next_token;
  }
  st->draft_count = drafts;
  st->draft_valid = drafts != 0U;
}

// checkpoint_request_state (dense_fp4_provider.cpp:9209-9269) for a full-attention model: the cache
// is append-only and rolled back by overwriting, so the checkpoint is the position itself; the
// reference additionally copies recurrent, PLE and sliding-window state, which this provider's
// models do not have.
int qllm_provider_checkpoint_request_state(qllm_provider* p, qllm_request_state* st, uint32_t next_position) {
  if (!p || !st) return fail(QLLM_INVALID_ARGUMENT, "null retention argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    if (next_position == 0U || next_position > p->cfg.max_context || st->retained_rows != 0U)
      throw Error(QLLM_INVALID_ARGUMENT, "retention checkpoint position is invalid");
    if (st->retention_position == next_position && st->mtp_length != next_position) {
      st->retention_valid = true;   // the state has moved on; the older checkpoint is declared valid again
      return;
    }
    if (st->mtp_length != next_position)
      throw Error(QLLM_INVALID_ARGUMENT, "retention checkpoint position is invalid");
    st->retention_position = next_position;
    st->retention_valid = true;
  });
}

// rewind_request_state (dense_fp4_provider.cpp:9271-9338): back to the checkpointed position; the
// drafts are dropped, so the next call is a chunk (or a scalar decode step) at next_position
// followed by a synchronisation batch that primes the drafts again.
int qllm_provider_rewind_request_state(qllm_provider* p, qllm_request_state* st, uint32_t next_position) {
  if (!p || !st) return fail(QLLM_INVALID_ARGUMENT, "null retention argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    if (!st->retention_valid || st->retention_position != next_position || st->retained_rows != 0U)
      throw Error(QLLM_INVALID_ARGUMENT, "retention rewind position is invalid");
    st->mtp_length = next_position;
    st->draft_valid = false;
    st->draft_count = 0U;
    st->retained_rows = 0U;
    p->poke(&st->state->position, next_position);
    p->poke(&st->state->draft_count, 0U);
  });
}

// One non-speculative decode step (the runner's start_step fallback, moe_vm_runner.cpp:349-360 and
// 1151-1157): the token at `position` through the target model, the next token chosen by the
// request's sampler -- any top_k, the whole vocabulary included -- at sample position `position`
// (run_head is called with current_position, dense_fp4_provider.cpp:10962-10964), and the draft
// cache kept in step by a one-row synchronisation batch
// (produce_final_draft as in qllm_provider_synchronize_exact_decode_batch; it needs a request the
// speculative path accepts).
int qllm_provider_scalar_decode(qllm_provider* p, qllm_request_state* st, const qllm_request* rq,
                                uint32_t token, uint32_t position, int produce_final_draft,
                                uint32_t* next_token) {
  if (!p || !st || !rq || !next_token) return fail(QLLM_INVALID_ARGUMENT, "null scalar-decode argument");
  std::lock_guard<std::recursive_mutex> lock(p->mutex);
  if (st->retained_rows != 0U || position != st->mtp_length)
    return fail(QLLM_INVALID_ARGUMENT, "scalar decode position is not the end of the cached stream");
  int rc = qllm_provider_prefill_chunk(p, st, &token, 1U, position);
  if (rc) return rc;
  rc = qllm_provider_first_token(p, st, rq, position, next_token);
  if (rc) { st->retained_rows = 0U; return rc; }
  return qllm_provider_synchronize_exact_decode_batch(p, st, rq, next_token, 1U, position, produce_final_draft);
}

int qllm_provider_execute_exact_decode(qllm_provider* p, qllm_request_state* st,
                                       const qllm_request* rq, uint32_t guaranteed_token,
                                       uint32_t position, uint32_t context_limit,
                                       qllm_exact_result* result) {
  if (!p || !st || !rq || !result) return fail(QLLM_INVALID_ARGUMENT, "null exact-decode argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    if (!st->draft_valid || guaranteed_token != st->synchronized_token || position != st->mtp_length ||
        position + 1U >= context_limit || context_limit > p->cfg.max_context ||
        context_limit != rq->reserved_context_tokens)
      throw Error(QLLM_INVALID_ARGUMENT, "exact MTP invocation stream is invalid");
    p->bind_request(*st, *rq);
    // the invocation's position, proposal count and guaranteed token travel to the device
    // cursor with the call (they equal what the previous step left there)
    const uint32_t cursor[3] = {position, st->draft_count, guaranteed_token};
    static_assert(offsetof(StepState, draft_count) == offsetof(StepState, position) + 4U &&
                      offsetof(StepState, verify_tokens) == offsetof(StepState, position) + 8U,
                  "cursor fields must be adjacent");
    cu(cudaMemcpyAsync(&st->state->position, cursor, sizeof(cursor), cudaMemcpyHostToDevice, p->stream),
       "upload invocation cursor");
    run_steps(p, st, rq, context_limit, 1U, result);
  });
}

int qllm_provider_execute_exact_decode_steps(qllm_provider* p, qllm_request_state* st,
                                             const qllm_request* rq, uint32_t context_limit,
                                             uint32_t steps, qllm_exact_result* results) {
  if (!p || !st || !rq || !results) return fail(QLLM_INVALID_ARGUMENT, "null exact-decode argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    if (!st->draft_valid || context_limit > p->cfg.max_context || context_limit != rq->reserved_context_tokens)
      throw Error(QLLM_INVALID_ARGUMENT, "exact MTP invocation stream is invalid");
    p->bind_request(*st, *rq);
    run_steps(p, st, rq, context_limit, steps, results);
  });
}

int qllm_provider_telemetry(qllm_provider* p, qllm_request_state* st, uint64_t* out, uint32_t count) {
  if (!p || !st || !out || count < 8U) return fail(QLLM_INVALID_ARGUMENT, "telemetry needs 8 slots");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    cu(cudaStreamSynchronize(p->stream), "sync");
    StepState host;
    p->settle();
    cu(cudaMemcpy(&host, st->state, offsetof(StepState, drafts), cudaMemcpyDeviceToHost), "read counters");
    std::memset(out, 0, count * sizeof(uint64_t));
    out[0] = host.exact_calls;
    out[1] = host.accepted_drafts;
    for (int i = 0; i < 5; ++i) out[2 + i] = host.accepted_depth_calls[i];
    out[7] = launches_counted();
  });
}

void* qllm_provider_stream(qllm_provider* p) { return p ? static_cast<void*>(p->stream) : nullptr; }
uint32_t qllm_provider_max_chunk_rows(const qllm_provider* p) { return p ? p->chunk_limit() : 0U; }

int qllm_provider_set_graph_mode(qllm_provider* p, int enabled) {
  if (!p) return fail(QLLM_INVALID_ARGUMENT, "null provider");
  p->graph_mode = enabled != 0;
  return QLLM_OK;
}
int qllm_provider_set_gemv_impl(qllm_provider* p, int impl) {
  if (!p || impl < 0 || impl > 1) return fail(QLLM_INVALID_ARGUMENT, "unknown GEMV implementation");
  p->gemv_impl = impl;
  return QLLM_OK;
}

int qllm_provider_tp_export(qllm_provider* p, uint32_t rank, uint32_t ranks, void* handle) {
  if (!p || !handle || !ranks || ranks > 8U || rank >= ranks)
    return fail(QLLM_INVALID_ARGUMENT, "tensor parallelism needs 1..8 ranks and a handle buffer");
  if (p->tp_area) return fail(QLLM_INVALID_ARGUMENT, "the exchange area of this provider exists already");
  if (p->cfg.experts) return fail(QLLM_INVALID_ARGUMENT, "tensor parallelism is built for the dense model only");
  return guarded([&] {
    const auto& c = p->cfg;
    cu(cudaSetDevice(p->device), "select device");
    // one slot holds every rank's partials of the larger of the two K-split projections
    const size_t per_rank = std::max(gemv_partial_floats(qllm_provider::kMaxRows, c.hidden, c.q_heads * c.head_dim),
                                     gemv_partial_floats(qllm_provider::kMaxRows, c.hidden, c.ffn));
    p->tp_slot_pairs = (per_rank + 63U) & ~static_cast<size_t>(63U);
    const size_t bytes = 2U * ranks * p->tp_slot_pairs * sizeof(uint2);
    void* area = nullptr;
    cu(cudaMalloc(&area, bytes), "allocate the exchange area");
    p->tp_area = static_cast<uint8_t*>(area);
    cu(cudaMemset(area, 0, bytes), "clear the exchange area");
    cu(cudaDeviceSynchronize(), "exchange set-up");
    cudaIpcMemHandle_t h{};
    static_assert(sizeof(h) == QLLM_TP_HANDLE_BYTES, "handle size");
    cu(cudaIpcGetMemHandle(&h, area), "export the exchange area");
    std::memcpy(handle, &h, sizeof(h));
    p->tp_ranks = ranks;
    p->tp_rank = rank;
    p->tp_peer[rank] = p->tp_area;
    if (ranks == 1U) p->tp_describe();
  });
}

int qllm_provider_tp_attach(qllm_provider* p, const void* handles) {
  if (!p || !handles || !p->tp_area) return fail(QLLM_INVALID_ARGUMENT, "call qllm_provider_tp_export first");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    for (uint32_t r = 0; r < p->tp_ranks; ++r) {
      if (r == p->tp_rank || p->tp_peer[r]) continue;
      cudaIpcMemHandle_t h{};
      std::memcpy(&h, static_cast<const uint8_t*>(handles) + static_cast<size_t>(r) * sizeof(h), sizeof(h));
      void* mapped = nullptr;
      cu(cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess), "map a peer's exchange area");
      p->tp_peer[r] = static_cast<uint8_t*>(mapped);
    }
    if (!p->tp_attached) p->tp_describe();
  });
}

size_t qllm_provider_tp_area_bytes(const qllm_provider* p) {
  return p && p->tp_area ? 2U * static_cast<size_t>(p->tp_ranks) * p->tp_slot_pairs * sizeof(uint2) : 0U;
}

// Exchange areas that are addressable from this process already (one process driving several GPUs
// with peer access enabled): device pointers instead of inter-process handles.
int qllm_provider_tp_attach_local(qllm_provider* p, void* const* areas) {
  if (!p || !areas || !p->tp_area) return fail(QLLM_INVALID_ARGUMENT, "call qllm_provider_tp_export first");
  if (p->tp_attached) return fail(QLLM_INVALID_ARGUMENT, "the exchange areas of this provider are attached already");
  for (uint32_t r = 0; r < p->tp_ranks; ++r) {
    if (r == p->tp_rank) continue;
    if (!areas[r] || (reinterpret_cast<uintptr_t>(areas[r]) & 15U))
      return fail(QLLM_INVALID_ARGUMENT, "a peer's exchange area is missing or not 16-byte aligned");
  }
  for (uint32_t r = 0; r < p->tp_ranks; ++r)
    if (r != p->tp_rank) p->tp_peer[r] = static_cast<uint8_t*>(areas[r]);
  p->tp_local = true;
  p->tp_describe();
  return QLLM_OK;
}

int qllm_provider_set_attention_impl(qllm_provider* p, int impl) {
  if (!p || impl < 0 || impl > 2) return fail(QLLM_INVALID_ARGUMENT, "unknown attention implementation");
  p->attention_impl = impl;
  return QLLM_OK;
}

int qllm_provider_read_logits(qllm_provider* p, float* out, uint32_t rows) {
  if (!p || !out || rows > qllm_provider::kMaxRows) return fail(QLLM_INVALID_ARGUMENT, "invalid logits read");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    cu(cudaStreamSynchronize(p->stream), "sync");
    p->settle();
    cu(cudaMemcpy(out, p->logits.p, static_cast<size_t>(rows) * p->cfg.vocab * sizeof(float), cudaMemcpyDeviceToHost), "read logits");
  });
}
int qllm_provider_read_hidden(qllm_provider* p, qllm_request_state* st, int which, float* out, uint32_t rows) {
  if (!p || !st || !out || rows > qllm_provider::kMaxRows) return fail(QLLM_INVALID_ARGUMENT, "invalid hidden read");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    cu(cudaStreamSynchronize(p->stream), "sync");
    const float* src = which ? p->hidden.p : st->retained_hidden;
    p->settle();
    cu(cudaMemcpy(out, src, static_cast<size_t>(rows) * p->cfg.hidden * sizeof(float), cudaMemcpyDeviceToHost), "read hidden");
  });
}
int qllm_provider_read_drafts(qllm_provider* p, qllm_request_state* st, uint32_t* tokens, uint32_t* count) {
  if (!p || !st || !tokens || !count) return fail(QLLM_INVALID_ARGUMENT, "invalid drafts read");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    cu(cudaStreamSynchronize(p->stream), "sync");
    StepState host;
    p->settle();
    cu(cudaMemcpy(&host, st->state, offsetof(StepState, drafts), cudaMemcpyDeviceToHost), "read drafts");
    *count = host.draft_count;
    for (uint32_t i = 0; i < host.draft_count && i < 4U; ++i) tokens[i] = host.verify_tokens[i + 1U];
  });
}
// Measurement aid: the verify pass alone (target forward over the pending guaranteed token and
// drafts, head, candidate selection), `repeats` times back to back, timed with CUDA events on the
// provider's stream.  It recomputes what the next step computes anyway (same inputs, same cache
// slots), so the request can go on decoding afterwards.
int qllm_provider_time_verify(qllm_provider* p, qllm_request_state* st, const qllm_request* rq, uint32_t repeats,
                              float* mean_ms) {
  if (!p || !st || !rq || !mean_ms || !repeats) return fail(QLLM_INVALID_ARGUMENT, "null verify-timing argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    if (!st->draft_valid) throw Error(QLLM_INVALID_ARGUMENT, "no drafts are pending: nothing to verify");
    p->bind_request(*st, *rq);
    const bool sampled = rq->sampling_temperature_ppm != 0U;
    const uint32_t R = c.draft_depth + 1U;
    const uint32_t splits = p->splits_for(st->mtp_length + 33U * R);
    auto enqueue = [&] {
      p->run_target(*st, st->state->verify_tokens, R, &st->state->position, splits, true);
      p->select_candidates(p->logits.p, R, c.vocab, c.vocab, sampled, rq->sampling_top_k);
    };
    cudaGraphExec_t exec = nullptr;
    if (p->graph_mode) {
      cudaGraph_t graph = nullptr;
      cu(cudaStreamBeginCapture(p->stream, cudaStreamCaptureModeThreadLocal), "begin verify capture");
      try {
        enqueue();
      } catch (...) {
        cudaStreamEndCapture(p->stream, &graph);
        if (graph) cudaGraphDestroy(graph);
        throw;
      }
      cu(cudaStreamEndCapture(p->stream, &graph), "end verify capture");
      const cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
      cudaGraphDestroy(graph);
      cu(e, "instantiate verify graph");
    }
    cudaEvent_t a = nullptr, b = nullptr;
    cu(cudaEventCreate(&a), "event");
    cu(cudaEventCreate(&b), "event");
    auto run = [&] {
      if (exec) cu(cudaGraphLaunch(exec, p->stream), "launch verify graph");
      else enqueue();
    };
    run();  // warm-up
    cu(cudaEventRecord(a, p->stream), "event record");
    for (uint32_t i = 0; i < repeats; ++i) run();
    cu(cudaEventRecord(b, p->stream), "event record");
    cu(cudaStreamSynchronize(p->stream), "verify timing");
    float ms = 0.0F;
    cu(cudaEventElapsedTime(&ms, a, b), "event time");
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (exec) cudaGraphExecDestroy(exec);
    *mean_ms = ms / static_cast<float>(repeats);
  });
}

size_t qllm_provider_page_bytes(qllm_provider* p) { return p ? p->page_bytes : 0; }
size_t qllm_provider_layer_offset(qllm_provider* p, uint32_t layer) {
  return p && layer < p->layer_off.size() ? p->layer_off[layer] : 0;
}
int qllm_provider_read_page(qllm_provider* p, qllm_request_state* st, uint32_t page, uint8_t* out) {
  if (!p || !st || !out || page >= st->pages) return fail(QLLM_INVALID_ARGUMENT, "invalid page read");
  return guarded([&] {
    cu(cudaSetDevice(p->device), "select device");
    cu(cudaStreamSynchronize(p->stream), "sync");
    p->settle();
    cu(cudaMemcpy(out, st->slab + static_cast<size_t>(page) * p->page_bytes, p->page_bytes, cudaMemcpyDeviceToHost), "read page");
  });
}

int qllm_provider_fill_synthetic_kv(qllm_provider* p, qllm_request_state* st, uint32_t first,
                                    uint32_t count, uint64_t seed) {
  if (!p || !st) return fail(QLLM_INVALID_ARGUMENT, "null synthetic-fill argument");
  return guarded([&] {
    std::lock_guard<std::recursive_mutex> lock(p->mutex);
    cu(cudaSetDevice(p->device), "select device");
    const auto& c = p->cfg;
    if (first != st->mtp_length || first + count > c.max_context)
      throw Error(QLLM_INVALID_ARGUMENT, "synthetic cache fill must extend the cached prefix");
    for (uint32_t l = 0; l <= c.layers; ++l)
      ok(launch_fill_synthetic_kv(st->page_table, p->layer_off[l], l < c.layers ? c.kv_encoding : c.mtp_kv_encoding,
                                  c.page_tokens, c.kv_heads, c.head_dim, first, count,
                                  seed + 0x9e3779b97f4a7c15ULL * (l + 1U), p->stream));
    cu(cudaStreamSynchronize(p->stream), "synthetic cache fill");
    st->mtp_length = first + count;
  });
}

}  // extern "C"
