/*
 * qllm_b200 -- C ABI of the B200 (sm_100a) provider for quantum-llm's MTP-4
 * speculative decode step.
 *
 * Two layers are exported:
 *   1. kernel launchers (qllm_k_*): one call per reference launcher in
 *      runtime/include/expert/runtime/cuda/transformer_kernels.hpp; raw device
 *      pointers, a CUDA stream as void*, int status (0 = ok).
 *   2. the provider (qllm_provider_*): the exact-decode subset of
 *      expert::runtime::IOperationProvider
 *      (runtime/include/expert/runtime/program_executor.hpp:244-370) flattened
 *      to C: prepare_exact_decode, create_request_state,
 *      synchronize_exact_decode_batch, execute_exact_decode.
 *
 * Every function returns 0 on success and a negative qllm_status otherwise;
 * qllm_last_error() gives the message of the calling thread's last failure.
 * No function falls back to a CPU path.
 */
#ifndef QLLM_B200_H_
#define QLLM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Mirrors expert::runtime::ErrorCode (runtime/include/expert/runtime/storage.hpp:17-29). */
typedef enum qllm_status {
  QLLM_OK = 0,
  QLLM_CANCELLED = -1,
  QLLM_DEADLINE_EXCEEDED = -2,
  QLLM_BACKPRESSURE = -3,
  QLLM_INVALID_ARGUMENT = -4,
  QLLM_UPLOAD_FAILED = -9,
  QLLM_INTERNAL = -10
} qllm_status;

/* PagedKvEncoding subset (runtime/src/cuda/transformer_kernels.cu:50-59). */
enum { QLLM_KV_F16 = 0, QLLM_KV_Q4H = 1, QLLM_KV_Q8 = 2 };

/* Nvfp4Block16Matrix (runtime/include/expert/runtime/cuda/transformer_kernels.hpp:47-54):
 * codes [rows, cols/2] (low nibble = even column), scales [rows, cols/16] E4M3FN. */
typedef struct qllm_matrix {
  const uint8_t* codes;
  const uint8_t* scales;
  float weight_scale; /* multiplier: 1 / stored weight divisor */
  float input_scale;  /* activation global scale */
  uint32_t rows;
  uint32_t cols;
} qllm_matrix;

typedef struct qllm_block {
  const float* input_norm;
  qllm_matrix qkv;     /* [(q+2kv)*head_dim, hidden] */
  qllm_matrix o;       /* [hidden, q*head_dim] */
  const float* post_norm;
  qllm_matrix gate_up; /* [2*ffn, hidden] gate rows then up rows */
  qllm_matrix down;    /* [hidden, ffn] */
  /* Routed mixture of experts in place of the dense FFN when config.experts != 0
   * (NVFP4 branch of run_router / run_routed_moe, dense_fp4_provider.cpp:8128-8166, 8207-8248;
   * expert arithmetic runtime/src/cuda/moe_kernels.cu:171-264, 430-510, 633-690, 759-790).
   * The arrays are host arrays of `experts` descriptors. */
  qllm_matrix router;              /* [experts, hidden] */
  const qllm_matrix* expert_gate;  /* each [expert_ffn, hidden] */
  const qllm_matrix* expert_up;    /* each [expert_ffn, hidden] */
  const qllm_matrix* expert_down;  /* each [hidden, expert_ffn] */
} qllm_block;

/* Geometry the artifact declares (runtime/tools/dense_fp4_provider.cpp:804-960). */
typedef struct qllm_config {
  uint32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, draft_vocab;
  uint32_t rotary_dim;
  float rope_theta;
  float eps;
  uint32_t page_tokens;
  uint32_t kv_encoding;
  uint32_t mtp_kv_encoding;
  uint32_t activation_bf16;
  uint32_t draft_depth;
  uint32_t max_context;
  uint32_t split_tokens;
  uint32_t experts;     /* 0 = dense FFN */
  uint32_t route_width; /* experts selected per token (<= 8) */
  uint32_t expert_ffn;  /* intermediate width of one expert */
  float route_scale;    /* routed scaling factor (route_scale_f32_bits) */
} qllm_config;

/* Tensor roles of the exact-decode program (dense_fp4_provider.cpp:4733-4786). */
typedef struct qllm_weights {
  const uint16_t* embedding; /* [vocab, hidden] bf16 */
  const qllm_block* layers;  /* host array [layers] of device (or host) pointers */
  const float* final_norm;
  qllm_matrix head;
  const float* mtp_embedding_norm;
  const float* mtp_hidden_norm;
  qllm_matrix mtp_fusion;
  qllm_block mtp_block;
  const float* mtp_draft_norm;
} qllm_weights;

/* ProgramRequestContext.parameters read on this path (runtime/tools/moe_vm_runner.cpp:318-347). */
typedef struct qllm_request {
  uint64_t sampling_seed;
  uint32_t sampling_temperature_ppm; /* 0 = greedy */
  uint32_t sampling_top_p_ppm;
  uint32_t sampling_top_k; /* 1..64 when sampling */
  uint32_t sampling_min_p_ppm;
  uint32_t reserved_context_tokens; /* context limit of the request */
  /* sampling_presence_penalty_biased_ppm: penalty * 1e6 + 2 000 000, i.e. 2 000 000 = no penalty,
   * at most 4 000 000 (apply_presence_penalty, runtime/tools/dense_fp4_provider.cpp:8336-8347):
   * logits[token] -= penalty for every token the request has emitted, and inside a speculative step
   * also for the proposals that precede the row being judged (:11182-11202); accepted proposals and
   * the selected token are committed to the request's mask by the step (:11261-11270). */
  uint32_t sampling_presence_penalty_biased_ppm;
  /* sampling_first_output_position (moe_vm_runner.cpp:341): the scalar head (first token, scalar
   * decode) penalises and marks only sample positions at or after it. */
  uint32_t sampling_first_output_position;
  uint32_t reserved; /* 0 */
} qllm_request;

/* ExactDecodeExecutionResult (program_executor.hpp:205-212). */
typedef struct qllm_exact_result {
  uint32_t emitted_tokens[8];
  uint32_t emitted_count;
  uint32_t next_token;
  uint32_t positions_advanced;
  uint32_t rejected;
} qllm_exact_result;

typedef struct qllm_provider qllm_provider;
typedef struct qllm_request_state qllm_request_state;

const char* qllm_last_error(void);
/* Capability string and ABI the provider advertises to the registry
 * (KernelCapability, runtime/include/expert/runtime/model_descriptor.hpp:65-80). */
const char* qllm_capability_name(void);
uint32_t qllm_capability_abi(void);

/* ------------------------------------------------------------ provider */
/* weights_on_device != 0: every pointer in `weights` is device memory that
 * outlives the provider (borrowed); otherwise host memory, uploaded once
 * (ensure_tensor, dense_fp4_provider.cpp:3486-3677).
 * Replaces make_dense_fp4_callable_provider + prepare_exact_decode
 * (dense_fp4_provider.cpp:11398-11499, 2865-2984). */
int qllm_provider_create(const qllm_config* config, const qllm_weights* weights,
                         int weights_on_device, int device, qllm_provider** out);
void qllm_provider_destroy(qllm_provider* provider);
/* IOperationProvider::create_request_state (program_executor.hpp:249). */
int qllm_provider_create_request_state(qllm_provider* provider, qllm_request_state** out);
void qllm_provider_destroy_request_state(qllm_provider* provider, qllm_request_state* state);
/* One prefill chunk of the target program (execute_program_sequence,
 * dense_fp4_provider.cpp:8854-9200 as driven by moe_vm_runner.cpp:679-778): stores
 * target KV for positions first_position.. and retains the hidden rows for the
 * following synchronisation batch. tokens: host. count <= qllm_provider_max_chunk_rows;
 * the results do not depend on how a prompt is cut into chunks. The chunk is enqueued on the
 * provider's stream and the call returns (tokens are staged before it does), so that the host
 * prepares the next chunk while this one runs; qllm_provider_first_token and the producing
 * synchronisation batch wait for the stream and report any device-side error. */
int qllm_provider_prefill_chunk(qllm_provider* provider, qllm_request_state* state,
                                const uint32_t* tokens, uint32_t count, uint32_t first_position);
/* Token selected by the head for the last retained row (run_head sampling
 * branch, dense_fp4_provider.cpp:8436-8517). */
int qllm_provider_first_token(qllm_provider* provider, qllm_request_state* state,
                              const qllm_request* request, uint32_t sample_position,
                              uint32_t* token);
/* One non-speculative decode step: the runner's fallback when a request is not eligible for
 * exact decode (session.execute({token, position}) followed by synchronize_exact_decode,
 * moe_vm_runner.cpp:349-360 and :1151-1157; head sampling dense_fp4_provider.cpp:8433-8517,
 * sample_token :771-802).  Runs `token` at `position` (the end of the cached stream) through the
 * target model, selects the next token with the request's sampler at sample position
 * `position` (dense_fp4_provider.cpp:10962-10964) -- greedy, sorted top-k (1..64), or the whole vocabulary ordered on the device
 * when sampling_top_k is 0 or above 64 -- and advances the draft cache by a one-row
 * synchronisation batch; produce_final_draft != 0 also primes the drafts (the request must then
 * be one the speculative path accepts). */
int qllm_provider_scalar_decode(qllm_provider* provider, qllm_request_state* state,
                                const qllm_request* request, uint32_t token, uint32_t position,
                                int produce_final_draft, uint32_t* next_token);
/* IOperationProvider::checkpoint_request_state / rewind_request_state (program_executor.hpp,
 * dense_fp4_provider.cpp:9209-9269 and :9271-9338) for a full-attention model.  A checkpoint
 * can be taken at next_position == the length of the cached stream with no chunk waiting for
 * its synchronisation batch; a rewind returns to exactly that position, drops the drafts and
 * expects the stream to continue with a chunk or a scalar decode step at next_position.  The
 * cache is rolled back by overwriting; the recurrent, PLE and sliding-window state the reference
 * also copies belongs to model families this provider does not run. */
int qllm_provider_checkpoint_request_state(qllm_provider* provider, qllm_request_state* state,
                                           uint32_t next_position);
int qllm_provider_rewind_request_state(qllm_provider* provider, qllm_request_state* state,
                                       uint32_t next_position);
/* IOperationProvider::synchronize_exact_decode_batch (program_executor.hpp:344;
 * dense_fp4_provider.cpp:11011-11137). next_tokens: host. */
int qllm_provider_synchronize_exact_decode_batch(qllm_provider* provider,
                                                 qllm_request_state* state,
                                                 const qllm_request* request,
                                                 const uint32_t* next_tokens, uint32_t count,
                                                 uint32_t first_target_position,
                                                 int produce_final_draft);
/* IOperationProvider::execute_exact_decode (program_executor.hpp:364;
 * dense_fp4_provider.cpp:11139-11318). Completes synchronously. */
int qllm_provider_execute_exact_decode(qllm_provider* provider, qllm_request_state* state,
                                       const qllm_request* request, uint32_t guaranteed_token,
                                       uint32_t position, uint32_t context_limit,
                                       qllm_exact_result* result);
/* Enqueue-only form for pipelined callers: `steps` consecutive steps whose
 * guaranteed token/position come from the device-resident state; results are
 * written to host memory after one synchronisation. */
int qllm_provider_execute_exact_decode_steps(qllm_provider* provider, qllm_request_state* state,
                                             const qllm_request* request, uint32_t context_limit,
                                             uint32_t steps, qllm_exact_result* results);
/* Counters of ExecutionProviderModule::telemetry (dense_fp4_provider.cpp:3109-, 11313-11316):
 * out[0]=exact_calls, out[1]=accepted_drafts, out[2..6]=accepted_depth_calls[0..4],
 * out[7]=kernel launches enqueued since creation. */
int qllm_provider_telemetry(qllm_provider* provider, qllm_request_state* state, uint64_t* out,
                            uint32_t count);
/* The cudaStream_t every call of this provider launches on (for event timing). */
void* qllm_provider_stream(qllm_provider* provider);
/* Most rows qllm_provider_prefill_chunk / _synchronize_exact_decode_batch take at once. The
 * reference's microbatch paths stop at kMaximumWorkspaceRows = 8 (dense_fp4_provider.cpp:8854-9200)
 * and its wider prompt batches go through fp4_gemm_block32_kernel; here a chunk of up to 128 rows
 * is one operand of the block-scaled tensor-core kernel (one pass over the weights per chunk),
 * attention takes it in tiles of 8 rows and only its last row reaches the head. A tensor-parallel
 * provider stays at 8 (the size of its exchange slots). */
uint32_t qllm_provider_max_chunk_rows(const qllm_provider* provider);
/* 0 = launch kernels one by one, 1 = replay the captured CUDA graph of the step. */
int qllm_provider_set_graph_mode(qllm_provider* provider, int enabled);
/* GEMV implementation: 0 = CUDA-core kernel, 1 = tcgen05 block-scaled MMA kernel. */
int qllm_provider_set_gemv_impl(qllm_provider* provider, int impl);
/* Attention implementation: 0 = the order-independent scalar kernel everywhere (the parity anchor);
 * 1 (default) = tensor-core kernels through mma.sync where the geometry allows (Q4H, Q8 and F16 caches,
 * head_dim 128); 2 = as 1, with the Q4H target cache on the tcgen05 kernel (INT8 MMAs with tensor-memory
 * accumulators; decode steps with at most 32 matrix rows per kv head, 128-token aligned splits). */
int qllm_provider_set_attention_impl(qllm_provider* provider, int impl);

/* Tensor-parallel verify (no reference counterpart: the reference runs one GPU per model; the
 * sharding follows its projection layout, runtime/tools/dense_fp4_provider.cpp:6189-6278).
 * One process per GPU, each with a provider over ITS shard: config.q_heads / kv_heads / ffn are
 * the local counts (global / ranks), qkv holds the rank's q, k and v head rows, gate_up its gate
 * and up rows, o and down its K columns (a slice of the same quantised tensor: one weight_scale
 * for all ranks); embedding, norms, heads and the fusion projection are replicated.  The o and
 * down projections then exchange FP32 partial sums through peer memory inside the GEMV kernel,
 * and every rank computes identical rows, tokens and acceptance decisions.
 *   1. every rank: qllm_provider_tp_export(provider, rank, ranks, handle)  -- allocates the
 *      rank's exchange area and returns its inter-process handle (QLLM_TP_HANDLE_BYTES bytes);
 *   2. the host exchanges the handles (all-gather in rank order);
 *   3. every rank: qllm_provider_tp_attach(provider, all_handles)  -- maps the peers' areas.
 * Needs the tensor-core GEMV (qllm_provider_set_gemv_impl(1)), K of the local o and down
 * projections a multiple of 64, and peer access between the GPUs.  ranks == 1 runs the same
 * code path without peers.  A value that has not arrived after about a second of polling sets the kernel
 * error word (the step fails with QLLM_INTERNAL); nothing waits without a limit. */
#define QLLM_TP_HANDLE_BYTES 64
int qllm_provider_tp_export(qllm_provider* provider, uint32_t rank, uint32_t ranks, void* handle);
int qllm_provider_tp_attach(qllm_provider* provider, const void* handles);
/* Size in bytes of this rank's exchange area (0 before qllm_provider_tp_export). */
size_t qllm_provider_tp_area_bytes(const qllm_provider* provider);
/* Step 3 for a host that drives all GPUs from ONE process (peer access enabled): `areas[r]` is rank
 * r's exchange area as a device pointer of at least qllm_provider_tp_area_bytes() bytes, zeroed
 * before the first step (the own rank's entry is ignored).  The areas stay owned by the caller. */
int qllm_provider_tp_attach_local(qllm_provider* provider, void* const* areas);

/* ---- runtime-model.tsv: the artifact's model descriptor -------------------------------------
 * Host-only.  qllm_descriptor_parse reads the descriptor text with the grammar and the validity
 * rules of the reference's parser (parse_model_descriptor_artifact and validate_model_descriptor,
 * runtime/src/model_descriptor.cpp:492-746, :107-341; namespace base 1): header line, tab-separated
 * records, duplicate keys and unknown records rejected, kernel requirements, contiguous layer and
 * operation programs, routed components, schema-3 data flow.  Rejections return
 * QLLM_INVALID_ARGUMENT with the reference's message in qllm_last_error() ("malformed model
 * descriptor line N", ...).
 * qllm_descriptor_negotiate is the provider side of capability selection
 * (runtime/tools/dense_fp4_provider.cpp:2367-2470, :2935-2966; registry rule
 * runtime/src/execution_provider.cpp:54-97): the artifact must list this library's capability
 * (qllm_capability_name / _abi) as a required kernel and as its exact_decode program, with
 * source_mtp_layers = 1, draft_depth = maximum emitted tokens - 1 (at most 4),
 * draft_vocabulary_size <= vocabulary, mtp_kv_encoding = 1, embedding_first = 1, post_norm = 1;
 * it then fills the geometry of `config` from the model record, the attributes
 * (attention_heads, kv_heads, head_dim, rotary_dimension, norm_epsilon_f32_bits,
 * rope_theta_f32_bits, activation_bf16, optional intermediate_size), the layer count and the first
 * routed component; kv_encoding, page_tokens, split_tokens and max_context stay the caller's
 * (max_context is clamped to the model's).
 * qllm_descriptor_tensor returns the tensor bound to a role of the exact-decode program
 * ("token_embedding", "fusion_projection", "layer.0.query_projection", ...; roles as in
 * dense_fp4_provider.cpp:4733-4786), else of the model, else NULL.
 * qllm_descriptor_dump writes what was understood in a canonical text form (tests compare it
 * with the same dump of the reference's own parser); returns the full length. */
typedef struct qllm_descriptor qllm_descriptor;
int qllm_descriptor_parse(const char* text, size_t bytes, qllm_descriptor** descriptor);
void qllm_descriptor_destroy(qllm_descriptor* descriptor);
int qllm_descriptor_negotiate(const qllm_descriptor* descriptor, qllm_config* config);
const char* qllm_descriptor_tensor(const qllm_descriptor* descriptor, const char* role);
size_t qllm_descriptor_dump(const qllm_descriptor* descriptor, char* out, size_t capacity);

/* ---- dense QPack records: the on-disk form of the weights ---------------------------------------
 * Host-only.  One dense tensor of the artifact manifest's index (the fields the reference's
 * runtime takes from it, runtime/src/model_tensor_store.cpp:146-166) and the checks the reference's
 * validator applies to its record (compiler/expert_pack/validate.py:131-318; record layout
 * docs/expert-pack-v1.md:20-40, header compiler/expert_pack/constants.py:72-97): 4 KiB record
 * alignment, 256-byte little-endian header with zero padding, magic and version, row-major flag,
 * rank and shape, SHA-256 of the tensor name, data and scale sections equal to the index's, and per
 * encoding: raw F32 / BF16 / I64 (ABI 0: no scale section, byte count = elements x width) or native
 * NVFP4 (ABI 5: symmetric flag, matrix, columns % 16 == 0, rows x columns / 2 code bytes, scale
 * section 256-byte aligned holding rows x columns / 16 finite E4M3FN bytes, the FP32 weight divisor
 * and the FP32 or BF16 activation divisor, both finite and positive); with verify_payload the
 * SHA-256 of everything after the header against the header's and the index's digests.  Other
 * encodings (INT8, FP4 block-32, MXFP6) are rejected: this provider does not read them.
 * qllm_pack_nvfp4_matrix additionally returns the matrix as the provider takes it: host pointers
 * into the pack, weight_scale = 1 / weight divisor, input_scale = activation divisor
 * (runtime/tools/dense_fp4_provider.cpp:3534-3568). */
enum { QLLM_PACK_F32 = 0, QLLM_PACK_BF16 = 1, QLLM_PACK_I64 = 2, QLLM_PACK_FP4_E2M1 = 3 };
typedef struct qllm_pack_entry {
  const char* name;                 /* tensor name (its SHA-256 is in the record header) */
  uint64_t offset, stored_bytes;    /* record position and size inside the pack */
  uint32_t rank, shape[5];          /* logical shape ("source_shape") */
  uint64_t data_offset, data_bytes; /* sections, relative to the record start */
  uint64_t scale_offset, scale_bytes;
  uint32_t stored_dtype;            /* QLLM_PACK_* ("stored_dtype") */
  uint8_t payload_sha256[32];
} qllm_pack_entry;
int qllm_pack_check_dense(const void* pack, size_t pack_bytes, const qllm_pack_entry* entry, int verify_payload);
int qllm_pack_nvfp4_matrix(const void* pack, size_t pack_bytes, const qllm_pack_entry* entry, int verify_payload,
                           qllm_matrix* matrix);
/* One routed expert of the manifest's expert index and its record (magic EPEXPR01; header
 * compiler/expert_pack/constants.py:88-92, writer compiler/expert_pack/writer.py:417-552, checks
 * compiler/expert_pack/validate.py:328-482), native NVFP4 (ABI 5) only: flags row-major | symmetric |
 * gate-up-fused, layer / expert identity, four 256-byte aligned, ordered, non-overlapping
 * sections equal to the index's — gate+up codes (gate then up, intermediate x hidden / 2 bytes
 * each), gate+up sidecars, down codes, down sidecars — where a matrix's sidecar is its E4M3FN
 * block scales followed by the FP32 weight divisor and the FP32 activation divisor (finite,
 * positive), decoded size 3 x hidden x intermediate x 4, and optionally the payload SHA-256.
 * qllm_pack_nvfp4_expert returns the three projections as the provider takes them
 * (qllm_block.expert_gate / expert_up / expert_down entries): gate and up [intermediate, hidden],
 * down [hidden, intermediate], pointers into the pack. */
typedef struct qllm_pack_expert_entry {
  int32_t layer, expert;
  uint64_t offset, stored_bytes;
  uint64_t section_offset[4], section_bytes[4]; /* gate_up_q, gate_up_scales, down_q, down_scales */
  uint64_t decoded_bytes;
  uint8_t payload_sha256[32];
} qllm_pack_expert_entry;
int qllm_pack_check_expert(const void* pack, size_t pack_bytes, const qllm_pack_expert_entry* entry,
                           int verify_payload);
int qllm_pack_nvfp4_expert(const void* pack, size_t pack_bytes, const qllm_pack_expert_entry* entry,
                           int verify_payload, qllm_matrix* gate, qllm_matrix* up, qllm_matrix* down);
void qllm_sha256(const void* bytes, size_t count, uint8_t digest[32]);

/* inspection for parity tests (device -> host copies) */
int qllm_provider_read_logits(qllm_provider* provider, float* out, uint32_t rows);
/* which = 0: rows retained by the last prefill chunk; 1: target rows of the last exact step. */
int qllm_provider_read_hidden(qllm_provider* provider, qllm_request_state* state, int which,
                              float* out, uint32_t rows);
int qllm_provider_read_drafts(qllm_provider* provider, qllm_request_state* state,
                              uint32_t* tokens, uint32_t* count);
size_t qllm_provider_page_bytes(qllm_provider* provider);
size_t qllm_provider_layer_offset(qllm_provider* provider, uint32_t layer);
int qllm_provider_read_page(qllm_provider* provider, qllm_request_state* state, uint32_t page,
                            uint8_t* out);
/* Test/bench hook without a reference counterpart: fill token positions
 * [first, first+count) of every layer's cache (target and draft) with seeded
 * pseudo-random records and advance the cached prefix; stands in for a long prompt. */
int qllm_provider_fill_synthetic_kv(qllm_provider* provider, qllm_request_state* state,
                                    uint32_t first, uint32_t count, uint64_t seed);

/* Measurement aid without a reference counterpart: runs the verify pass alone (target forward over
 * the pending guaranteed token and drafts, head, candidate selection) `repeats` times back to back
 * and returns its mean duration in milliseconds, measured with CUDA events on the provider's
 * stream.  It recomputes what the next step computes anyway, so decoding can continue afterwards.
 * Needs pending drafts (after a prefill or a step). */
int qllm_provider_time_verify(qllm_provider* provider, qllm_request_state* state,
                              const qllm_request* request, uint32_t repeats, float* mean_ms);

/* ------------------------------------------------------- kernel layer */
/* All pointers are device memory unless stated; stream is a cudaStream_t. */

/* embedding_bf16_batch (transformer_kernels.cu:1901-1915) */
int qllm_k_embedding_bf16(const uint16_t* table, const uint32_t* tokens, float* out,
                          uint32_t rows, uint32_t hidden, uint32_t vocab, void* stream);
/* rms_norm_batch (transformer_kernels.cu:2487-2503) */
int qllm_k_rms_norm(const float* x, const float* weight, float* out, uint32_t rows,
                    uint32_t cols, float eps, void* stream);
/* nvfp4_quant_dequant_kernel (transformer_kernels.cu:1943-1968) */
int qllm_k_nvfp4_fake_quant(const float* x, float* out, uint32_t rows, uint32_t cols,
                            float global_scale, void* stream);
/* nvfp4_gemv_f32_batch (transformer_kernels.cu:7970-8001): y[batch, row_count] =
 * bf16(fakequant(x) . W[first_row..]^T).  workspace: device scratch of at least
 * qllm_k_nvfp4_gemv_workspace_bytes(batch, row_count, cols) bytes. impl as in
 * qllm_provider_set_gemv_impl. */
size_t qllm_k_nvfp4_gemv_workspace_bytes(uint32_t batch, uint32_t rows, uint32_t cols);
int qllm_k_nvfp4_gemv(const qllm_matrix* matrix, uint32_t first_row, uint32_t row_count,
                      const float* x, float* y, uint32_t batch, void* workspace,
                      size_t workspace_bytes, int impl, void* stream);
/* No counterpart in the reference.  qllm_k_nvfp4_gemv (CUDA-core implementation, impl 0)
 * for callers that cannot hand over a device workspace at call time and must not reach the
 * CUDA allocator: a runtime that gave all device memory to its own pool at start-up, or a
 * thread holding a lock under which cudaMalloc/cudaFree (which synchronise the device) would
 * stall other streams.  The quantised activations live in a fixed array inside the library
 * (qllm_k_nvfp4_gemv_static_scratch_bytes() bytes, 2 MiB: batch * cols * 1.25 must fit,
 * otherwise QLLM_INVALID_ARGUMENT).  The array is shared by all calls on a device: calls on
 * one stream are ordered, calls that overlap in time on different streams or threads race.
 * Nothing in it needs to start at zero.  The first call on a device looks up the array's
 * address; issue it once during start-up, before any stream capture on that device. */
size_t qllm_k_nvfp4_gemv_static_scratch_bytes(void);
int qllm_k_nvfp4_gemv_static(const qllm_matrix* matrix, uint32_t first_row, uint32_t row_count,
                             const float* x, float* y, uint32_t batch, void* stream);
/* Load-time preparation of one matrix (the provider does this once per tensor when it binds
 * the weights, cf. ensure_tensor, dense_fp4_provider.cpp:3486-3677): builds the TMA descriptor
 * and the re-tiled block scales the tensor-core GEMV reads.  The matrix memory must outlive
 * the handle.  qllm_k_nvfp4_gemv_prepared is qllm_k_nvfp4_gemv without that per-call work
 * and without a final synchronisation. */
typedef struct qllm_prepared_matrix qllm_prepared_matrix;
int qllm_k_matrix_prepare(const qllm_matrix* matrix, void* stream, qllm_prepared_matrix** out);
void qllm_k_matrix_release(qllm_prepared_matrix* prepared);
int qllm_k_nvfp4_gemv_prepared(const qllm_prepared_matrix* prepared, const float* x, float* y,
                               uint32_t batch, void* workspace, size_t workspace_bytes, int impl,
                               void* stream);
/* The tensor-core GEMV kernel alone (nvfp4_gemv_batch_reuse_kernel's role,
 * transformer_kernels.cu:1970-2002, without the activation quantiser and the split-K
 * finalisation): re-runs it over the quantised operand that a qllm_k_nvfp4_gemv_prepared
 * call (impl 1) with the same handle, batch and workspace left behind, leaving split-K
 * partial sums in the workspace.  This is how the provider chains it between fused
 * producer/consumer kernels, and what the benchmark times as the dominant kernel. */
int qllm_k_nvfp4_gemv_prepared_core(const qllm_prepared_matrix* prepared, uint32_t batch,
                                    void* workspace, size_t workspace_bytes, void* stream);
/* Harness-owned weight quantiser on the device (formula of transformer_kernels.cu:1960-1967
 * applied to weight rows); w is fp32 [rows, cols]. */
int qllm_k_nvfp4_quantize_weights(const float* w, uint32_t rows, uint32_t cols,
                                  float global_scale, uint8_t* codes, uint8_t* scales,
                                  void* stream);
/* add_kernel / silu_product_kernel (transformer_kernels.cu:2522-2528, 2774-2783) */
int qllm_k_add(float* dst, const float* src, uint64_t count, int bf16, void* stream);
int qllm_k_silu_product(const float* gate_up, float* out, uint32_t rows, uint32_t ffn, int bf16,
                        void* stream);
/* RoPE of q and k heads in place + K/V record store
 * (gated_gqa_qkv_rope_paged_batch_kernel without the per-head norm, 3551-3643;
 * store_paged_kv_record 229-288 / 601-625; store_gqa_kv_fp16_to_paged 4208-4230).
 * qkv: [rows, (q+2kv)*head_dim]; position of row r = *first_position + r;
 * rotary position = that + rotary_offset. inv_freq: [rotary_dim/2]. */
int qllm_k_rope_kv_store(float* qkv, uint32_t rows, uint32_t q_heads, uint32_t kv_heads,
                         uint32_t head_dim, uint32_t rotary_dim, const float* inv_freq,
                         const uint32_t* first_position, uint32_t position_offset,
                         uint32_t rotary_offset, uint8_t* const* page_table, size_t layer_offset,
                         uint32_t page_tokens, uint32_t encoding, int bf16, void* stream);
size_t qllm_k_kv_layer_bytes(uint32_t encoding, uint32_t page_tokens, uint32_t kv_heads,
                             uint32_t head_dim);
/* Split attention + combine (Q4H: 4391-4976, Q8: 4985-5340, F16: 6610-6665; combine
 * 5741-5798).  workspace >= qllm_k_attention_workspace_bytes(...). impl 0 = scalar
 * kernel (all encodings), 1 = tensor-core kernel (Q4H). */
size_t qllm_k_attention_workspace_bytes(uint32_t rows, uint32_t q_heads, uint32_t head_dim,
                                        uint32_t max_splits);
int qllm_k_attention(uint32_t encoding, const uint8_t* const* page_table, size_t layer_offset,
                     uint32_t page_tokens, const float* query, uint32_t query_row_stride,
                     uint32_t rows, const uint32_t* first_position, uint32_t position_offset,
                     uint32_t q_heads, uint32_t kv_heads, uint32_t head_dim,
                     uint32_t split_tokens, uint32_t max_splits, int bf16, void* workspace,
                     float* out, int impl, void* stream);
/* argmax_batch / topk_logits (transformer_kernels.cu:7059-7178) */
int qllm_k_argmax(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride,
                  uint32_t* out, void* stream);
/* router_topk_normalized_logits_batch (transformer_kernels.cu:8652-8672, select kernel 2947-3006)
 * with the BF16 rounding of logits and scores of run_router (dense_fp4_provider.cpp:8153-8164):
 * logits [rows, experts] -> indices / scores [rows, top_k], top_k <= 8, experts <= 256. */
int qllm_k_moe_route(const float* logits, uint32_t rows, uint32_t experts, uint32_t top_k,
                     float route_scale, uint32_t* indices, float* scores, void* stream);
size_t qllm_k_topk_workspace_bytes(uint32_t rows, uint32_t count, uint32_t k);
int qllm_k_topk(const float* values, uint32_t rows, uint32_t count, uint32_t row_stride,
                uint32_t k, float* out_values, uint32_t* out_tokens, void* workspace,
                void* stream);
/* sample_token (dense_fp4_provider.cpp:771-802): every id ordered by (logit descending, NaN last,
 * id ascending), the first top_k kept (0 = all), make_sampling_distribution and
 * sample_distribution (speculative_sampling.cpp:52-128) with counter_uniform(seed, position, 0).
 * logits, workspace (qllm_k_sample_token_workspace_bytes), status and token are device pointers;
 * *status = 5 where the reference throws "no retained mass" / "invalid sorted sampling candidates". */
size_t qllm_k_sample_token_workspace_bytes(uint32_t vocabulary);
int qllm_k_sample_token(const float* logits, uint32_t vocabulary, uint64_t seed, uint32_t temperature_ppm,
                        uint32_t top_p_ppm, uint32_t top_k, uint32_t min_p_ppm, uint32_t position,
                        void* workspace, uint32_t* status, uint32_t* token, void* stream);
/* Device form of rejection_sample / make_sampling_distribution / counter_uniform
 * (runtime/src/speculative_sampling.cpp:52-182) over host-visible arrays, for the
 * parity tests of the acceptance kernel: one decision per call.
 * All pointers here are HOST memory; the call copies, runs the device kernel
 * and copies back. Returns 1 accepted / 0 rejected / negative status. */
int qllm_k_rejection_sample_host(uint32_t proposal, const uint32_t* target_tokens,
                                 const double* target_probabilities, uint32_t target_count,
                                 const uint32_t* draft_tokens, const double* draft_probabilities,
                                 uint32_t draft_count, double acceptance_uniform,
                                 double correction_uniform, uint32_t* token);
int qllm_k_make_distribution_host(const float* sorted_logits, const uint32_t* sorted_tokens,
                                  uint32_t count, uint32_t temperature_ppm, uint32_t top_p_ppm,
                                  uint32_t min_p_ppm, uint32_t* out_tokens,
                                  double* out_probabilities);
int qllm_k_counter_uniform_host(uint64_t seed, uint32_t position, uint32_t stream_id,
                                uint32_t index, double* out);

#ifdef __cplusplus
}
#endif
#endif /* QLLM_B200_H_ */
