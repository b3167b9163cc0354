/*
 * CPU oracle for the MTP-4 speculative decode step -- TEST INFRASTRUCTURE ONLY.
 *
 * This is a scalar restatement, on the host, of the arithmetic and control
 * flow of quantum-llm's exact-decode path.  It exists so that the CUDA path
 * can be checked against it; nothing in the shipped library links, loads or
 * calls it.  Only tests, the smoke check and the CPU-baseline leg of the
 * benchmark may use it.
 *
 * Reference files restated (paths inside the quantum-llm project):
 *   runtime/src/speculative_sampling.cpp              sampler, counter RNG
 *   runtime/src/cuda/transformer_kernels.cu:1917-2002 NVFP4 fake-quant + GEMV
 *   runtime/src/cuda/transformer_kernels.cu:229-288   Q4H record store
 *   runtime/src/cuda/transformer_kernels.cu:601-625   Q8 record store
 *   runtime/src/cuda/transformer_kernels.cu:4391-4976 Q8 query + Q4H attention
 *   runtime/src/cuda/transformer_kernels.cu:4985-5340 Q8-KV attention (BF16 MMA)
 *   runtime/src/cuda/transformer_kernels.cu:6610-6665 exact-F16 softmax
 *   runtime/src/cuda/transformer_kernels.cu:5741-5798 split combine
 *   runtime/src/cuda/transformer_kernels.cu:7059-7178 argmax / top-k tie rules
 *   runtime/tools/dense_fp4_provider.cpp:8529-8852    run_target / run_mtp / rollout
 *   runtime/tools/dense_fp4_provider.cpp:11011-11318  sync batch / execute_exact_decode
 *
 * Parity pin status: the sampler (incl. the whole-row sampler of the scalar
 * fallback), the counter RNG and the E2M1/E4M3 decoders are pinned on the CPU
 * against the reference's own code and vectors; the NVFP4 GEMV and activation
 * quantiser, the Q4H and Q8 record bytes, Q4H and Q8 attention, argmax and
 * top-k are pinned on the GPU against the reference's own CUDA kernels
 * compiled unmodified for sm_100a (oracle/_ref, tests/test_reference_kernels.py).
 * The control flow of the whole step (accepted-token sequences) is "parity
 * unpinned": the reference holds no end-to-end vector for its MTP loop; it is
 * protected by invariants instead (speculative run == plain run, with and
 * without a presence penalty; rollback leaves the state identical).
 */
#ifndef QLLM_ORACLE_H_
#define QLLM_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { QO_KV_F16 = 0, QO_KV_Q4H = 1, QO_KV_Q8 = 2 };

typedef struct qo_matrix {
  const uint8_t* codes;   /* [rows, cols/2], low nibble = even column */
  const uint8_t* scales;  /* [rows, cols/16] E4M3FN */
  float weight_scale;     /* multiplier applied at run time (1 / stored divisor) */
  float input_scale;      /* activation global scale (multiplier before E4M3) */
  uint32_t rows;
  uint32_t cols;
} qo_matrix;

typedef struct qo_block {
  const float* input_norm;  /* [hidden] */
  qo_matrix qkv;            /* [(q+2kv)*head_dim, hidden]: q rows, k rows, v rows */
  qo_matrix o;              /* [hidden, q*head_dim] */
  const float* post_norm;   /* [hidden] */
  qo_matrix gate_up;        /* [2*ffn, hidden]: gate rows then up rows */
  qo_matrix down;           /* [hidden, ffn] */
  /* routed mixture of experts instead of the dense FFN when cfg.experts != 0
   * (runtime/tools/dense_fp4_provider.cpp:8128-8248, runtime/src/cuda/moe_kernels.cu:121-264) */
  qo_matrix router;               /* [experts, hidden] */
  const qo_matrix* expert_gate;   /* [experts], each [expert_ffn, hidden] */
  const qo_matrix* expert_up;     /* [experts], each [expert_ffn, hidden] */
  const qo_matrix* expert_down;   /* [experts], each [hidden, expert_ffn] */
} qo_block;

typedef struct qo_config {
  uint32_t layers, hidden, q_heads, kv_heads, head_dim, ffn, vocab, draft_vocab;
  uint32_t rotary_dim;
  float rope_theta;
  float eps;
  uint32_t page_tokens;
  uint32_t kv_encoding;      /* target KV: QO_KV_* */
  uint32_t mtp_kv_encoding;  /* draft KV */
  uint32_t activation_bf16;  /* round at the reference's BF16 points */
  uint32_t draft_depth;      /* D (<= 4) */
  uint32_t max_context;
  uint32_t split_tokens;     /* attention split length (multiple of 32) */
  uint32_t experts;          /* 0 = dense FFN */
  uint32_t route_width;      /* experts selected per token (<= 8) */
  uint32_t expert_ffn;       /* intermediate width of one expert */
  float route_scale;         /* routed scaling factor applied to the normalised scores */
} qo_config;

typedef struct qo_weights {
  const uint16_t* embedding;  /* [vocab, hidden] bf16 bits */
  const qo_block* layers;     /* [layers] */
  const float* final_norm;
  qo_matrix head;             /* [vocab, hidden] */
  const float* mtp_embedding_norm;
  const float* mtp_hidden_norm;
  qo_matrix mtp_fusion;       /* [hidden, 2*hidden] */
  qo_block mtp_block;
  const float* mtp_draft_norm;
} qo_weights;

typedef struct qo_request {
  uint64_t seed;
  uint32_t temperature_ppm; /* 0 = greedy */
  uint32_t top_p_ppm;
  uint32_t top_k;           /* 1..64 when temperature_ppm != 0 */
  uint32_t min_p_ppm;
  uint32_t context_limit;   /* reserved_context_tokens */
  uint32_t presence_penalty_biased_ppm; /* penalty * 1e6 + 2000000; 2000000 = none; at most 4000000 */
  uint32_t first_output_position;       /* the scalar head penalises and marks from this position on */
  uint32_t reserved;                    /* 0 */
} qo_request;

typedef struct qo_step_result {
  uint32_t emitted[8];
  uint32_t emitted_count;
  uint32_t next_token;
  uint32_t positions_advanced;
  uint32_t rejected; /* 1 when next_token came from the residual distribution */
} qo_step_result;

typedef struct qo_session qo_session;

/* ---- number formats ------------------------------------------------ */
float qo_e2m1_decode(uint8_t code);
uint8_t qo_e2m1_encode(float value);
float qo_e4m3_decode(uint8_t code);
uint8_t qo_e4m3_encode(float value);
float qo_bf16_round(float value);
uint16_t qo_f16_bits(float value);
float qo_f16_value(uint16_t bits);

/* ---- NVFP4 ----------------------------------------------------------- */
void qo_nvfp4_quantize_weights(const float* w, uint32_t rows, uint32_t cols,
                               float global_scale, uint8_t* codes,
                               uint8_t* scales);
void qo_nvfp4_dequant(const qo_matrix* m, float* out);
void qo_nvfp4_fake_quant(const float* x, uint32_t rows, uint32_t cols,
                         float global_scale, float* out);
/* codes: one E2M1 code per byte [rows, cols]; scales: E4M3 [rows, cols/16] */
void qo_nvfp4_quantize_activations(const float* x, uint32_t rows, uint32_t cols,
                                   float global_scale, uint8_t* codes, uint8_t* scales);
void qo_nvfp4_gemv(const qo_matrix* m, uint32_t first_row, uint32_t row_count,
                   const float* x, uint32_t batch, float* y);

/* ---- layer pieces ---------------------------------------------------- */
void qo_rmsnorm(const float* x, const float* w, float* out, uint32_t rows,
                uint32_t cols, float eps);
void qo_rope(float* heads, uint32_t rows, uint32_t head_count,
             uint32_t head_dim, uint32_t rotary_dim, float theta,
             const uint32_t* positions, int act_bf16);
size_t qo_kv_layer_bytes(uint32_t encoding, uint32_t page_tokens,
                         uint32_t kv_heads, uint32_t head_dim);
void qo_kv_store(uint32_t encoding, uint8_t* const* pages, size_t layer_offset,
                 uint32_t page_tokens, uint32_t kv_heads, uint32_t head_dim,
                 const float* key, const float* value, uint32_t rows,
                 uint32_t row_stride, uint32_t first_cache_position);
void qo_attention(uint32_t encoding, const uint8_t* const* pages,
                  size_t layer_offset, uint32_t page_tokens, const float* query,
                  uint32_t query_row_stride, uint32_t rows,
                  uint32_t first_context_tokens, uint32_t q_heads,
                  uint32_t kv_heads, uint32_t head_dim, uint32_t split_tokens,
                  int act_bf16, float* out);
uint32_t qo_argmax(const float* values, uint32_t count);
/* router of the routed-expert FFN: top_k (<= 8) experts and their BF16-rounded weights */
void qo_moe_route(const float* logits, uint32_t experts, uint32_t top_k, float route_scale,
                  uint32_t* indices, float* scores);
/* thread count of the OpenMP loops (timed CPU baseline) */
void qo_set_threads(uint32_t threads);
uint32_t qo_max_threads(void);
void qo_topk(const float* values, uint32_t count, uint32_t k, float* out_values,
             uint32_t* out_tokens);

/* ---- sampler ---------------------------------------------------------- */
double qo_counter_uniform(uint64_t seed, uint32_t position, uint32_t stream,
                          uint32_t index);
/* returns the number of retained entries, or -1 on invalid input */
int qo_make_distribution(const float* sorted_logits,
                         const uint32_t* sorted_tokens, uint32_t count,
                         uint32_t temperature_ppm, uint32_t top_p_ppm,
                         uint32_t min_p_ppm, uint32_t* out_tokens,
                         double* out_probabilities);
uint32_t qo_sample_distribution(const uint32_t* tokens,
                                const double* probabilities, uint32_t count,
                                double uniform);
/* sample_token (dense_fp4_provider.cpp:771-802): full-vocabulary ordering, the first top_k kept
 * (0 = all), distribution and sample at counter_uniform(seed, position, 0).  0, or -1 on the
 * inputs the reference throws on. */
int qo_sample_token(const float* logits, uint32_t vocabulary, const qo_request* request,
                    uint32_t position, uint32_t* token);
/* returns 1 accepted, 0 rejected (token = residual sample), -1 error */
int qo_rejection_sample(uint32_t proposal, const uint32_t* target_tokens,
                        const double* target_probabilities,
                        uint32_t target_count, const uint32_t* draft_tokens,
                        const double* draft_probabilities, uint32_t draft_count,
                        double acceptance_uniform, double correction_uniform,
                        uint32_t* token);

/* ---- whole step -------------------------------------------------------- */
qo_session* qo_session_create(const qo_config* config,
                              const qo_weights* weights);
void qo_session_destroy(qo_session* session);
/* Prefill the prompt through the target in chunks of chunk_rows, prime the
 * draft cache through synchronisation batches, pick the first token and roll
 * out the first drafts.  Returns 0 on success. */
int qo_prefill(qo_session* session, const uint32_t* tokens, uint32_t count,
               uint32_t chunk_rows, const qo_request* request,
               uint32_t* first_token);
/* The same for prompt positions [base, base + count) behind a cached prefix of `base` positions. */
int qo_prefill_at(qo_session* session, const uint32_t* tokens, uint32_t count, uint32_t base,
                  uint32_t chunk_rows, const qo_request* request, uint32_t* first_token);
/* Seeded synthetic cache records for positions [first, first + count) of every layer -- the host
 * twin of the CUDA library's synthetic cache fill (same bytes); extends the cached prefix. */
int qo_fill_synthetic_kv(qo_session* session, uint32_t first, uint32_t count, uint64_t seed);
int qo_execute_exact_decode(qo_session* session, const qo_request* request,
                            uint32_t guaranteed_token, uint32_t position,
                            qo_step_result* result);
/* inspection for parity tests */
uint32_t qo_draft_count(const qo_session* session);
void qo_drafts(const qo_session* session, uint32_t* tokens);
const float* qo_last_logits(const qo_session* session); /* [rows, vocab] */
const float* qo_last_hidden(const qo_session* session); /* [rows, hidden] */
size_t qo_page_bytes(const qo_session* session);
uint32_t qo_page_count(const qo_session* session);
const uint8_t* qo_page(const qo_session* session, uint32_t index);
size_t qo_layer_offset(const qo_session* session, uint32_t layer); /* layer == layers -> draft layer */
uint32_t qo_mtp_length(const qo_session* session);
const char* qo_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* QLLM_ORACLE_H_ */
