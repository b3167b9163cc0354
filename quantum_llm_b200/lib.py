"""ctypes binding of libqllm_b200.so (the C ABI declared in include/qllm_b200.h)."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libqllm_b200.so")

KV_F16, KV_Q4H, KV_Q8 = 0, 1, 2
TP_HANDLE_BYTES = 64   # QLLM_TP_HANDLE_BYTES


class QllmError(RuntimeError):
    def __init__(self, status, message):
        super().__init__(f"qllm status {status}: {message}")
        self.status = status


class Matrix(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("weight_scale", C.c_float),
                ("input_scale", C.c_float), ("rows", C.c_uint32), ("cols", C.c_uint32)]


class PackEntry(C.Structure):
    _fields_ = [("name", C.c_char_p), ("offset", C.c_uint64), ("stored_bytes", C.c_uint64), ("rank", C.c_uint32),
                ("shape", C.c_uint32 * 5), ("data_offset", C.c_uint64), ("data_bytes", C.c_uint64),
                ("scale_offset", C.c_uint64), ("scale_bytes", C.c_uint64), ("stored_dtype", C.c_uint32),
                ("payload_sha256", C.c_uint8 * 32)]


class PackExpertEntry(C.Structure):
    _fields_ = [("layer", C.c_int32), ("expert", C.c_int32), ("offset", C.c_uint64), ("stored_bytes", C.c_uint64),
                ("section_offset", C.c_uint64 * 4), ("section_bytes", C.c_uint64 * 4), ("decoded_bytes", C.c_uint64),
                ("payload_sha256", C.c_uint8 * 32)]


PACK_DTYPES = {"F32": 0, "BF16": 1, "I64": 2, "FP4_E2M1": 3}


class Block(C.Structure):
    _fields_ = [("input_norm", C.c_void_p), ("qkv", Matrix), ("o", Matrix), ("post_norm", C.c_void_p),
                ("gate_up", Matrix), ("down", Matrix),
                # routed experts (config.experts != 0): router + host arrays of `experts` matrices
                ("router", Matrix), ("expert_gate", C.POINTER(Matrix)), ("expert_up", C.POINTER(Matrix)),
                ("expert_down", C.POINTER(Matrix))]


class Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn",
                                          "vocab", "draft_vocab", "rotary_dim")] + \
               [("rope_theta", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_uint32) for n in ("page_tokens", "kv_encoding", "mtp_kv_encoding", "activation_bf16",
                                          "draft_depth", "max_context", "split_tokens",
                                          "experts", "route_width", "expert_ffn")] + [("route_scale", C.c_float)]


class Weights(C.Structure):
    _fields_ = [("embedding", C.c_void_p), ("layers", C.POINTER(Block)), ("final_norm", C.c_void_p),
                ("head", Matrix), ("mtp_embedding_norm", C.c_void_p), ("mtp_hidden_norm", C.c_void_p),
                ("mtp_fusion", Matrix), ("mtp_block", Block), ("mtp_draft_norm", C.c_void_p)]


class Request(C.Structure):
    _fields_ = [("sampling_seed", C.c_uint64), ("sampling_temperature_ppm", C.c_uint32),
                ("sampling_top_p_ppm", C.c_uint32), ("sampling_top_k", C.c_uint32),
                ("sampling_min_p_ppm", C.c_uint32), ("reserved_context_tokens", C.c_uint32),
                ("sampling_presence_penalty_biased_ppm", C.c_uint32),
                ("sampling_first_output_position", C.c_uint32), ("reserved", C.c_uint32)]


class ExactResult(C.Structure):
    _fields_ = [("emitted_tokens", C.c_uint32 * 8), ("emitted_count", C.c_uint32),
                ("next_token", C.c_uint32), ("positions_advanced", C.c_uint32), ("rejected", C.c_uint32)]


u8, u32, u64, f32, f64, vp, sz, ci = (C.c_uint8, C.c_uint32, C.c_uint64, C.c_float, C.c_double,
                                      C.c_void_p, C.c_size_t, C.c_int)
P = C.POINTER

# name -> (restype, argtypes); kept in step with include/qllm_b200.h (tests check every
# declared symbol is exported).
SIGNATURES = {
    "qllm_last_error": (C.c_char_p, []),
    "qllm_capability_name": (C.c_char_p, []),
    "qllm_capability_abi": (u32, []),
    "qllm_provider_create": (ci, [P(Config), P(Weights), ci, ci, P(vp)]),
    "qllm_provider_destroy": (None, [vp]),
    "qllm_provider_create_request_state": (ci, [vp, P(vp)]),
    "qllm_provider_destroy_request_state": (None, [vp, vp]),
    "qllm_provider_prefill_chunk": (ci, [vp, vp, vp, u32, u32]),
    "qllm_provider_first_token": (ci, [vp, vp, P(Request), u32, P(u32)]),
    "qllm_provider_scalar_decode": (ci, [vp, vp, P(Request), u32, u32, ci, P(u32)]),
    "qllm_provider_checkpoint_request_state": (ci, [vp, vp, u32]),
    "qllm_provider_rewind_request_state": (ci, [vp, vp, u32]),
    "qllm_provider_synchronize_exact_decode_batch": (ci, [vp, vp, P(Request), vp, u32, u32, ci]),
    "qllm_provider_execute_exact_decode": (ci, [vp, vp, P(Request), u32, u32, u32, P(ExactResult)]),
    "qllm_provider_execute_exact_decode_steps": (ci, [vp, vp, P(Request), u32, u32, P(ExactResult)]),
    "qllm_provider_telemetry": (ci, [vp, vp, P(u64), u32]),
    "qllm_provider_stream": (vp, [vp]),
    "qllm_provider_max_chunk_rows": (u32, [vp]),
    "qllm_provider_set_graph_mode": (ci, [vp, ci]),
    "qllm_provider_set_gemv_impl": (ci, [vp, ci]),
    "qllm_provider_set_attention_impl": (ci, [vp, ci]),
    "qllm_pack_check_dense": (ci, [vp, sz, vp, ci]),
    "qllm_pack_nvfp4_matrix": (ci, [vp, sz, vp, ci, vp]),
    "qllm_pack_check_expert": (ci, [vp, sz, vp, ci]),
    "qllm_pack_nvfp4_expert": (ci, [vp, sz, vp, ci, vp, vp, vp]),
    "qllm_sha256": (None, [vp, sz, vp]),
    "qllm_descriptor_parse": (ci, [C.c_char_p, sz, P(vp)]),
    "qllm_descriptor_destroy": (None, [vp]),
    "qllm_descriptor_negotiate": (ci, [vp, vp]),
    "qllm_descriptor_tensor": (C.c_char_p, [vp, C.c_char_p]),
    "qllm_descriptor_dump": (sz, [vp, vp, sz]),
    "qllm_provider_tp_export": (ci, [vp, u32, u32, vp]),
    "qllm_provider_tp_attach": (ci, [vp, vp]),
    "qllm_provider_tp_area_bytes": (sz, [vp]),
    "qllm_provider_tp_attach_local": (ci, [vp, vp]),
    "qllm_provider_read_logits": (ci, [vp, vp, u32]),
    "qllm_provider_read_hidden": (ci, [vp, vp, ci, vp, u32]),
    "qllm_provider_read_drafts": (ci, [vp, vp, vp, P(u32)]),
    "qllm_provider_page_bytes": (sz, [vp]),
    "qllm_provider_layer_offset": (sz, [vp, u32]),
    "qllm_provider_read_page": (ci, [vp, vp, u32, vp]),
    "qllm_provider_fill_synthetic_kv": (ci, [vp, vp, u32, u32, u64]),
    "qllm_provider_time_verify": (ci, [vp, vp, P(Request), u32, P(f32)]),
    "qllm_k_embedding_bf16": (ci, [vp, vp, vp, u32, u32, u32, vp]),
    "qllm_k_rms_norm": (ci, [vp, vp, vp, u32, u32, f32, vp]),
    "qllm_k_nvfp4_fake_quant": (ci, [vp, vp, u32, u32, f32, vp]),
    "qllm_k_nvfp4_gemv_workspace_bytes": (sz, [u32, u32, u32]),
    "qllm_k_nvfp4_gemv": (ci, [P(Matrix), u32, u32, vp, vp, u32, vp, sz, ci, vp]),
    "qllm_k_nvfp4_gemv_static_scratch_bytes": (sz, []),
    "qllm_k_nvfp4_gemv_static": (ci, [P(Matrix), u32, u32, vp, vp, u32, vp]),
    "qllm_k_matrix_prepare": (ci, [P(Matrix), vp, P(vp)]),
    "qllm_k_matrix_release": (None, [vp]),
    "qllm_k_nvfp4_gemv_prepared": (ci, [vp, vp, vp, u32, vp, sz, ci, vp]),
    "qllm_k_nvfp4_gemv_prepared_core": (ci, [vp, u32, vp, sz, vp]),
    "qllm_k_nvfp4_quantize_weights": (ci, [vp, u32, u32, f32, vp, vp, vp]),
    "qllm_k_moe_route": (ci, [vp, u32, u32, u32, f32, vp, vp, vp]),
    "qllm_k_add": (ci, [vp, vp, u64, ci, vp]),
    "qllm_k_silu_product": (ci, [vp, vp, u32, u32, ci, vp]),
    "qllm_k_rope_kv_store": (ci, [vp, u32, u32, u32, u32, u32, vp, vp, u32, u32, vp, sz, u32, u32, ci, vp]),
    "qllm_k_kv_layer_bytes": (sz, [u32, u32, u32, u32]),
    "qllm_k_attention_workspace_bytes": (sz, [u32, u32, u32, u32]),
    "qllm_k_attention": (ci, [u32, vp, sz, u32, vp, u32, u32, vp, u32, u32, u32, u32, u32, u32, ci, vp, vp, ci, vp]),
    "qllm_k_argmax": (ci, [vp, u32, u32, u32, vp, vp]),
    "qllm_k_topk_workspace_bytes": (sz, [u32, u32, u32]),
    "qllm_k_topk": (ci, [vp, u32, u32, u32, u32, vp, vp, vp, vp]),
    "qllm_k_sample_token_workspace_bytes": (sz, [u32]),
    "qllm_k_sample_token": (ci, [vp, u32, u64, u32, u32, u32, u32, u32, vp, vp, vp, vp]),
    "qllm_k_rejection_sample_host": (ci, [u32, vp, vp, u32, vp, vp, u32, f64, f64, P(u32)]),
    "qllm_k_make_distribution_host": (ci, [vp, vp, u32, u32, u32, u32, vp, vp]),
    "qllm_k_counter_uniform_host": (ci, [u64, u32, u32, u32, P(f64)]),
}

_lib = None


def load():
    """Load the compiled library; raises when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m quantum_llm_b200.build` "
                              "(there is no CPU fallback)")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def check(status):
    if status < 0:
        raise QllmError(status, load().qllm_last_error().decode())
    return status
