"""ctypes binding of the CPU oracle (test infrastructure only).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
KV_F16, KV_Q4H, KV_Q8 = 0, 1, 2


class Matrix(C.Structure):
    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p),
                ("weight_scale", C.c_float), ("input_scale", C.c_float),
                ("rows", C.c_uint32), ("cols", C.c_uint32)]


class Block(C.Structure):
    _fields_ = [("input_norm", C.c_void_p), ("qkv", Matrix), ("o", Matrix),
                ("post_norm", C.c_void_p), ("gate_up", Matrix), ("down", Matrix),
                ("router", Matrix), ("expert_gate", C.POINTER(Matrix)), ("expert_up", C.POINTER(Matrix)),
                ("expert_down", C.POINTER(Matrix))]


class Config(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in
                ("layers", "hidden", "q_heads", "kv_heads", "head_dim", "ffn",
                 "vocab", "draft_vocab", "rotary_dim")] + \
               [("rope_theta", C.c_float), ("eps", C.c_float)] + \
               [(n, C.c_uint32) for n in
                ("page_tokens", "kv_encoding", "mtp_kv_encoding",
                 "activation_bf16", "draft_depth", "max_context", "split_tokens",
                 "experts", "route_width", "expert_ffn")] + [("route_scale", C.c_float)]


class Weights(C.Structure):
    _fields_ = [("embedding", C.c_void_p), ("layers", C.POINTER(Block)),
                ("final_norm", C.c_void_p), ("head", Matrix),
                ("mtp_embedding_norm", C.c_void_p), ("mtp_hidden_norm", C.c_void_p),
                ("mtp_fusion", Matrix), ("mtp_block", Block),
                ("mtp_draft_norm", C.c_void_p)]


class Request(C.Structure):
    _fields_ = [("seed", C.c_uint64), ("temperature_ppm", C.c_uint32),
                ("top_p_ppm", C.c_uint32), ("top_k", C.c_uint32),
                ("min_p_ppm", C.c_uint32), ("context_limit", C.c_uint32),
                ("presence_penalty_biased_ppm", C.c_uint32), ("first_output_position", C.c_uint32),
                ("reserved", C.c_uint32)]


class StepResult(C.Structure):
    _fields_ = [("emitted", C.c_uint32 * 8), ("emitted_count", C.c_uint32),
                ("next_token", C.c_uint32), ("positions_advanced", C.c_uint32),
                ("rejected", C.c_uint32)]


def reference_root():
    """Where the reference's source tree lies: QLLM_REFERENCE, else a directory named
    `reference` beside this repository; "" when neither exists."""
    env = os.environ.get("QLLM_REFERENCE", "")
    if env:
        return env
    sibling = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return sibling if os.path.isdir(os.path.join(sibling, "runtime")) else ""


REFERENCE_DEFAULT = reference_root()


def build(force=False):
    """Compile the oracle (and oracle/_ref when the reference tree exists)."""
    lib = os.path.join(HERE, "libqllm_oracle.so")
    src_time = max(os.path.getmtime(os.path.join(HERE, f))
                   for f in ("qllm_oracle.cpp", "qllm_oracle.h"))
    if force or not os.path.exists(lib) or os.path.getmtime(lib) < src_time:
        subprocess.run(["make", "-C", HERE, "libqllm_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    # the reference's own sampler and descriptor parser, where the reference tree is present
    # (reference_root()); prebuilt files are kept otherwise
    refs = [os.path.join(HERE, "_ref", name) for name in ("libqllm_ref_sampler.so", "libqllm_ref_descriptor.so")]
    reference = reference_root()
    shims = [os.path.join(HERE, name) for name in ("ref_sampler_shim.cpp", "ref_descriptor_shim.cpp")]
    stale = not all(os.path.exists(r) for r in refs) or any(
        os.path.getmtime(r) < os.path.getmtime(sh) for r, sh in zip(refs, shims))
    if (force or stale) and reference and os.path.isdir(reference):
        subprocess.run(["make", "-C", HERE, "ref", f"REFERENCE={reference}"], check=True, stdout=subprocess.DEVNULL)
    # the reference's own CUDA kernels (GPU pins of the oracle): built once, where the reference tree lies
    kernels = os.path.join(HERE, "_ref", "libqllm_ref_kernels.so")
    shim = os.path.join(HERE, "ref_kernels_shim.cu")
    if reference and os.path.isdir(reference) and (
            force or not os.path.exists(kernels) or os.path.getmtime(kernels) < os.path.getmtime(shim)):
        subprocess.run(["make", "-C", HERE, "ref_kernels", f"REFERENCE={reference}"], check=True,
                       stdout=subprocess.DEVNULL)
    # the reference's own CPU FFN executor (benchmark's CPU leg)
    host = os.path.join(HERE, "_ref", "libqllm_ref_fp4_host.so")
    host_shim = os.path.join(HERE, "ref_fp4_host_shim.cpp")
    if reference and os.path.isdir(reference) and (
            force or not os.path.exists(host) or os.path.getmtime(host) < os.path.getmtime(host_shim)):
        subprocess.run(["make", "-C", HERE, "ref_fp4_host", f"REFERENCE={reference}"], check=True,
                       stdout=subprocess.DEVNULL)
    return lib


_lib = None
_ref = None


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        u8, u16, u32, u64, f32, f64, vp, sz = (C.c_uint8, C.c_uint16, C.c_uint32, C.c_uint64,
                                               C.c_float, C.c_double, C.c_void_p, C.c_size_t)
        sig = {
            "qo_e2m1_decode": (f32, [u8]), "qo_e2m1_encode": (u8, [f32]),
            "qo_e4m3_decode": (f32, [u8]), "qo_e4m3_encode": (u8, [f32]),
            "qo_bf16_round": (f32, [f32]), "qo_f16_bits": (u16, [f32]), "qo_f16_value": (f32, [u16]),
            "qo_nvfp4_quantize_weights": (None, [vp, u32, u32, f32, vp, vp]),
            "qo_nvfp4_dequant": (None, [C.POINTER(Matrix), vp]),
            "qo_nvfp4_fake_quant": (None, [vp, u32, u32, f32, vp]),
            "qo_nvfp4_quantize_activations": (None, [vp, u32, u32, f32, vp, vp]),
            "qo_nvfp4_gemv": (None, [C.POINTER(Matrix), u32, u32, vp, u32, vp]),
            "qo_rmsnorm": (None, [vp, vp, vp, u32, u32, f32]),
            "qo_rope": (None, [vp, u32, u32, u32, u32, f32, vp, C.c_int]),
            "qo_kv_layer_bytes": (sz, [u32, u32, u32, u32]),
            "qo_kv_store": (None, [u32, vp, sz, u32, u32, u32, vp, vp, u32, u32, u32]),
            "qo_attention": (None, [u32, vp, sz, u32, vp, u32, u32, u32, u32, u32, u32, u32, C.c_int, vp]),
            "qo_argmax": (u32, [vp, u32]), "qo_set_threads": (None, [u32]), "qo_moe_route": (None, [vp, u32, u32, C.c_float, vp, vp]), "qo_max_threads": (u32, []), "qo_topk": (None, [vp, u32, u32, vp, vp]),
            "qo_counter_uniform": (f64, [u64, u32, u32, u32]),
            "qo_make_distribution": (C.c_int, [vp, vp, u32, u32, u32, u32, vp, vp]),
            "qo_sample_distribution": (u32, [vp, vp, u32, f64]),
            "qo_rejection_sample": (C.c_int, [u32, vp, vp, u32, vp, vp, u32, f64, f64, vp]),
            "qo_sample_token": (C.c_int, [vp, u32, C.POINTER(Request), u32, vp]),
            "qo_session_create": (vp, [C.POINTER(Config), C.POINTER(Weights)]),
            "qo_session_destroy": (None, [vp]),
            "qo_prefill": (C.c_int, [vp, vp, u32, u32, C.POINTER(Request), vp]),
            "qo_prefill_at": (C.c_int, [vp, vp, u32, u32, u32, C.POINTER(Request), vp]),
            "qo_fill_synthetic_kv": (C.c_int, [vp, u32, u32, u64]),
            "qo_execute_exact_decode": (C.c_int, [vp, C.POINTER(Request), u32, u32, C.POINTER(StepResult)]),
            "qo_draft_count": (u32, [vp]), "qo_drafts": (None, [vp, vp]),
            "qo_last_logits": (vp, [vp]), "qo_last_hidden": (vp, [vp]),
            "qo_page_bytes": (sz, [vp]), "qo_page_count": (u32, [vp]), "qo_page": (vp, [vp, u32]),
            "qo_layer_offset": (sz, [vp, u32]), "qo_mtp_length": (u32, [vp]),
            "qo_last_error": (C.c_char_p, []),
        }
        for name, (res, args) in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = res, args
        _lib = L
    return _lib


def ref_sampler():
    """The reference's own sampler (oracle/_ref), or None when it was not built."""
    global _ref
    if _ref is None:
        build()
        path = os.path.join(HERE, "_ref", "libqllm_ref_sampler.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        u32, u64, f64, vp = C.c_uint32, C.c_uint64, C.c_double, C.c_void_p
        R.ref_counter_uniform.restype, R.ref_counter_uniform.argtypes = f64, [u64, u32, u32, u32]
        R.ref_make_distribution.restype = C.c_int
        R.ref_make_distribution.argtypes = [vp, vp, u32, u32, u32, u32, vp, vp]
        if hasattr(R, "ref_acceptance_seconds_per_step"):
            R.ref_acceptance_seconds_per_step.restype = C.c_double
            R.ref_acceptance_seconds_per_step.argtypes = [u32, u32, C.c_uint64, C.POINTER(C.c_uint64)]
        R.ref_sample_distribution.restype = C.c_int
        R.ref_sample_distribution.argtypes = [vp, vp, u32, f64, vp]
        R.ref_rejection_sample.restype = C.c_int
        R.ref_rejection_sample.argtypes = [u32, vp, vp, u32, vp, vp, u32, f64, f64, vp]
        _ref = R
    return _ref


_ref_kernels = None


_ref_fp4_host = None


def ref_fp4_host():
    """The reference's own CPU FFN executor (runtime/src/cpu/fp4_host_executor.cpp) behind
    oracle/ref_fp4_host_shim.cpp, or None when it was not built or this host has no AVX2."""
    global _ref_fp4_host
    if _ref_fp4_host is None:
        build()
        path = os.path.join(HERE, "_ref", "libqllm_ref_fp4_host.so")
        try:
            flags = open("/proc/cpuinfo").read()
        except OSError:
            flags = ""
        if not os.path.exists(path) or " avx2" not in flags:
            return None
        R = C.CDLL(path)
        R.ref_fp4_host_ffn_seconds.restype = C.c_double
        R.ref_fp4_host_ffn_seconds.argtypes = [C.c_uint32] * 5 + [C.c_uint64, C.POINTER(C.c_double)]
        _ref_fp4_host = R
    return _ref_fp4_host


def ref_kernels():
    """The reference's own CUDA kernels behind oracle/ref_kernels_shim.cu (oracle/_ref), or None
    when they were not built.  Needs a GPU to call."""
    global _ref_kernels
    if _ref_kernels is None:
        build()
        path = os.path.join(HERE, "_ref", "libqllm_ref_kernels.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        u32, f32, vp, sz, i = C.c_uint32, C.c_float, C.c_void_p, C.c_size_t, C.c_int
        sig = {
            "qr_last_error": (C.c_char_p, []),
            "qr_nvfp4_gemv": (i, [vp, vp, f32, f32, u32, u32, vp, vp, vp, u32]),
            "qr_store_q4h": (i, [vp, vp, vp, u32, u32, u32, u32, u32, u32]),
            "qr_store_q8": (i, [vp, vp, vp, u32, u32, u32, u32, u32, u32]),
            "qr_quantize_queries_q8": (i, [vp, vp, vp, u32, u32, u32]),
            "qr_attention_q4h": (i, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, u32, i]),
            "qr_attention_q8": (i, [vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32, u32, u32, i]),
            "qr_argmax_batch": (i, [vp, u32, u32, vp]),
            "qr_topk_workspace_items": (sz, [u32]),
            "qr_topk": (i, [vp, u32, u32, vp, vp, vp, sz, vp, sz]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(R, name)
            fn.restype, fn.argtypes = res, args
        _ref_kernels = R
    return _ref_kernels


# ------------------------------------------------------------------ helpers
def quantize_weights(w, global_scale):
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, cols = w.shape
    codes = np.empty((rows, cols // 2), np.uint8)
    scales = np.empty((rows, cols // 16), np.uint8)
    lib().qo_nvfp4_quantize_weights(_ptr(w), rows, cols, np.float32(global_scale), _ptr(codes), _ptr(scales))
    return codes, scales


def matrix(codes, scales, weight_scale, input_scale):
    return Matrix(_ptr(codes), _ptr(scales), float(weight_scale), float(input_scale),
                  codes.shape[0], codes.shape[1] * 2)


def gemv(m, x, first_row=0, row_count=None):
    x = np.ascontiguousarray(x, dtype=np.float32)
    row_count = m.rows if row_count is None else row_count
    y = np.empty((x.shape[0], row_count), np.float32)
    lib().qo_nvfp4_gemv(C.byref(m), first_row, row_count, _ptr(x), x.shape[0], _ptr(y))
    return y


def make_distribution(logits, tokens, temperature_ppm, top_p_ppm, min_p_ppm, impl=None):
    logits = np.ascontiguousarray(logits, np.float32)
    tokens = np.ascontiguousarray(tokens, np.uint32)
    ot = np.empty(len(tokens), np.uint32)
    op = np.empty(len(tokens), np.float64)
    fn = lib().qo_make_distribution if impl is None else impl.ref_make_distribution
    n = fn(_ptr(logits), _ptr(tokens), len(tokens), temperature_ppm, top_p_ppm, min_p_ppm, _ptr(ot), _ptr(op))
    if n < 0:
        return None
    return ot[:n].copy(), op[:n].copy()


def sample_token(logits, request, position):
    """The scalar decode fallback's sampler over a whole logits row; None where the reference throws."""
    logits = np.ascontiguousarray(logits, np.float32)
    token = C.c_uint32(0)
    rc = lib().qo_sample_token(_ptr(logits), logits.size, C.byref(request), int(position), C.byref(token))
    return token.value if rc == 0 else None


def rejection_sample(proposal, target, draft, ua, uc, impl=None):
    tt, tp = (np.ascontiguousarray(target[0], np.uint32), np.ascontiguousarray(target[1], np.float64))
    dt, dp = (np.ascontiguousarray(draft[0], np.uint32), np.ascontiguousarray(draft[1], np.float64))
    token = C.c_uint32(0)
    fn = lib().qo_rejection_sample if impl is None else impl.ref_rejection_sample
    r = fn(int(proposal), _ptr(tt), _ptr(tp), len(tt), _ptr(dt), _ptr(dp), len(dt), ua, uc, C.byref(token))
    return r, token.value


class Session:
    """Whole-step oracle over a synthetic model (see tests/synth.py)."""

    def __init__(self, config, weights, keepalive):
        self._keep = (config, weights, keepalive)
        self.config = config
        self.h = lib().qo_session_create(C.byref(config), C.byref(weights))
        if not self.h:
            raise RuntimeError(lib().qo_last_error().decode())

    def close(self):
        if self.h:
            lib().qo_session_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:   # interpreter shutdown: the module globals may be gone already
            pass

    def prefill(self, tokens, chunk_rows, request):
        tokens = np.ascontiguousarray(tokens, np.uint32)
        first = C.c_uint32(0)
        if lib().qo_prefill(self.h, _ptr(tokens), len(tokens), chunk_rows, C.byref(request), C.byref(first)):
            raise RuntimeError(lib().qo_last_error().decode())
        return first.value

    def prefill_at(self, tokens, base, chunk_rows, request):
        """Prompt positions [base, base + len(tokens)) behind a cached prefix of `base` positions."""
        tokens = np.ascontiguousarray(tokens, np.uint32)
        first = C.c_uint32(0)
        if lib().qo_prefill_at(self.h, _ptr(tokens), len(tokens), base, chunk_rows, C.byref(request), C.byref(first)):
            raise RuntimeError(lib().qo_last_error().decode())
        return first.value

    def fill_synthetic_kv(self, first, count, seed):
        if lib().qo_fill_synthetic_kv(self.h, first, count, seed):
            raise RuntimeError(lib().qo_last_error().decode())

    def execute_exact_decode(self, request, guaranteed_token, position):
        res = StepResult()
        if lib().qo_execute_exact_decode(self.h, C.byref(request), guaranteed_token, position, C.byref(res)):
            raise RuntimeError(lib().qo_last_error().decode())
        return res

    def drafts(self):
        n = lib().qo_draft_count(self.h)
        out = np.zeros(max(n, 1), np.uint32)
        lib().qo_drafts(self.h, _ptr(out))
        return out[:n].copy()

    def last_logits(self, rows):
        p = lib().qo_last_logits(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), (rows, self.config.vocab)).copy()

    def last_hidden(self, rows):
        p = lib().qo_last_hidden(self.h)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), (rows, self.config.hidden)).copy()

    def page(self, index):
        n = lib().qo_page_bytes(self.h)
        p = lib().qo_page(self.h, index)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), (n,)).copy()

    def layer_offset(self, layer):
        return lib().qo_layer_offset(self.h, layer)

    @property
    def mtp_length(self):
        return lib().qo_mtp_length(self.h)
