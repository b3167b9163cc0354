"""CPU checks of the drop-in boundary: the library loads without a GPU and
exports every entry point that include/qllm_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "qllm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qllm_[a-z0-9_]+)\s*\(", text)))


def test_build_produces_library():
    from quantum_llm_b200 import build
    assert os.path.exists(build.build())


def test_every_declared_symbol_is_exported_and_bound():
    from quantum_llm_b200 import lib
    L = ctypes.CDLL(lib.LIB_PATH)
    names = declared_symbols()
    assert len(names) >= 35
    for name in names:
        assert hasattr(L, name), f"{name} declared in include/qllm_b200.h but not exported"
        assert name in lib.SIGNATURES, f"{name} has no ctypes signature"
    assert sorted(lib.SIGNATURES) == names


def test_capability_follows_reference_naming():
    from quantum_llm_b200 import Nvfp4MtpProvider
    name, abi = Nvfp4MtpProvider.capability()
    # reference capability: decode.mtp.dense-full-attention.fp4-block32.exact.v2, ABI 2
    assert name.startswith("decode.mtp.dense-full-attention.nvfp4-block16.exact") and abi == 2


def test_struct_layouts_match_the_oracle_structs():
    # the harness builds both sides from the same numpy arrays, so the C layouts must agree
    from oracle import binding as ob
    from quantum_llm_b200 import lib
    for a, b in ((lib.Matrix, ob.Matrix), (lib.Block, ob.Block), (lib.Config, ob.Config),
                 (lib.Weights, ob.Weights), (lib.Request, ob.Request), (lib.ExactResult, ob.StepResult)):
        assert ctypes.sizeof(a) == ctypes.sizeof(b)
        assert [f[0] for f in a._fields_][:3] and len(a._fields_) == len(b._fields_)


def test_missing_library_fails_loudly(monkeypatch):
    from quantum_llm_b200 import lib
    monkeypatch.setattr(lib, "_lib", None)
    monkeypatch.setattr(lib, "LIB_PATH", "/nonexistent/libqllm_b200.so")
    with pytest.raises(ImportError):
        lib.load()


def test_no_gpu_means_error_not_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from quantum_llm_b200 import lib
    L = lib.load()
    out = ctypes.c_double(0)
    assert L.qllm_k_counter_uniform_host(1, 2, 3, 4, ctypes.byref(out)) < 0
    assert b"probe alloc" in L.qllm_last_error() or L.qllm_last_error()


def test_gemv_entry_points_reject_bad_arguments_before_any_cuda_call():
    """Row ranges that wrap around 2^32 and misaligned operands are refused on the host (status -4,
    QLLM_INVALID_ARGUMENT) by the caller-workspace GEMV and by the static-scratch GEMV alike; the
    checks precede every CUDA call, so they run here without a GPU (the pointers are never read)."""
    from quantum_llm_b200 import lib
    L = lib.load()
    rows, cols, batch = 256, 512, 2
    m = lib.Matrix(0x10000, 0x20000, 1.0, 1.0, rows, cols)
    odd = lib.Matrix(0x10001, 0x20000, 1.0, 1.0, rows, cols)
    x, y, ws = 0x30000, 0x40000, 0x50000
    static, plain = L.qllm_k_nvfp4_gemv_static, L.qllm_k_nvfp4_gemv
    for first, count in ((0xFFFFFF00, 0x200), (rows, 1), (0, rows + 1), (1, 0xFFFFFFFF)):
        assert static(ctypes.byref(m), first, count, x, y, batch, None) == -4
        assert plain(ctypes.byref(m), first, count, x, y, batch, ws, 1 << 20, 0, None) == -4
    assert static(ctypes.byref(m), 0, rows, x + 4, y, batch, None) == -4
    assert static(ctypes.byref(odd), 0, rows, x, y, batch, None) == -4
    assert plain(ctypes.byref(m), 0, rows, x + 4, y, batch, ws, 1 << 20, 0, None) == -4
    assert plain(ctypes.byref(m), 0, rows, x, y, batch, ws + 8, 1 << 20, 0, None) == -4
    assert plain(ctypes.byref(odd), 0, rows, x, y, batch, ws, 1 << 20, 0, None) == -4
    assert b"boundar" in L.qllm_last_error()
    # the static array's size limit is a host-side check too
    limit = L.qllm_k_nvfp4_gemv_static_scratch_bytes()
    wide = lib.Matrix(0x10000, 0x20000, 1.0, 1.0, 128, 4096)
    assert static(ctypes.byref(wide), 0, 128, x, y, limit // 4096 + 1, None) == -4
    assert b"static array holds" in L.qllm_last_error()
