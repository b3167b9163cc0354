"""qllm_k_nvfp4_gemv_static: the NVFP4 GEMV whose workspace is a fixed array inside the
library, for callers that cannot allocate device memory at call time.  Checked through the
C ABI against the CPU oracle's GEMV and against qllm_k_nvfp4_gemv (CUDA-core implementation)
on two calls in a row that share the array, for its size limit, and for the argument checks
that run on the host before anything is launched (row range that wraps, misaligned pointers).  Collected last on purpose: it must pass alone and after
every other test has used the device."""
import ctypes as C

import numpy as np
import pytest

from tests import synth
from tests.gpu_util import dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    import torch
    assert torch.cuda.is_available()
    from quantum_llm_b200 import lib
    return lib.load()


def _matrix(rng, rows, cols):
    from quantum_llm_b200 import lib
    m = synth.SynthMatrix(rng.normal(0, 0.02, (rows, cols)).astype(np.float32))
    dc, ds = dev(m.codes), dev(m.scales)
    cm = lib.Matrix(dc.data_ptr(), ds.data_ptr(), float(m.weight_scale), float(m.input_scale), rows, cols)
    return cm, (dc, ds, m)


def _reference(L, cm, x, rows, cols, batch):
    import torch
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(batch, rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    rc = L.qllm_k_nvfp4_gemv(C.byref(cm), 0, rows, x.data_ptr(), y.data_ptr(), batch, ws.data_ptr(), ws_bytes, 0, None)
    assert rc == 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    return y.cpu().numpy()


def test_static_scratch_gemv_equals_the_workspace_form_on_consecutive_calls(L):
    import torch
    rng = np.random.default_rng(77)
    # two different shapes back to back: the second call reuses (and overwrites) the array
    cases = [(512, 1024, 5), (384, 2048, 3)]
    prepared = []
    for rows, cols, batch in cases:
        cm, keep = _matrix(rng, rows, cols)
        x = dev(rng.normal(0, 1, (batch, cols)).astype(np.float32))
        prepared.append((cm, keep, x, rows, cols, batch, _reference(L, cm, x, rows, cols, batch)))
    outs = []
    for cm, keep, x, rows, cols, batch, want in prepared:   # no synchronisation in between
        y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
        rc = L.qllm_k_nvfp4_gemv_static(C.byref(cm), 0, rows, x.data_ptr(), y.data_ptr(), batch, None)
        assert rc == 0, L.qllm_last_error().decode()
        outs.append(y)
    torch.cuda.synchronize()
    from oracle import binding as ob
    for y, case in zip(outs, prepared):
        assert np.array_equal(y.cpu().numpy(), case[-1])
        cm, keep, x, rows, cols, batch, want = case
        assert np.array_equal(y.cpu().numpy(), ob.gemv(keep[2].oracle(), x.cpu().numpy())), "static-scratch GEMV vs the CPU oracle"
    # and once more with the first shape, after the array held the second one
    cm, keep, x, rows, cols, batch, want = prepared[0]
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
    assert L.qllm_k_nvfp4_gemv_static(C.byref(cm), 0, rows, x.data_ptr(), y.data_ptr(), batch, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), want)


def test_static_scratch_gemv_rejects_what_does_not_fit(L):
    import torch
    limit = L.qllm_k_nvfp4_gemv_static_scratch_bytes()
    assert limit == 2 << 20
    rng = np.random.default_rng(78)
    rows, cols = 128, 4096
    cm, keep = _matrix(rng, rows, cols)
    batch = limit // cols + 1           # batch * cols * 1.25 bytes is beyond the array
    x = torch.zeros((batch, cols), dtype=torch.float32, device="cuda")
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
    rc = L.qllm_k_nvfp4_gemv_static(C.byref(cm), 0, rows, x.data_ptr(), y.data_ptr(), batch, None)
    assert rc == -4 and b"static array holds" in L.qllm_last_error()


def test_static_scratch_gemv_checks_its_arguments_on_the_host(L):
    import torch
    rng = np.random.default_rng(79)
    rows, cols, batch = 256, 512, 2
    cm, keep = _matrix(rng, rows, cols)
    x = torch.zeros((batch, cols + 4), dtype=torch.float32, device="cuda")
    y = torch.full((batch, rows), 7.0, dtype=torch.float32, device="cuda")
    call = L.qllm_k_nvfp4_gemv_static
    # first_row + row_count wraps around 2^32: refused, not taken for a short range
    assert call(C.byref(cm), 0xFFFFFF00, 0x200, x.data_ptr(), y.data_ptr(), batch, None) == -4
    assert call(C.byref(cm), rows, 1, x.data_ptr(), y.data_ptr(), batch, None) == -4
    assert call(C.byref(cm), 0, rows + 1, x.data_ptr(), y.data_ptr(), batch, None) == -4
    # activations must be 16-byte aligned (vector loads), codes 8-byte aligned
    assert call(C.byref(cm), 0, rows, x.data_ptr() + 4, y.data_ptr(), batch, None) == -4
    from quantum_llm_b200 import lib
    odd = lib.Matrix(cm.codes + 1, cm.scales, cm.weight_scale, cm.input_scale, rows, cols)
    assert call(C.byref(odd), 0, rows, x.data_ptr(), y.data_ptr(), batch, None) == -4
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()), "a refused call must not launch anything"
    # the caller-workspace form applies the same checks
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(batch, rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    plain = L.qllm_k_nvfp4_gemv
    assert plain(C.byref(cm), 0xFFFFFF00, 0x200, x.data_ptr(), y.data_ptr(), batch, ws.data_ptr(), ws_bytes, 0, None) == -4
    assert plain(C.byref(cm), 0, rows, x.data_ptr() + 4, y.data_ptr(), batch, ws.data_ptr(), ws_bytes, 0, None) == -4
    assert plain(C.byref(odd), 0, rows, x.data_ptr(), y.data_ptr(), batch, ws.data_ptr(), ws_bytes, 0, None) == -4
