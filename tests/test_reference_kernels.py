"""GPU pins of the CPU oracle against the reference's OWN CUDA kernels.

oracle/Makefile (`make ref_kernels`) compiles the reference's runtime/src/cuda/transformer_kernels.cu,
unmodified, for sm_100a behind oracle/ref_kernels_shim.cu into oracle/_ref/libqllm_ref_kernels.so.
Here those kernels run on small cases shaped like the reference's own smoke fixtures
(runtime/tools/native_nvfp4_cuda_smoke.cpp:76-269, runtime/tools/dense_fp4_cuda_smoke.cpp:1551-2106,
:895-1178, :4307-) and three things are compared on the same inputs: the reference kernel, the
CPU oracle, and this library's kernel through its C ABI.  Byte and index work must be identical;
floating-point results use the reference's own gates (2e-4 for Q4H attention against a host
mirror of its INT8 approximations, 2e-3 for the Q8 cache, one BF16 step for the GEMV, whose
FP32 summation order is free)."""
import ctypes as C

import numpy as np
import pytest

from oracle import binding as ob
from tests import synth
from tests.gpu_util import bf16_ulps, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def R():
    import torch
    assert torch.cuda.is_available()
    ref = ob.ref_kernels()
    if ref is None:
        pytest.skip("oracle/_ref/libqllm_ref_kernels.so was not built (needs the reference tree at build time)")
    return ref


@pytest.fixture(scope="module")
def L():
    from quantum_llm_b200 import lib
    return lib.load()


def _ok(R, rc):
    assert rc == 0, R.qr_last_error().decode()


def _okl(L, rc):
    assert rc >= 0, L.qllm_last_error().decode()


def _sync():
    import torch
    torch.cuda.synchronize()


def _fixture_matrix(seed, rows, cols):
    """Deterministic nibble pattern in the style of the reference's NVFP4 smoke fixture (non-zero
    magnitudes 1..7, alternating signs on the high nibble) with every block scale 1.0 (0x38)."""
    r = np.arange(rows, dtype=np.uint32)[:, None]
    p = np.arange(cols // 2, dtype=np.uint32)[None, :]
    low = 1 + (seed + r + 3 * p) % 7
    high = (1 + (seed + 2 * r + p) % 7) | np.where((seed + r + p) & 1, 8, 0)
    codes = (low | (high << 4)).astype(np.uint8)
    scales = np.full((rows, cols // 16), 0x38, np.uint8)
    return codes, scales


@pytest.mark.parametrize("case", ["fixture64", "random640x1024", "random256x512_batch8"])
def test_nvfp4_quantiser_and_gemv(R, L, case):
    import torch
    from quantum_llm_b200 import lib
    rng = np.random.default_rng(len(case))
    if case == "fixture64":
        rows, cols, batch = 64, 64, 5
        codes, scales = _fixture_matrix(3, rows, cols)
        weight_scale, input_scale = np.float32(1.0 / 96.0), np.float32(64.0)
        x = rng.normal(0, 1, (batch, cols)).astype(np.float32)
    else:
        rows, cols, batch = (640, 1024, 5) if "640" in case else (256, 512, 8)
        m = synth.SynthMatrix(rng.normal(0, 0.02, (rows, cols)).astype(np.float32))
        codes, scales, weight_scale, input_scale = m.codes, m.scales, m.weight_scale, m.input_scale
        x = (rng.normal(0, 1, (batch, cols)) * rng.choice([1e-2, 1, 8], (batch, 1))).astype(np.float32)
        x[0, :16] = 0                                   # an all-zero block: scale 0, codes 0
    dc, ds, dx = dev(codes), dev(scales), dev(x)
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda")
    qdq = torch.empty((batch, cols), dtype=torch.float32, device="cuda")
    _ok(R, R.qr_nvfp4_gemv(dc.data_ptr(), ds.data_ptr(), float(weight_scale), float(input_scale), rows, cols,
                           dx.data_ptr(), y.data_ptr(), qdq.data_ptr(), batch))
    ref_y, ref_qdq = y.cpu().numpy(), qdq.cpu().numpy()
    # activation quantise/dequantise: the same bits as the oracle
    want_qdq = np.empty_like(x)
    ob.lib().qo_nvfp4_fake_quant(ob._ptr(x), batch, cols, np.float32(input_scale), ob._ptr(want_qdq))
    assert np.array_equal(ref_qdq.view(np.uint32), want_qdq.view(np.uint32))
    # GEMV: the reference sums FP32 products in lane order, the oracle sums exact block terms in
    # double; both round to BF16 -> at most one BF16 step apart, on few elements
    om = ob.matrix(np.ascontiguousarray(codes), np.ascontiguousarray(scales), weight_scale, input_scale)
    want = ob.gemv(om, x)
    assert bf16_ulps(ref_y, want).max() <= 1
    assert (ref_y != want).mean() < 0.02
    # this library's kernels against the reference kernel
    cm = lib.Matrix(dc.data_ptr(), ds.data_ptr(), float(weight_scale), float(input_scale), rows, cols)
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(batch, rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    for impl in (0, 1):
        if impl == 1 and cols % 256:
            continue
        _okl(L, L.qllm_k_nvfp4_gemv(C.byref(cm), 0, rows, dx.data_ptr(), y.data_ptr(), batch, ws.data_ptr(), ws_bytes,
                                    impl, None)); _sync()
        got = y.cpu().numpy()
        close = (bf16_ulps(got, ref_y) <= 1) | (np.abs(got - ref_y) <= 1e-3 * np.sqrt((ref_y ** 2).mean()))
        assert close.all() and (got != ref_y).mean() < 0.02, (impl, np.abs(got - ref_y).max())


def _device_pages(layer_bytes, layers, count):
    import torch
    pages = [torch.zeros(layer_bytes * layers, dtype=torch.uint8, device="cuda") for _ in range(count)]
    table = dev(np.array([p.data_ptr() for p in pages], np.uint64))
    return pages, table


def _host_pages(layer_bytes, layers, count):
    pages = [np.zeros(layer_bytes * layers, np.uint8) for _ in range(count)]
    return pages, (C.c_void_p * count)(*[p.ctypes.data for p in pages])


@pytest.mark.parametrize("enc,hd", [(ob.KV_Q4H, 256), (ob.KV_Q8, 128), (ob.KV_Q8, 256), (ob.KV_Q8, 64)])
def test_kv_record_bytes(R, L, enc, hd):
    """Q4H (the reference kernel takes head_dim 256 only) and Q8 records: reference kernel, oracle and
    this library's store kernel write identical page bytes, in a layer at a non-zero offset, for rows
    that straddle a page boundary, with an all-zero head and a dominant element among them."""
    import torch
    rng = np.random.default_rng(enc * 1000 + hd)
    kv, pt, rows, first, layer, layers, qh = 4, 64, 5, 61, 1, 2, 4
    k = torch.from_numpy(rng.normal(0, 1.3, (rows, kv * hd)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    v = torch.from_numpy(rng.normal(0, 0.8, (rows, kv * hd)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    k[1, hd:2 * hd] = 0
    v[2, 3] = 29952.0           # (BF16-representable, like every activation on this path)
    k[3, 7] = -65024.0          # record scale near the top of the F16 range
    layer_bytes = ob.lib().qo_kv_layer_bytes(enc, pt, kv, hd)
    # reference kernel
    ref_pages, ref_table = _device_pages(layer_bytes, layers, 2)
    dk, dv = dev(k), dev(v)
    store = R.qr_store_q4h if enc == ob.KV_Q4H else R.qr_store_q8
    _ok(R, store(dk.data_ptr(), dv.data_ptr(), ref_table.data_ptr(), layer, pt, first, rows, kv, hd))
    # oracle
    host_pages, host_table = _host_pages(layer_bytes, layers, 2)
    ob.lib().qo_kv_store(enc, host_table, layer * layer_bytes, pt, kv, hd, ob._ptr(k), ob._ptr(v), rows, kv * hd, first)
    for i in range(2):
        assert np.array_equal(ref_pages[i].cpu().numpy(), host_pages[i]), f"oracle page {i} differs from the reference kernel"
    # this library (rotary_dim 0: store the rows as they are)
    our_pages, our_table = _device_pages(layer_bytes, layers, 2)
    qkv = np.concatenate([np.zeros((rows, qh * hd), np.float32), k, v], axis=1)
    dq = dev(qkv)
    dinv = dev(np.ones(max(hd // 2, 1), np.float32)); dpos = dev(np.array([first], np.uint32))
    _okl(L, L.qllm_k_rope_kv_store(dq.data_ptr(), rows, qh, kv, hd, 0, dinv.data_ptr(), dpos.data_ptr(), 0, 0,
                                   our_table.data_ptr(), layer * layer_bytes, pt, enc, 1, None)); _sync()
    for i in range(2):
        assert np.array_equal(our_pages[i].cpu().numpy(), ref_pages[i].cpu().numpy()), f"page {i} differs from the reference kernel"


def _gated(q, qh, hd, gate=40.0):
    """[rows, qh*hd] queries -> the reference's [rows, qh, 2*hd] layout with an output gate whose
    sigmoid is exactly 1 in FP32, so that its gated attention equals plain attention."""
    rows = q.shape[0]
    out = np.full((rows, qh, 2 * hd), gate, np.float32)
    out[:, :, :hd] = q.reshape(rows, qh, hd)
    return np.ascontiguousarray(out.reshape(rows, qh * 2 * hd))


@pytest.mark.parametrize("ctx,rows,qh,kv", [(4, 5, 24, 4), (300, 5, 24, 4), (1000, 2, 16, 2), (77, 1, 8, 1)])
def test_q4h_attention(R, L, ctx, rows, qh, kv):
    """The reference's batch-5 Q4H attention (head_dim 256; first case = its smoke geometry: 24 q / 4 kv
    heads, 8 stored tokens, first row sees 4) against the oracle (< 2e-4) and against this library."""
    import torch
    hd, pt, split = 256, 64, 64
    rng = np.random.default_rng(ctx * 31 + rows)
    tokens = ctx + rows - 1
    count = (tokens + pt - 1) // pt
    layer_bytes = ob.lib().qo_kv_layer_bytes(ob.KV_Q4H, pt, kv, hd)
    host_pages, host_table = _host_pages(layer_bytes, 1, count)
    k = rng.normal(0, 1.0, (tokens, kv * hd)).astype(np.float32)
    v = rng.normal(0, 1.0, (tokens, kv * hd)).astype(np.float32)
    ob.lib().qo_kv_store(ob.KV_Q4H, host_table, 0, pt, kv, hd, ob._ptr(k), ob._ptr(v), tokens, kv * hd, 0)
    q = rng.normal(0, 1.0, (rows, qh * hd)).astype(np.float32)
    want = np.empty((rows, qh * hd), np.float32)
    ob.lib().qo_attention(ob.KV_Q4H, host_table, 0, pt, ob._ptr(q), qh * hd, rows, ctx, qh, kv, hd, split, 1, ob._ptr(want))
    # reference: INT8 queries by its own kernel, then the tensor-core attention + combine
    dpages = [dev(p) for p in host_pages]
    dtable = dev(np.array([p.data_ptr() for p in dpages], np.uint64))
    dqg = dev(_gated(q, qh, hd))
    q8 = torch.empty((rows, qh, hd), dtype=torch.int8, device="cuda")
    qs = torch.empty((rows, qh), dtype=torch.float32, device="cuda")
    _ok(R, R.qr_quantize_queries_q8(dqg.data_ptr(), q8.data_ptr(), qs.data_ptr(), rows, qh, hd))
    # its INT8 query codes follow scale = max(absmax/127, 2^-24), code = rn(q / scale)
    qr = q.reshape(rows, qh, hd)
    scale = np.maximum(np.abs(qr).max(axis=2) / np.float32(127.0), np.float32(2.0 ** -24)).astype(np.float32)
    codes = np.clip(np.rint(qr / scale[:, :, None]), -127, 127).astype(np.int8)
    assert np.array_equal(q8.cpu().numpy(), codes) and np.array_equal(qs.cpu().numpy(), scale)
    max_splits = (tokens + split - 1) // split + 1
    pm = torch.zeros((rows, max_splits, qh), dtype=torch.float32, device="cuda")
    ps = torch.zeros_like(pm)
    po = torch.zeros((rows, max_splits, qh, hd), dtype=torch.float32, device="cuda")
    out = torch.empty((rows, qh * hd), dtype=torch.float32, device="cuda")
    _ok(R, R.qr_attention_q4h(dqg.data_ptr(), q8.data_ptr(), qs.data_ptr(), dtable.data_ptr(), out.data_ptr(),
                              pm.data_ptr(), ps.data_ptr(), po.data_ptr(), ctx, rows, 0, pt, qh, kv, hd, split,
                              max_splits, 1))
    ref = out.cpu().numpy()
    assert np.isfinite(ref).all()
    assert np.abs(ref - want).max() < 2e-4, np.abs(ref - want).max()
    # this library at the same geometry (head_dim 256 runs on its order-independent kernel)
    dq = dev(q); dpos = dev(np.array([ctx - 1], np.uint32))
    ws = torch.empty(L.qllm_k_attention_workspace_bytes(rows, qh, hd, max_splits), dtype=torch.uint8, device="cuda")
    _okl(L, L.qllm_k_attention(ob.KV_Q4H, dtable.data_ptr(), 0, pt, dq.data_ptr(), qh * hd, rows, dpos.data_ptr(), 0,
                               qh, kv, hd, split, max_splits, 1, ws.data_ptr(), out.data_ptr(), 0, None)); _sync()
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() < 2e-4, np.abs(got - ref).max()


@pytest.mark.parametrize("ctx,rows,qh,kv,hd", [(4, 5, 10, 2, 128), (300, 5, 10, 2, 128), (700, 4, 16, 2, 128)])
def test_q8_attention(R, L, ctx, rows, qh, kv, hd):
    """The draft layer's Q8 cache: the reference's BF16 tensor-core microbatch kernel against the
    oracle and against this library's tensor-core kernel, the reference's own gate (2e-3)."""
    import torch
    pt, split = 64, 128
    rng = np.random.default_rng(ctx * 17 + rows)
    tokens = ctx + rows - 1
    count = (tokens + pt - 1) // pt
    layer_bytes = ob.lib().qo_kv_layer_bytes(ob.KV_Q8, pt, kv, hd)
    host_pages, host_table = _host_pages(layer_bytes, 1, count)
    k = rng.normal(0, 1.0, (tokens, kv * hd)).astype(np.float32)
    v = rng.normal(0, 1.0, (tokens, kv * hd)).astype(np.float32)
    ob.lib().qo_kv_store(ob.KV_Q8, host_table, 0, pt, kv, hd, ob._ptr(k), ob._ptr(v), tokens, kv * hd, 0)
    q = rng.normal(0, 1.0, (rows, qh * hd)).astype(np.float32)
    want = np.empty((rows, qh * hd), np.float32)
    ob.lib().qo_attention(ob.KV_Q8, host_table, 0, pt, ob._ptr(q), qh * hd, rows, ctx, qh, kv, hd, split, 1, ob._ptr(want))
    dpages = [dev(p) for p in host_pages]
    dtable = dev(np.array([p.data_ptr() for p in dpages], np.uint64))
    dqg = dev(_gated(q, qh, hd))
    max_splits = (tokens + split - 1) // split + 1
    pm = torch.zeros((rows, max_splits, qh), dtype=torch.float32, device="cuda")
    ps = torch.zeros_like(pm)
    po = torch.zeros((rows, max_splits, qh, hd), dtype=torch.float32, device="cuda")
    out = torch.empty((rows, qh * hd), dtype=torch.float32, device="cuda")
    _ok(R, R.qr_attention_q8(dqg.data_ptr(), dtable.data_ptr(), out.data_ptr(), pm.data_ptr(), ps.data_ptr(),
                             po.data_ptr(), ctx, rows, 0, pt, qh, kv, hd, split, max_splits, 1))
    ref = out.cpu().numpy()
    assert np.isfinite(ref).all()
    assert np.abs(ref - want).max() < 2e-3, np.abs(ref - want).max()
    dq = dev(q); dpos = dev(np.array([ctx - 1], np.uint32))
    ws = torch.empty(L.qllm_k_attention_workspace_bytes(rows, qh, hd, max_splits), dtype=torch.uint8, device="cuda")
    for impl in (0, 1):
        _okl(L, L.qllm_k_attention(ob.KV_Q8, dtable.data_ptr(), 0, pt, dq.data_ptr(), qh * hd, rows, dpos.data_ptr(), 0,
                                   qh, kv, hd, split, max_splits, 1, ws.data_ptr(), out.data_ptr(), impl, None)); _sync()
        got = out.cpu().numpy()
        assert np.abs(got - ref).max() < 2e-3, (impl, np.abs(got - ref).max())


def test_argmax_and_topk(R, L):
    """Greedy token and sorted top-k of vocabulary-wide rows with many exact ties: the reference
    kernels, the oracle and this library return the same indices and values."""
    import torch
    rng = np.random.default_rng(5)
    rows, count = 3, 151936
    v = torch.from_numpy(rng.normal(0, 1.5, (rows, count)).astype(np.float32)).to(torch.bfloat16).float().numpy()
    v[0, 100] = v[0, 90000] = v[0].max() + 1       # tie for the maximum: the lower id wins
    dv = dev(v)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    _ok(R, R.qr_argmax_batch(dv.data_ptr(), count, rows, out.data_ptr()))
    ref_arg = out.cpu().numpy().astype(np.uint32)
    want = [ob.lib().qo_argmax(ob._ptr(np.ascontiguousarray(v[r])), count) for r in range(rows)]
    assert list(ref_arg) == want and want[0] == 100
    _okl(L, L.qllm_k_argmax(dv.data_ptr(), rows, count, count, out.data_ptr(), None)); _sync()
    assert list(out.cpu().numpy().astype(np.uint32)) == want
    items = R.qr_topk_workspace_items(count)
    wv = torch.empty(items, dtype=torch.float32, device="cuda"); wi = torch.empty(items, dtype=torch.int32, device="cuda")
    v[1, 5] = np.nan                               # excluded from the top-k
    dv = dev(v)
    for k in (1, 20, 64):
        tv = torch.empty(k, dtype=torch.float32, device="cuda"); ti = torch.empty(k, dtype=torch.int32, device="cuda")
        ws = torch.empty(L.qllm_k_topk_workspace_bytes(rows, count, k), dtype=torch.uint8, device="cuda")
        ov = torch.empty((rows, k), dtype=torch.float32, device="cuda"); oi = torch.empty((rows, k), dtype=torch.int32, device="cuda")
        _okl(L, L.qllm_k_topk(dv.data_ptr(), rows, count, count, k, ov.data_ptr(), oi.data_ptr(), ws.data_ptr(), None)); _sync()
        for r in range(rows):
            _ok(R, R.qr_topk(dv[r].data_ptr(), count, k, tv.data_ptr(), ti.data_ptr(), wv.data_ptr(), items * 4,
                             wi.data_ptr(), items * 4))
            cv = np.empty(k, np.float32); ci = np.empty(k, np.uint32)
            ob.lib().qo_topk(ob._ptr(np.ascontiguousarray(v[r])), count, k, ob._ptr(cv), ob._ptr(ci))
            assert np.array_equal(ti.cpu().numpy().astype(np.uint32), ci) and np.array_equal(tv.cpu().numpy(), cv)
            assert np.array_equal(oi[r].cpu().numpy().astype(np.uint32), ci) and np.array_equal(ov[r].cpu().numpy(), cv)


def test_reference_gemv_time_on_this_gpu(R, L, capsys):
    """Same-GPU baseline, reported not asserted: the reference's NVFP4 GEMV kernel and this library's
    tensor-core GEMV on the gate/up shape of the 27B model (34816 x 5120, 5 rows)."""
    import torch
    from quantum_llm_b200 import lib
    rows, cols, batch = 34816, 5120, 5
    gen = torch.Generator(device="cuda"); gen.manual_seed(1)
    codes = torch.randint(0, 256, (rows, cols // 2), dtype=torch.uint8, device="cuda", generator=gen)
    scales = torch.randint(0x30, 0x40, (rows, cols // 16), dtype=torch.uint8, device="cuda", generator=gen)
    x = torch.randn((batch, cols), dtype=torch.float32, device="cuda", generator=gen)
    y = torch.empty((batch, rows), dtype=torch.float32, device="cuda"); qdq = torch.empty_like(x)
    y2 = torch.empty_like(y)
    cm = lib.Matrix(codes.data_ptr(), scales.data_ptr(), 1e-3, 336.0, rows, cols)
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(batch, rows, cols)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    prepared = C.c_void_p()
    _okl(L, L.qllm_k_matrix_prepare(C.byref(cm), None, C.byref(prepared)))

    def timed(fn, n=5):
        fn(); _sync()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record(); _sync()
        return a.elapsed_time(b) / n * 1e3

    t_ref = timed(lambda: _ok(R, R.qr_nvfp4_gemv(codes.data_ptr(), scales.data_ptr(), 1e-3, 336.0, rows, cols,
                                                 x.data_ptr(), y.data_ptr(), qdq.data_ptr(), batch)))
    t_own = timed(lambda: _okl(L, L.qllm_k_nvfp4_gemv_prepared(prepared, x.data_ptr(), y2.data_ptr(), batch, ws.data_ptr(),
                                                             ws_bytes, 1, None)))
    L.qllm_k_matrix_release(prepared)
    a, b = y.cpu().numpy(), y2.cpu().numpy()
    close = (bf16_ulps(a, b) <= 1) | (np.abs(a - b) <= 1e-3 * np.sqrt((a ** 2).mean()))
    assert close.all()
    # How often does a kernel that sums in FP32 land one BF16 step away from the exactly rounded
    # result?  The oracle (exact block terms, double sums, one rounding) is the yardstick; the
    # reference's own kernel sums FP32 products in lane order, this library's tensor-core kernel in
    # the tensor core's FP32 accumulator, its CUDA-core kernel exactly.  A W4A4 decoder amplifies
    # every such step (the next activation quantiser may flip an E2M1 code), so whole-step logits of
    # ANY FP32-accumulating kernel -- the reference's included -- differ from the oracle's by
    # percents of their RMS; that is the reference's own reproducibility, not a tolerance this
    # library may be held below.
    host_codes, host_scales = codes.cpu().numpy(), scales.cpu().numpy()   # kept alive: the oracle matrix holds pointers
    om = ob.matrix(host_codes, host_scales, 1e-3, 336.0)
    want = ob.gemv(om, x.cpu().numpy())
    y0 = torch.empty_like(y)
    _okl(L, L.qllm_k_nvfp4_gemv(C.byref(cm), 0, rows, x.data_ptr(), y0.data_ptr(), batch, ws.data_ptr(), ws_bytes, 0, None)); _sync()
    flips_ref, flips_tc, flips_exact = (float((t != want).mean()) for t in (a, b, y0.cpu().numpy()))
    assert flips_exact == 0.0
    assert flips_tc <= max(2.0 * flips_ref, 2e-3), (flips_tc, flips_ref)
    bytes_ = 0.5625 * rows * cols
    with capsys.disabled():
        print(f"\n[reference kernel on this GPU] nvfp4 gemv 34816x5120 M=5: reference {t_ref:.1f} us "
              f"({bytes_ / t_ref / 1e3:.0f} GB/s), this library {t_own:.1f} us ({bytes_ / t_own / 1e3:.0f} GB/s, "
              f"quantiser + GEMV + split sum); outputs one BF16 step away from the exactly rounded result: "
              f"reference kernel {flips_ref:.2e}, tensor-core kernel {flips_tc:.2e}, CUDA-core kernel {flips_exact:.1e}")
