"""Parity at the benchmark's own context length: 32768 cached tokens, Q4H target cache, Q8 draft
cache, head_dim 128 -- the size at which bench.py times the step.  A prompt pass of that length
through the CPU oracle would take an hour, so both sides start from the same seeded synthetic
cache records (qllm_provider_fill_synthetic_kv and its host twin qo_fill_synthetic_kv write
identical bytes, checked here page by page), run the last 40 prompt tokens for real, and decode.

* exact path: tokens, drafts and every verify row's logits identical to the oracle's;
* the tensor-core attention kernels (INT8 mma.sync and tcgen05) over all 32768 + 4 cached tokens, 64
  splits of 512 tokens per kv head: every output within 1e-3 of the oracle's attention (half the
  reference's own gate for its tensor-core kernel against its host check);
* the benchmarked kernels inside the step: a W4A4 decoder turns a last-place difference into a
  flipped E2M1 code and a flipped code into a moved row (at hidden 512 by tenths), so rows come out
  either bit-identical to the oracle's or visibly apart; asserted: the first token agrees, at least
  a quarter of the compared rows are bit-identical, none is further than 0.5 relative RMS away.
"""
import numpy as np
import pytest

from oracle import binding as ob
from tests import synth
from tests.gpu_util import provider_from_synth, request_pair

pytestmark = pytest.mark.gpu

CONTEXT, REAL, STEPS = 32768, 40, 4
CFG = dict(synth.TINY, hidden=512, q_heads=10, kv_heads=2, head_dim=128, rotary_dim=128, ffn=1024,
           kv_encoding=ob.KV_Q4H, page_tokens=256, split_tokens=512, max_context=CONTEXT + 1024)


def _oracle_run(model, prompt):
    _, orq = request_pair(context_limit=CFG["max_context"])
    o = model.oracle_session()
    o.fill_synthetic_kv(0, CONTEXT - REAL, 99)
    first = o.prefill_at(prompt, CONTEXT - REAL, 5, orq)
    run = dict(first=first, drafts=[int(t) for t in o.drafts()], steps=[], oracle=o)
    position, token = CONTEXT, first
    for _ in range(STEPS):
        r = o.execute_exact_decode(orq, token, position)
        run["steps"].append(dict(emitted=[int(t) for t in r.emitted[:r.emitted_count]], next=int(r.next_token),
                                 logits=o.last_logits(5), drafts=[int(t) for t in o.drafts()]))
        position += r.positions_advanced
        token = r.next_token
    return run


def _gpu_run(model, prompt, gemv_impl, attention_impl, graph):
    prq, _ = request_pair(context_limit=CFG["max_context"])
    p = provider_from_synth(model)
    p.set_gemv_impl(gemv_impl)
    p.set_attention_impl(attention_impl)
    p.set_graph_mode(graph)
    st = p.create_request_state()
    p.fill_synthetic_kv(st, 0, CONTEXT - REAL, seed=99)
    first = p.prefill(st, prq, prompt, first_position=CONTEXT - REAL, chunk_rows=5)
    run = dict(first=first, drafts=[int(t) for t in p.read_drafts(st)], steps=[], provider=p, state=st)
    position, token = CONTEXT, first
    for _ in range(STEPS):
        r = p.execute_exact_decode(st, prq, token, position, CFG["max_context"])
        run["steps"].append(dict(emitted=list(r.emitted_tokens), next=r.next_token, logits=p.read_logits(5).copy(),
                                 drafts=[int(t) for t in p.read_drafts(st)]))
        position += r.positions_advanced
        token = r.next_token
    return run


def test_mma_sync_attention_at_32k_context(case):
    model, prompt, cpu = case
    gpu = _gpu_run(model, prompt, 1, 1, True)
    assert gpu["first"] == cpu["first"]
    a, b = gpu["steps"][0]["logits"][0], cpu["steps"][0]["logits"][0]
    assert np.abs(a - b).max() <= 2e-2


@pytest.fixture(scope="module")
def case():
    model = synth.SynthModel(CFG, seed=5)
    prompt = synth.prompt(CFG["vocab"], REAL, 3)
    return model, prompt, _oracle_run(model, prompt)


def test_synthetic_cache_records_are_the_same_bytes_on_both_sides(case):
    model, prompt, cpu = case
    gpu = _gpu_run(model, prompt, 0, 0, False)
    p, st, o = gpu["provider"], gpu["state"], cpu["oracle"]
    for page in (0, 1, 63, 126):            # synthetic records only (the real prompt starts in page 127)
        want = o.page(page)
        assert np.array_equal(p.read_page(st, page)[:want.size], want), f"cache page {page}"


def test_exact_path_at_32k_context(case):
    model, prompt, cpu = case
    gpu = _gpu_run(model, prompt, 0, 0, True)
    assert gpu["first"] == cpu["first"] and gpu["drafts"] == cpu["drafts"]
    for i, (g, c) in enumerate(zip(gpu["steps"], cpu["steps"])):
        assert g["emitted"] == c["emitted"] and g["next"] == c["next"] and g["drafts"] == c["drafts"], f"step {i}"
        assert np.array_equal(g["logits"], c["logits"]), f"logits of step {i}"


def test_benchmarked_kernels_at_32k_context(case):
    model, prompt, cpu = case
    gpu = _gpu_run(model, prompt, 1, 2, True)
    assert gpu["first"] == cpu["first"]
    inputs_gpu, inputs_cpu = [gpu["first"]] + gpu["drafts"], [cpu["first"]] + cpu["drafts"]
    rows, report = 0, []
    for i, (g, c) in enumerate(zip(gpu["steps"], cpu["steps"])):
        same = 0
        while same < min(len(inputs_gpu), len(inputs_cpu), 5) and inputs_gpu[same] == inputs_cpu[same]:
            same += 1
        for r in range(same):
            a, b = g["logits"][r], c["logits"][r]
            d_abs = float(np.abs(a - b).max())
            d_rms = float(np.sqrt(((a - b).astype(np.float64) ** 2).mean()) / np.sqrt((b.astype(np.float64) ** 2).mean()))
            report.append((i, r, round(d_abs, 5), round(d_rms, 6)))
            rows += 1
        if g["emitted"] != c["emitted"] or g["next"] != c["next"]:
            break
        inputs_gpu, inputs_cpu = [g["next"]] + g["drafts"], [c["next"]] + c["drafts"]
    print("\n32k context, benchmarked kernels vs oracle (step, row, max-abs, rel-rms):", report)
    assert rows >= 5
    assert all(d_rms <= 0.5 for _, _, _, d_rms in report), report
    assert 4 * sum(1 for _, _, d_abs, _ in report if d_abs == 0.0) >= rows, report


@pytest.mark.parametrize("impl", [1, 2], ids=["mma_sync", "tcgen05"])
def test_attention_kernels_over_the_whole_32k_cache(case, impl):
    import torch
    from quantum_llm_b200 import lib
    from tests.gpu_util import dev
    L = lib.load()
    model, prompt, cpu = case
    o = cpu["oracle"]
    qh, kv, hd, pt, split = CFG["q_heads"], CFG["kv_heads"], CFG["head_dim"], CFG["page_tokens"], CFG["split_tokens"]
    rows, ctx = 5, CONTEXT          # row r sees ctx + r cached tokens of layer 0 (synthetic + real + decoded)
    tokens = ctx + rows - 1
    pages = [o.page(i) for i in range((tokens + pt - 1) // pt)]
    import ctypes as C
    table = (C.c_void_p * len(pages))(*[p.ctypes.data for p in pages])
    q = np.random.default_rng(8).normal(0, 1.0, (rows, qh * hd)).astype(np.float32)
    want = np.empty_like(q)
    ob.lib().qo_attention(ob.KV_Q4H, table, 0, pt, ob._ptr(q), qh * hd, rows, ctx, qh, kv, hd, split, 1, ob._ptr(want))
    dpages = [dev(p) for p in pages]
    dtable = dev(np.array([p.data_ptr() for p in dpages], np.uint64))
    dq, dpos = dev(q), dev(np.array([ctx - 1], np.uint32))
    max_splits = (tokens + split - 1) // split + 1
    ws = torch.empty(L.qllm_k_attention_workspace_bytes(rows, qh, hd, max_splits), dtype=torch.uint8, device="cuda")
    out = torch.empty((rows, qh * hd), dtype=torch.float32, device="cuda")
    rc = L.qllm_k_attention(ob.KV_Q4H, dtable.data_ptr(), 0, pt, dq.data_ptr(), qh * hd, rows, dpos.data_ptr(), 0,
                            qh, kv, hd, split, max_splits, 1, ws.data_ptr(), out.data_ptr(), impl, None)
    assert rc >= 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.isfinite(got).all() and np.abs(got - want).max() < 1e-3, np.abs(got - want).max()
