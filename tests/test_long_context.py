"""Parity at the benchmark's own context length: 32768 cached tokens, Q4H target cache, Q8 draft
cache, head_dim 128 -- the size at which bench.py times the step.  A prompt pass of that length
through the CPU oracle would take an hour, so both sides start from the same seeded synthetic
cache records (qllm_provider_fill_synthetic_kv and its host twin qo_fill_synthetic_kv write
identical bytes, checked here page by page), run the last 40 prompt tokens for real, and decode.

* exact path: tokens, drafts and every verify row's logits identical to the oracle's;
* tensor-core attention + tcgen05 GEMV (the benchmarked kernels, 64 splits of 512 tokens per kv head):
  every row fed by agreed tokens within 2e-2 max-abs / 1e-3 relative RMS of the oracle's.
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
    assert all(d_abs <= 2e-2 and d_rms <= 1e-3 for _, _, d_abs, d_rms in report), report
