"""Sampling presence penalty on the GPU against the CPU oracle, through the C ABI.

The oracle's penalty is checked on the CPU (tests/test_oracle_step.py: the speculative stream with
a penalty equals token-by-token penalised decoding).  Here the CUDA provider has to reproduce the
oracle's penalised runs on the exact path: same first token, drafts, emitted tokens and -- because
both sides penalise the logits rows in place, as the reference does -- the same bits in every
verify row, for a positive and a negative penalty, greedy and sampled, and in the scalar decode
fallback.

These tests have not been run on a GPU yet (no device was available when they were written); they
are marked xfail(strict=False) for that reason only -- a pass is reported as XPASS -- and sit in a
file collected late so that nothing else depends on them.
"""
import numpy as np
import pytest

from tests import synth
from tests.gpu_util import provider_from_synth, request_pair

pytestmark = [pytest.mark.gpu,
              pytest.mark.xfail(strict=False, reason="not yet run on a GPU")]

CFG = dict(synth.TINY)
PROMPT = 40


def _gpu(model, prq, prompt, steps):
    p = provider_from_synth(model)
    p.set_gemv_impl(0)
    p.set_attention_impl(0)
    p.set_graph_mode(True)
    st = p.create_request_state()
    first = p.prefill(st, prq, prompt, chunk_rows=5)
    run = dict(first=first, drafts=[int(t) for t in p.read_drafts(st)], steps=[])
    position, token = len(prompt), first
    for _ in range(steps):
        r = p.execute_exact_decode(st, prq, token, position, CFG["max_context"])
        run["steps"].append(dict(emitted=list(r.emitted_tokens), next=r.next_token, logits=p.read_logits(5).copy(),
                                 drafts=[int(t) for t in p.read_drafts(st)]))
        position += r.positions_advanced
        token = r.next_token
    return run


def _cpu(model, orq, prompt, steps):
    o = model.oracle_session()
    first = o.prefill(prompt, 5, orq)
    run = dict(first=first, drafts=[int(t) for t in o.drafts()], steps=[])
    position, token = len(prompt), first
    for _ in range(steps):
        r = o.execute_exact_decode(orq, token, position)
        run["steps"].append(dict(emitted=[int(t) for t in r.emitted[:r.emitted_count]], next=int(r.next_token),
                                 logits=o.last_logits(5).copy(), drafts=[int(t) for t in o.drafts()]))
        position += r.positions_advanced
        token = r.next_token
    return run


@pytest.mark.parametrize("temperature_ppm", [0, 800000], ids=["greedy", "sampled"])
@pytest.mark.parametrize("penalty_ppm", [1500000, -1000000])
def test_penalised_speculative_steps_equal_the_oracle(penalty_ppm, temperature_ppm):
    model = synth.SynthModel(CFG, seed=4)
    prompt = synth.prompt(CFG["vocab"], PROMPT, 4)
    prq, orq = request_pair(seed=11, temperature_ppm=temperature_ppm, context_limit=CFG["max_context"],
                            presence_penalty_ppm=penalty_ppm, first_output_position=PROMPT - 1)
    gpu, cpu = _gpu(model, prq, prompt, 10), _cpu(model, orq, prompt, 10)
    assert gpu["first"] == cpu["first"] and gpu["drafts"] == cpu["drafts"]
    for i, (g, c) in enumerate(zip(gpu["steps"], cpu["steps"])):
        assert g["emitted"] == c["emitted"] and g["next"] == c["next"] and g["drafts"] == c["drafts"], f"step {i}"
        assert np.array_equal(g["logits"][:1], c["logits"][:1]), f"penalised logits of step {i}"
    # the penalty does something: the neutral run of the same model parts from it
    nrq, _ = request_pair(seed=11, temperature_ppm=temperature_ppm, context_limit=CFG["max_context"])
    neutral = _gpu(model, nrq, prompt, 10)
    assert [s["emitted"] for s in neutral["steps"]] != [s["emitted"] for s in gpu["steps"]]


def test_every_verify_row_is_penalised_like_the_oracles():
    model = synth.SynthModel(CFG, seed=5)
    prompt = synth.prompt(CFG["vocab"], PROMPT, 5)
    prq, orq = request_pair(context_limit=CFG["max_context"], presence_penalty_ppm=2000000,
                            first_output_position=PROMPT - 1)
    gpu, cpu = _gpu(model, prq, prompt, 6), _cpu(model, orq, prompt, 6)
    for i, (g, c) in enumerate(zip(gpu["steps"], cpu["steps"])):
        assert np.array_equal(g["logits"], c["logits"]), f"all five penalised rows of step {i}"


def test_penalised_scalar_decode_equals_the_oracle():
    from oracle import binding as ob
    model = synth.SynthModel(CFG, seed=6)
    prompt = synth.prompt(CFG["vocab"], PROMPT, 6)
    prq, orq = request_pair(context_limit=CFG["max_context"], presence_penalty_ppm=1200000,
                            first_output_position=PROMPT - 1)
    p = provider_from_synth(model)
    p.set_gemv_impl(0)
    p.set_attention_impl(0)
    st = p.create_request_state()
    p.prefill(st, prq, prompt[:-1], chunk_rows=5)       # the head of this call is before the first output position
    o = model.oracle_session()
    o.prefill(prompt[:-1], 5, orq)
    token = int(prompt[-1])
    for position in range(PROMPT - 1, PROMPT + 8):
        nxt = p.scalar_decode(st, prq, token, position)
        want = o.prefill_at(np.array([token], np.uint32), position, 5, orq)
        assert nxt == want, f"position {position}"
        assert np.array_equal(p.read_logits(1)[0], o.last_logits(1)[0]), f"penalised logits at {position}"
        token = nxt


def test_an_invalid_presence_penalty_is_refused():
    from quantum_llm_b200 import QllmError
    from quantum_llm_b200.provider import RequestParameters
    model = synth.SynthModel(CFG, seed=6)
    p = provider_from_synth(model)
    st = p.create_request_state()
    bad = RequestParameters(1, 0, 950000, 20, 0, CFG["max_context"], 4_000_001)
    p.prefill_chunk(st, synth.prompt(CFG["vocab"], 5, 0), 0)
    with pytest.raises(QllmError):
        p.first_token(st, bad, 4)
