"""The scalar decode fallback and session retention on the GPU, through the C ABI.

* qllm_k_sample_token -- the full-vocabulary sampler (top_k 0 or above 64): the committed vectors
  made with the reference's own sampler functions (tests/golden/sampler_cases.json), and seeded
  rows of the benchmark's vocabulary width against the CPU oracle, bit for bit (ties, infinities,
  NaNs, signed zeros, min-p and top-p cuts, top_k between 65 and the whole row);
* qllm_provider_scalar_decode -- a request the speculative path refuses (top_k 0) decodes token by
  token, every token equal to the oracle's sampler over the oracle's logits;
* qllm_provider_checkpoint_request_state / _rewind_request_state -- speculative steps, a rewind to
  the checkpoint, a scalar step that primes the drafts again, and the continuation equals the
  stream decoded without the detour; invalid checkpoints and rewinds are refused.
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

from oracle import binding as ob
from tests import synth
from tests.gpu_util import dev, provider_from_synth, request_pair

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gpu_sample(L, logits, seed, t_ppm, p_ppm, top_k, m_ppm, position):
    import torch
    d = dev(np.ascontiguousarray(logits, np.float32))
    ws = torch.empty(L.qllm_k_sample_token_workspace_bytes(d.numel()), dtype=torch.uint8, device="cuda")
    out = torch.zeros(2, dtype=torch.int32, device="cuda")      # [status, token]
    rc = L.qllm_k_sample_token(d.data_ptr(), d.numel(), seed, t_ppm, p_ppm, top_k, m_ppm, position, ws.data_ptr(),
                               out.data_ptr(), out.data_ptr() + 4, None)
    assert rc == 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    status, token = (int(v) for v in out.cpu().numpy().view(np.uint32))
    return None if status else token


@pytest.fixture(scope="module")
def L():
    from quantum_llm_b200 import lib
    return lib.load()


def test_full_vocabulary_sampler_matches_the_reference_vectors(L):
    cases = json.load(open(os.path.join(GOLDEN, "sampler_cases.json")))["sample_token"]
    for i, case in enumerate(cases):
        logits = np.array(case["logits_f32_bits"], np.uint32).view(np.float32)
        got = _gpu_sample(L, logits, case["seed"], case["temperature_ppm"], case["top_p_ppm"], case["top_k"],
                          case["min_p_ppm"], case["position"])
        assert got == case["token"], f"case {i}"


@pytest.mark.parametrize("vocab", [151936, 4099, 2048])
def test_full_vocabulary_sampler_equals_the_oracle_at_full_width(L, vocab):
    rng = np.random.default_rng(vocab)
    hits = set()
    for case in range(12):
        logits = rng.normal(0, 3.0, vocab).astype(np.float32)
        logits[rng.integers(0, vocab, 40)] = logits[int(rng.integers(0, vocab))]      # ties, also for the maximum
        if case % 3 == 0:
            top = int(np.argmax(logits))
            logits[rng.integers(0, vocab, 3)] = logits[top]
        if case % 4 == 1:
            logits[rng.integers(0, vocab, 50)] = -np.inf
        if case % 4 == 2:
            logits[rng.integers(0, vocab, 5)] = np.nan
        if case % 4 == 3:
            logits[rng.integers(0, vocab, 4)] = [0.0, -0.0, 0.0, -0.0]
        top_k = [0, 65, 1000, vocab, 0, 300][case % 6]
        t_ppm = [1000000, 2000000, 700000, 1500000][case % 4]
        p_ppm = [1000000, 950000, 999999][case % 3]
        m_ppm = [0, 1000, 0, 100000][case % 4]
        seed, position = int(rng.integers(0, 2**63)), int(rng.integers(0, 2**24))
        want = ob.sample_token(logits, ob.Request(seed, t_ppm, p_ppm, top_k, m_ppm, 0, 2000000), position)
        got = _gpu_sample(L, logits, seed, t_ppm, p_ppm, top_k, m_ppm, position)
        assert want is not None and got == want, (case, top_k, t_ppm, p_ppm, m_ppm)
        hits.add(want)
    assert len(hits) > 3     # the cases do not all fall on one token


def test_full_vocabulary_sampler_reports_rows_without_mass(L):
    rq = ob.Request(1, 700000, 900000, 0, 0, 0, 2000000)
    row = np.full(5000, -np.inf, np.float32)
    assert ob.sample_token(row, rq, 3) is None
    assert _gpu_sample(L, row, 1, 700000, 900000, 0, 0, 3) is None
    row[:] = np.nan
    assert ob.sample_token(row, rq, 3) is None
    assert _gpu_sample(L, row, 1, 700000, 900000, 0, 0, 3) is None


CFG = dict(synth.TINY)


def test_scalar_decode_with_unbounded_top_k_equals_the_oracle():
    from quantum_llm_b200 import QllmError
    model = synth.SynthModel(CFG, seed=2)
    prompt = synth.prompt(CFG["vocab"], 24, 5)
    prq, orq = request_pair(seed=99, temperature_ppm=900000, top_p_ppm=1000000, top_k=0, min_p_ppm=0,
                            context_limit=CFG["max_context"])
    greedy_p, greedy_o = request_pair(context_limit=CFG["max_context"])
    p = provider_from_synth(model)
    p.set_gemv_impl(0)
    p.set_attention_impl(0)
    st = p.create_request_state()
    # prompt minus its last token through chunks; the speculative path refuses this request
    p.prefill(st, greedy_p, prompt[:-1], chunk_rows=5)
    with pytest.raises(QllmError):
        p.execute_exact_decode(st, prq, 0, len(prompt) - 1, CFG["max_context"])
    o = model.oracle_session()
    o.prefill(prompt[:-1], 5, greedy_o)
    token, tokens = int(prompt[-1]), []
    for position in range(len(prompt) - 1, len(prompt) + 7):
        nxt = p.scalar_decode(st, prq, token, position)
        # the oracle's logits for the same row, then the oracle's sampler
        o.prefill_at(np.array([token], np.uint32), position, 5, greedy_o)
        want = ob.sample_token(o.last_logits(1)[0], orq, position)
        assert np.array_equal(p.read_logits(1)[0], o.last_logits(1)[0]), f"logits at {position}"
        assert nxt == want, f"position {position}"
        tokens.append(nxt)
        token = nxt
    assert len(set(tokens)) > 1
    # top_k above 64 takes the same route
    prq2, orq2 = request_pair(seed=5, temperature_ppm=1200000, top_p_ppm=900000, top_k=200, min_p_ppm=1000,
                              context_limit=CFG["max_context"])
    position = len(prompt) + 7
    nxt = p.scalar_decode(st, prq2, token, position)
    o.prefill_at(np.array([token], np.uint32), position, 5, greedy_o)
    assert nxt == ob.sample_token(o.last_logits(1)[0], orq2, position)


def _steps(p, st, prq, token, position, count, limit):
    stream = []
    for _ in range(count):
        r = p.execute_exact_decode(st, prq, token, position, limit)
        stream += list(r.emitted_tokens)
        position += r.positions_advanced
        token = r.next_token
    return stream, token, position


def test_rewind_to_a_checkpoint_and_decode_again():
    from quantum_llm_b200 import QllmError
    model = synth.SynthModel(CFG, seed=3)
    prompt = synth.prompt(CFG["vocab"], 20, 9)
    limit = CFG["max_context"]
    prq, _ = request_pair(context_limit=limit)
    p = provider_from_synth(model)
    p.set_gemv_impl(0)
    p.set_attention_impl(0)
    st = p.create_request_state()
    with pytest.raises(QllmError):
        p.rewind_request_state(st, 5)                 # nothing checkpointed
    first = p.prefill(st, prq, prompt, chunk_rows=8)
    n = len(prompt)
    with pytest.raises(QllmError):
        p.checkpoint_request_state(st, n - 1)         # not the end of the cached stream
    with pytest.raises(QllmError):
        p.checkpoint_request_state(st, 0)
    p.checkpoint_request_state(st, n)
    want, _, _ = _steps(p, st, prq, first, n, 6, limit)
    assert want[0] == first
    with pytest.raises(QllmError):
        p.rewind_request_state(st, n + 1)             # only the checkpointed position
    p.checkpoint_request_state(st, n)                 # the state has moved on: the old checkpoint is confirmed
    p.rewind_request_state(st, n)
    with pytest.raises(QllmError):                    # the drafts are gone with the rewind
        p.execute_exact_decode(st, prq, first, n, limit)
    # the runner's fallback step feeds the first generated token again and primes the drafts
    second = p.scalar_decode(st, prq, first, n, produce_final_draft=True)
    assert second == want[1]
    again, _, _ = _steps(p, st, prq, second, n + 1, 5, limit)
    m = min(len(again), len(want) - 1)
    assert m >= 4 and again[:m] == want[1:1 + m]
    # a second rewind to the same checkpoint, this time continued through prompt chunks
    p.rewind_request_state(st, n)
    follow = np.array(want[:3], np.uint32)
    token = p.prefill(st, prq, follow, first_position=n, chunk_rows=8)
    assert token == want[3]
    tail, _, _ = _steps(p, st, prq, token, n + 3, 2, limit)
    assert tail[:2] == want[3:5]
