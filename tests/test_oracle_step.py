"""CPU checks of the whole-step oracle: properties that must hold whatever the
weights are (the reference holds no end-to-end vector for its MTP loop)."""
import numpy as np
import pytest

from oracle import binding as ob
from tests import synth


def decode(session, rq, first, position, count):
    out, tok, steps, accepted = [], first, 0, 0
    while len(out) < count:
        r = session.execute_exact_decode(rq, tok, position)
        assert r.emitted[0] == tok and r.positions_advanced == r.emitted_count
        out += list(r.emitted[:r.emitted_count])
        position += r.positions_advanced
        tok = r.next_token
        steps += 1
        accepted += r.emitted_count - 1
        assert session.mtp_length == position
    return out[:count], steps, accepted


def echo_model(seed=0):
    """A model whose drafts can be right: attention and FFN outputs are scaled to almost
    nothing, so the target's next token is a function of the current token alone, and the
    fusion matrix passes the normalised embedding through, so the draft block sees the same
    input.  Used to exercise acceptance lengths above zero."""
    cfg = dict(synth.TINY)
    m = synth.SynthModel(cfg, seed)
    H = cfg["hidden"]
    for b in m.layers + [m.mtp_block]:
        for name in ("o", "down"):
            w = b.master[name] * 1e-4
            setattr(b, name, synth.SynthMatrix(w))
    fusion = np.zeros((H, 2 * H), np.float32)
    fusion[np.arange(H), np.arange(H)] = 1.0
    m.mtp_fusion = synth.SynthMatrix(fusion)
    return m


def test_greedy_output_does_not_depend_on_the_draft_model():
    # speculative greedy decoding must equal the target's own greedy continuation, so two
    # different draft blocks give the same tokens
    prompt = synth.prompt(4096, 48, 0)
    rq = synth.request(context_limit=256)
    outs = []
    for noise_seed in (0, 1):
        m = synth.SynthModel(synth.TINY, seed=0)
        if noise_seed:
            rng = np.random.default_rng(99)
            m.mtp_fusion = synth.SynthMatrix(rng.normal(0, 0.02, (256, 512)).astype(np.float32))
        s = m.oracle_session()
        first = s.prefill(prompt, 5, rq)
        outs.append(decode(s, rq, first, len(prompt), 24)[0])
    assert outs[0] == outs[1]


def test_prefill_chunking_does_not_change_the_first_token_or_drafts():
    m = synth.SynthModel(synth.TINY, seed=3)
    prompt = synth.prompt(4096, 33, 1)
    rq = synth.request(context_limit=256)
    seen = []
    for chunk in (1, 5, 8):
        s = m.oracle_session()
        first = s.prefill(prompt, chunk, rq)
        seen.append((first, tuple(s.drafts())))
    assert len(set(seen)) == 1 and len(seen[0][1]) == 4


def test_echo_model_accepts_drafts_and_counts_positions():
    m = echo_model()
    prompt = synth.prompt(4096, 40, 2)
    for temperature in (0, 700000):
        rq = synth.request(temperature_ppm=temperature, context_limit=256)
        s = m.oracle_session()
        first = s.prefill(prompt, 5, rq)
        out, steps, accepted = decode(s, rq, first, len(prompt), 40)
        assert steps < 40 and accepted > 0
        if temperature == 0:
            assert accepted / steps > 1.0


def test_sampled_run_is_reproducible_and_seed_dependent():
    m = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 32, 0)
    runs = []
    for seed in (7, 7, 8):
        rq = synth.request(seed=seed, temperature_ppm=700000, context_limit=256)
        s = m.oracle_session()
        first = s.prefill(prompt, 5, rq)
        runs.append([first] + decode(s, rq, first, len(prompt), 16)[0])
    assert runs[0] == runs[1] and runs[0] != runs[2]


def test_invocation_stream_is_validated():
    import pytest
    m = synth.SynthModel(synth.TINY, seed=0)
    rq = synth.request(context_limit=256)
    s = m.oracle_session()
    first = s.prefill(synth.prompt(4096, 16, 0), 5, rq)
    with pytest.raises(RuntimeError):
        s.execute_exact_decode(rq, first + 1, 16)       # wrong guaranteed token
    with pytest.raises(RuntimeError):
        s.execute_exact_decode(rq, first, 17)           # position != draft cache length
    s.execute_exact_decode(rq, first, 16)


def _decode(o, rq, prompt, generate):
    first = o.prefill(prompt, 5, rq)
    stream, pos, tok = [first], len(prompt), first
    while len(stream) < generate + 1:
        r = o.execute_exact_decode(rq, tok, pos)
        stream += list(r.emitted[1:r.emitted_count]) + [r.next_token]
        pos += r.positions_advanced
        tok = r.next_token
    return [int(t) for t in stream[:generate + 1]]


@pytest.mark.parametrize("penalty_ppm", [1500000, -1000000])
def test_presence_penalty_in_the_speculative_step_equals_plain_penalised_decoding(penalty_ppm):
    """Greedy decoding with a presence penalty (dense_fp4_provider.cpp:8336-8347, :11182-11202,
    :11261-11270): a verify row must be judged against the tokens emitted so far PLUS the proposals
    before it, and accepted proposals must be committed -- then the speculative stream equals
    token-by-token decoding with the same penalty, computed here from the target's plain logits and
    a mask kept in the test."""
    cfg = synth.TINY
    model = synth.SynthModel(cfg, seed=4)
    prompt = synth.prompt(cfg["vocab"], 48, 4)
    rq = synth.request(context_limit=cfg["max_context"], presence_penalty_ppm=penalty_ppm,
                       first_output_position=len(prompt) - 1)
    got = _decode(model.oracle_session(), rq, prompt, 40)
    # plain decoding: one target row at a time, the mask and the penalty applied by the test
    plain = synth.request(context_limit=cfg["max_context"])
    o = model.oracle_session()
    o.prefill(prompt[:-1], 5, plain)
    penalty = np.float32(penalty_ppm / 1e6)
    mask = np.zeros(cfg["vocab"], bool)
    want, token = [], int(prompt[-1])
    for position in range(len(prompt) - 1, len(prompt) + 40):
        o.prefill_at(np.array([token], np.uint32), position, 5, plain)
        row = o.last_logits(1)[0].copy()
        row[mask] -= penalty
        token = int(ob.lib().qo_argmax(ob._ptr(row), row.size))
        mask[token] = True
        want.append(token)
    assert got == want
    if penalty_ppm > 0:
        free = _decode(model.oracle_session(), synth.request(context_limit=cfg["max_context"]), prompt, 40)
        assert got != free and len(set(got)) > len(set(free))     # the penalty does move the stream


def test_presence_penalty_is_validated_and_neutral_by_default():
    cfg = synth.TINY
    model = synth.SynthModel(cfg, seed=4)
    prompt = synth.prompt(cfg["vocab"], 32, 1)
    a = _decode(model.oracle_session(), synth.request(context_limit=cfg["max_context"]), prompt, 16)
    b = _decode(model.oracle_session(), synth.request(context_limit=cfg["max_context"], presence_penalty_ppm=0,
                                                      first_output_position=7), prompt, 16)
    assert a == b
    with pytest.raises(RuntimeError):
        model.oracle_session().prefill(prompt, 5, ob.Request(1, 0, 950000, 20, 0, cfg["max_context"], 4000001, 0))


def test_sampled_presence_penalty_keeps_acceptance_consistent():
    """Sampled mode with a penalty: reproducible, seed dependent, and the acceptance counters stay
    within the draft depth (the proposal mask of a rollout feeds the draft distributions that the
    next verify pass divides by)."""
    cfg = synth.TINY
    model = synth.SynthModel(cfg, seed=4)
    prompt = synth.prompt(cfg["vocab"], 32, 2)
    rq = synth.request(seed=5, temperature_ppm=800000, context_limit=cfg["max_context"], presence_penalty_ppm=700000,
                       first_output_position=len(prompt) - 1)
    a = _decode(model.oracle_session(), rq, prompt, 32)
    b = _decode(model.oracle_session(), rq, prompt, 32)
    c = _decode(model.oracle_session(), synth.request(seed=6, temperature_ppm=800000, context_limit=cfg["max_context"],
                                                      presence_penalty_ppm=700000,
                                                      first_output_position=len(prompt) - 1), prompt, 32)
    assert a == b and a != c
