"""CPU checks of the whole-step oracle: properties that must hold whatever the
weights are (the reference holds no end-to-end vector for its MTP loop)."""
import numpy as np

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
