"""Whole-step parity on the tiny configuration (2 layers, hidden 256, 4q/2kv heads,
head_dim 64, FFN 1024, vocab 4096; prompt of 128 seeded ids, 64 generated tokens):
the CUDA provider against the CPU oracle through the provider C ABI."""
import numpy as np
import pytest

from oracle import binding as ob
from tests import synth
from tests.gpu_util import provider_from_synth, request_pair
from tests.test_oracle_step import echo_model

pytestmark = pytest.mark.gpu

LOGIT_MAX_ABS, LOGIT_REL_RMS = 2e-2, 1e-3   # the stated F16-KV parity tolerance


def run_gpu(model, prompt, temperature, generate, graph=False, gemv_impl=0, seed=1234, attention_impl=1):
    """Decode `generate` tokens on the CUDA provider.  Returns the token stream (first token
    onwards), {position: logits row whose inputs are emitted tokens}, and the provider."""
    prq, _ = request_pair(seed=seed, temperature_ppm=temperature, context_limit=model.cfg["max_context"])
    p = provider_from_synth(model)
    p.set_graph_mode(graph)
    p.set_gemv_impl(gemv_impl)
    p.set_attention_impl(attention_impl)
    st = p.create_request_state()
    first = p.prefill(st, prq, prompt, chunk_rows=5)
    drafts = [int(t) for t in p.read_drafts(st)]
    stream, rows, pos, tok, steps, accepted = [first], {}, len(prompt), first, 0, 0
    while len(stream) < generate + 1:
        r = p.execute_exact_decode(st, prq, tok, pos, prq.reserved_context_tokens)
        assert r.emitted_tokens[0] == tok and r.positions_advanced == len(r.emitted_tokens)
        logits = p.read_logits(5)
        for i in range(r.positions_advanced):
            rows[pos + i] = logits[i]
        stream += r.emitted_tokens[1:] + [r.next_token]
        pos += r.positions_advanced
        tok = r.next_token
        steps += 1
        accepted += r.positions_advanced - 1
    return dict(stream=stream, rows=rows, drafts=drafts, steps=steps, accepted=accepted, provider=p, state=st)


def run_cpu(model, prompt, temperature, generate, seed=1234):
    _, orq = request_pair(seed=seed, temperature_ppm=temperature, context_limit=model.cfg["max_context"])
    o = model.oracle_session()
    first = o.prefill(prompt, 5, orq)
    drafts = [int(t) for t in o.drafts()]
    stream, rows, pos, tok, steps, accepted = [first], {}, len(prompt), first, 0, 0
    while len(stream) < generate + 1:
        r = o.execute_exact_decode(orq, tok, pos)
        logits = o.last_logits(5)
        for i in range(r.positions_advanced):
            rows[pos + i] = logits[i]
        stream += list(r.emitted[1:r.emitted_count]) + [r.next_token]
        pos += r.positions_advanced
        tok = r.next_token
        steps += 1
        accepted += r.positions_advanced - 1
    return dict(stream=stream, rows=rows, drafts=drafts, steps=steps, accepted=accepted, oracle=o)


def row_within_tolerance(a, b):
    return (np.abs(a - b).max() <= LOGIT_MAX_ABS and
            np.sqrt(((a - b) ** 2).mean()) / np.sqrt((b ** 2).mean()) <= LOGIT_REL_RMS)


def compare(gpu, cpu, prompt_len):
    """Common prefix of the two token streams, and how many of the logit rows fed by agreed
    tokens are within the stated tolerance.  W4A4 activation quantisation makes the decoder
    discontinuous: a last-place difference that crosses an E2M1/E4M3 rounding threshold moves
    a whole row by ~1e-1, so single rows may fall outside while their neighbours are exact."""
    n = 0
    while n < min(len(gpu["stream"]), len(cpu["stream"])) and gpu["stream"][n] == cpu["stream"][n]:
        n += 1
    shared = [p for p in sorted(gpu["rows"]) if p in cpu["rows"] and p < prompt_len + n]
    good = [p for p in shared if row_within_tolerance(gpu["rows"][p], cpu["rows"][p])]
    exact = [p for p in shared if np.array_equal(gpu["rows"][p], cpu["rows"][p])]
    tie = None
    if n < min(len(gpu["stream"]), len(cpu["stream"])):
        q = prompt_len + n - 1            # the row that chose the first differing token
        if q in cpu["rows"]:
            row = cpu["rows"][q]
            tie = abs(float(row[cpu["stream"][n]]) - float(row[gpu["stream"][n]])) <= 2 * LOGIT_MAX_ABS
    return dict(prefix=n, shared=len(shared), good=len(good), exact=len(exact), tie=tie)


@pytest.mark.parametrize("graph", [False, True])
def test_tiny_greedy_tokens_and_logits(graph):
    model = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 128, 0)
    # exact path (CUDA-core GEMV, order-independent attention): the same bits as the oracle
    gpu = run_gpu(model, prompt, 0, 64, graph=graph, attention_impl=0)
    cpu = run_cpu(model, prompt, 0, 64)
    c = compare(gpu, cpu, len(prompt))
    print("greedy parity", c, "drafts", gpu["drafts"], cpu["drafts"])
    assert gpu["stream"] == cpu["stream"] and gpu["drafts"] == cpu["drafts"]
    assert gpu["steps"] == cpu["steps"] and gpu["accepted"] == cpu["accepted"]
    assert c["shared"] >= 64 and c["exact"] == c["shared"]
    t = gpu["provider"].telemetry(gpu["state"])
    assert t["exact_calls"] == gpu["steps"] and t["kernel_launches"] > 0


def test_tiny_greedy_with_tensor_core_gemv():
    # tcgen05 accumulates in FP32 inside the tensor core: results may land one BF16 step
    # away from the exactly-rounded oracle, and W4A4 re-quantisation can amplify that for a
    # row; most rows stay within the stated tolerance and the stream follows the oracle until
    # a tie or such an event
    model = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 128, 0)
    gpu = run_gpu(model, prompt, 0, 64, graph=True, gemv_impl=1)
    cpu = run_cpu(model, prompt, 0, 64)
    c = compare(gpu, cpu, len(prompt))
    print("tensor-core greedy parity", c)
    assert c["shared"] >= 8 and c["good"] >= 0.8 * c["shared"]


# The tiny geometry with head_dim 128 and a Q4H target cache: the shapes the warp-per-head
# RoPE/KV-store kernel and the tensor-core attention kernels (INT8 MMA over Q4H for the target
# layers, BF16 MMA over Q8 for the draft layer) are written for.
WIDE = dict(synth.TINY, head_dim=128, rotary_dim=128, kv_encoding=ob.KV_Q4H)


@pytest.mark.parametrize("attention_impl", [0, 1, 2])
@pytest.mark.parametrize("kv_encoding", [ob.KV_Q4H, ob.KV_F16])
def test_head_dim_128_caches(kv_encoding, attention_impl):
    model = synth.SynthModel(dict(WIDE, kv_encoding=kv_encoding), seed=2)
    prompt = synth.prompt(4096, 128, 2)
    gpu = run_gpu(model, prompt, 0, 32, graph=True, attention_impl=attention_impl)
    cpu = run_cpu(model, prompt, 0, 32)
    c = compare(gpu, cpu, len(prompt))
    print("head_dim 128 parity, attention_impl", attention_impl, c)
    p, st, o = gpu["provider"], gpu["state"], cpu["oracle"]
    # layer 0 of the prompt pages: RoPE + KV store see identical inputs -> identical bytes
    for page in range(2):
        g, want = p.read_page(st, page), o.page(page)
        lo, hi = o.layer_offset(0), o.layer_offset(1)
        assert np.array_equal(g[lo:hi], want[lo:hi])
    assert gpu["stream"][0] == cpu["stream"][0]
    if attention_impl == 0:
        # scalar attention: order-independent arithmetic end to end -> the same bits
        assert c["prefix"] == 33 and c["exact"] == c["shared"] and gpu["drafts"] == cpu["drafts"]
        for page in range(2):   # every layer, including the Q8 records of the draft layer
            want = o.page(page)
            assert np.array_equal(p.read_page(st, page)[:want.size], want)
    else:
        # tensor-core attention: exp() from ex2.approx, FP32 accumulation -> stated tolerance
        assert c["shared"] >= 8 and c["good"] >= 0.8 * c["shared"]


@pytest.mark.parametrize("kv_encoding", [ob.KV_Q4H, ob.KV_F16])
def test_rope_and_kv_store_fused_into_the_projection_give_the_same_bits(kv_encoding, monkeypatch):
    # tensor-core GEMV, head_dim 128: the CTA that finishes a head of the fused q/k/v projection
    # rotates and stores it itself.  Same arithmetic as the separate kernel -> same tokens, logits
    # and cache bytes (target records and the Q8 records of the draft layer).
    model = synth.SynthModel(dict(WIDE, kv_encoding=kv_encoding), seed=4)
    prompt = synth.prompt(4096, 96, 4)
    runs = []
    for fused in ("1", "0"):
        monkeypatch.setenv("QLLM_ROPE_TAIL", fused)
        runs.append(run_gpu(model, prompt, 0, 24, graph=True, gemv_impl=1, attention_impl=1))
    a, b = runs
    assert a["stream"] == b["stream"] and a["drafts"] == b["drafts"]
    for pos in a["rows"]:
        assert np.array_equal(a["rows"][pos], b["rows"][pos])
    for page in range(2):
        assert np.array_equal(a["provider"].read_page(a["state"], page), b["provider"].read_page(b["state"], page))
    launches = [r["provider"].telemetry(r["state"])["kernel_launches"] for r in runs]
    print("kernel launches with / without the fused tail:", launches)


def test_group_8_tensor_core_attention_inside_a_step():
    # 8 query heads on one kv head (the routed model's grouping: 40 matrix rows per kv head),
    # two layers, so that the second layer's records sit at a non-zero layer offset
    cfg = dict(WIDE, q_heads=8, kv_heads=1, kv_encoding=ob.KV_Q4H)
    model = synth.SynthModel(cfg, seed=6)
    prompt = synth.prompt(4096, 128, 6)
    gpu = run_gpu(model, prompt, 0, 24, graph=True, attention_impl=1)
    cpu = run_cpu(model, prompt, 0, 24)
    c = compare(gpu, cpu, len(prompt))
    print("group 8 parity", c)
    assert gpu["stream"][0] == cpu["stream"][0]
    assert c["shared"] >= 8 and c["good"] >= 0.8 * c["shared"]
    exact = run_gpu(model, prompt, 0, 24, graph=True, attention_impl=0)
    e = compare(exact, cpu, len(prompt))
    assert e["prefix"] == 25 and e["exact"] == e["shared"]


@pytest.mark.parametrize("attention_impl", [0, 1, 2])
def test_one_eighth_shard_geometry(attention_impl):
    # what one rank of an 8-way split of the 27B model sees: 5 query heads on one kv head, an
    # o projection with K = 640 and a down projection whose K is not a multiple of 256, and
    # rows x splits x heads odd (one draft row or five verify rows, three splits, five heads),
    # which once left the float4 section of the split partials on an 8-byte boundary
    cfg = dict(WIDE, q_heads=5, kv_heads=1, ffn=1088, kv_encoding=ob.KV_Q4H)
    model = synth.SynthModel(cfg, seed=8)
    prompt = synth.prompt(4096, 130, 8)
    cpu = run_cpu(model, prompt, 0, 24)
    gemv_impl = 0 if attention_impl == 0 else 1
    gpu = run_gpu(model, prompt, 0, 24, graph=True, gemv_impl=gemv_impl, attention_impl=attention_impl)
    c = compare(gpu, cpu, len(prompt))
    print("one-eighth shard geometry, attention_impl", attention_impl, c)
    assert gpu["stream"][0] == cpu["stream"][0]
    if attention_impl == 0:
        assert c["prefix"] == 25 and c["exact"] == c["shared"]
    else:
        assert c["shared"] >= 4 and c["good"] >= 0.5 * c["shared"]


def test_greedy_stream_equals_plain_target_decoding_on_gpu():
    # property that needs no oracle: speculative greedy output does not depend on the drafts,
    # so a provider with a different draft block emits the same tokens
    prompt = synth.prompt(4096, 64, 3)
    model = synth.SynthModel(synth.TINY, seed=0)
    a = run_gpu(model, prompt, 0, 32)
    rng = np.random.default_rng(5)
    model.mtp_fusion = synth.SynthMatrix(rng.normal(0, 0.02, (256, 512)).astype(np.float32))
    b = run_gpu(model, prompt, 0, 32)
    assert a["stream"][:33] == b["stream"][:33]


def test_tiny_kv_pages_match_the_oracle():
    model = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 128, 0)
    gpu = run_gpu(model, prompt, 0, 4, attention_impl=0)
    cpu = run_cpu(model, prompt, 0, 4)
    p, st, o = gpu["provider"], gpu["state"], cpu["oracle"]
    assert p.page_bytes() >= o.page(0).size
    for layer in range(3):
        assert p.layer_offset(layer) == o.layer_offset(layer)
    # exact path: every record of every layer (F16 target layers, Q8 draft layer) byte for byte --
    # the two prompt pages whole, and of the page the decode steps reach every committed position
    # (slots past the accepted prefix hold speculative rows that are overwritten before any read;
    # the provider also stores the padding rows of its fixed-width draft pass there)
    committed = o.mtp_length
    pt = model.cfg["page_tokens"]
    for page in range(3):
        want = o.page(page)
        got = p.read_page(st, page)[:want.size]
        if (page + 1) * pt <= committed:
            assert np.array_equal(got, want), f"cache page {page}"
            continue
        tokens = committed - page * pt
        assert tokens > 0
        for layer in range(3):   # F16 and Q8 layers are token-major: [K: pt records][V: pt records]
            lo = o.layer_offset(layer)
            hi = o.layer_offset(layer + 1) if layer < 2 else want.size
            half = (hi - lo) // 2
            n = half // pt * tokens
            for base in (lo, lo + half):
                assert np.array_equal(got[base:base + n], want[base:base + n]), f"page {page} layer {layer}"


def test_tiny_sampled_decisions():
    model = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 128, 0)
    gpu = run_gpu(model, prompt, 700000, 48, seed=77, attention_impl=0)
    cpu = run_cpu(model, prompt, 700000, 48, seed=77)
    c = compare(gpu, cpu, len(prompt))
    print("sampled parity", c)
    # exact path: the same accept / reject / residual decisions, the same rows
    assert gpu["stream"] == cpu["stream"] and gpu["accepted"] == cpu["accepted"] and c["exact"] == c["shared"]
    # every emitted token must come from the top-k support of the row that chose it
    for pos, row in gpu["rows"].items():
        tok = gpu["stream"][pos + 1 - len(prompt)]
        assert (row > row[tok]).sum() < 20
    assert c["shared"] >= 16


@pytest.mark.parametrize("temperature", [0, 700000])
def test_echo_model_acceptance_lengths(temperature):
    model = echo_model()
    prompt = synth.prompt(4096, 64, 5)
    gpu = run_gpu(model, prompt, temperature, 48, graph=True, attention_impl=0)
    cpu = run_cpu(model, prompt, temperature, 48)
    c = compare(gpu, cpu, len(prompt))
    print("echo parity", c, "accepted gpu/cpu", gpu["accepted"], cpu["accepted"], "steps", gpu["steps"], cpu["steps"])
    assert cpu["accepted"] > 0 and gpu["accepted"] > 0
    assert gpu["steps"] < 48
    t = gpu["provider"].telemetry(gpu["state"])
    assert t["accepted_drafts"] == gpu["accepted"] and sum(t["accepted_depth_calls"]) == gpu["steps"]
    # exact path: the same acceptance lengths, partial accepts and bonus tokens as the oracle
    assert gpu["stream"] == cpu["stream"] and gpu["steps"] == cpu["steps"] and gpu["accepted"] == cpu["accepted"]
    assert c["exact"] == c["shared"]


def test_multi_step_enqueue_equals_single_steps():
    model = synth.SynthModel(synth.TINY, seed=0)
    prompt = synth.prompt(4096, 64, 4)
    outs = []
    for batched in (False, True):
        prq, _ = request_pair(context_limit=256)
        p = provider_from_synth(model)
        st = p.create_request_state()
        first = p.prefill(st, prq, prompt)
        toks, pos, tok = [], len(prompt), first
        if batched:
            for r in p.execute_exact_decode_steps(st, prq, 256, 6):
                toks += r.emitted_tokens + [r.next_token]
        else:
            for _ in range(6):
                r = p.execute_exact_decode(st, prq, tok, pos, 256)
                toks += r.emitted_tokens + [r.next_token]
                pos += r.positions_advanced
                tok = r.next_token
        outs.append(toks)
    assert outs[0] == outs[1]


def test_invalid_invocations_are_rejected():
    from quantum_llm_b200 import QllmError
    model = synth.SynthModel(synth.TINY, seed=0)
    prq, _ = request_pair(context_limit=256)
    p = provider_from_synth(model)
    st = p.create_request_state()
    with pytest.raises(QllmError):                      # no draft yet
        p.execute_exact_decode(st, prq, 1, 0, 256)
    first = p.prefill(st, prq, synth.prompt(4096, 16, 0))
    with pytest.raises(QllmError):                      # wrong guaranteed token
        p.execute_exact_decode(st, prq, (first + 1) % 4096, 16, 256)
    with pytest.raises(QllmError):                      # position != draft cache length
        p.execute_exact_decode(st, prq, first, 17, 256)
    with pytest.raises(QllmError):                      # context limit beyond max_context
        p.execute_exact_decode(st, prq, first, 16, 100000)
    r = p.execute_exact_decode(st, prq, first, 16, 256)
    assert r.emitted_tokens[0] == first and r.positions_advanced == len(r.emitted_tokens)
