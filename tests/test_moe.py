"""Routed mixture-of-experts FFN (NVFP4 experts) inside the MTP step: the oracle's router
against an independent numpy restatement, and the CUDA provider against the oracle."""
import ctypes as C

import numpy as np
import pytest

from oracle import binding as ob
from tests import synth

# the tiny decoder with 8 experts of width 128, 2 selected per token
MOE = dict(synth.TINY, experts=8, route_width=2, expert_ffn=128, route_scale=1.0)


def _bf16(x):
    b = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return b.astype(np.uint32).view(np.float32)


def _route_numpy(logits, top_k, scale):
    """Top-k by (value desc, index asc) over BF16-rounded logits, softmax over the selected
    values with a sequential FP32 sum, times the scale, rounded to BF16."""
    v = _bf16(logits)
    order = sorted(range(len(v)), key=lambda i: (-float(v[i]), i))[:top_k]
    top = max(float(v[i]) for i in order)
    e = [np.float32(np.exp(np.float64(np.float32(v[i]) - np.float32(top)))) for i in order]
    total = np.float32(0)
    for x in e:
        total = np.float32(total + x)
    s = [np.float32(x / total) for x in e]
    if scale != 1.0:
        s = [np.float32(x * np.float32(scale)) for x in s]
    return np.array(order, np.uint32), _bf16(np.array(s, np.float32))


def _route_oracle(logits, top_k, scale):
    idx = np.zeros(top_k, np.uint32)
    sc = np.zeros(top_k, np.float32)
    ob.lib().qo_moe_route(ob._ptr(np.ascontiguousarray(logits, np.float32)), len(logits), top_k, np.float32(scale),
                          ob._ptr(idx), ob._ptr(sc))
    return idx, sc


@pytest.mark.parametrize("experts,top_k,scale", [(8, 2, 1.0), (128, 8, 2.5), (128, 8, 1.0), (64, 1, 1.0), (7, 7, 0.5)])
def test_router_matches_an_independent_restatement(experts, top_k, scale):
    rng = np.random.default_rng(experts * 100 + top_k)
    for trial in range(20):
        logits = rng.normal(0, 2.0, experts).astype(np.float32)
        if trial % 3 == 0:   # exact ties after BF16 rounding: the lower expert id wins
            logits[rng.integers(0, experts, 4)] = logits.max()
        want_idx, want_sc = _route_numpy(logits, top_k, scale)
        idx, sc = _route_oracle(logits, top_k, scale)
        assert np.array_equal(idx, want_idx)
        assert np.array_equal(sc, want_sc)


def test_router_known_answer():
    # 2.004 rounds to 2.0 in BF16: four-way tie, ids 1, 2, 4 win; equal weights 2.5 / 3
    logits = np.array([0.5, 2.0, 2.0, -1.0, 2.004, 0.1, 1.99, 2.0], np.float32)
    idx, sc = _route_oracle(logits, 3, 2.5)
    assert list(idx) == [1, 2, 4]
    assert np.array_equal(sc, _bf16(np.full(3, np.float32(np.float32(1) / np.float32(3)) * np.float32(2.5), np.float32)))


def _decode(session, rq, first, position, count):
    out, tok = [], first
    while len(out) < count:
        r = session.execute_exact_decode(rq, tok, position)
        out += list(r.emitted[:r.emitted_count])
        position += r.positions_advanced
        tok = r.next_token
    return out[:count]


def test_oracle_speculation_does_not_change_the_routed_model_s_greedy_output():
    prompt = synth.prompt(4096, 40, 2)
    rq = synth.request(context_limit=256)
    outs = []
    for other_draft in (False, True):
        m = synth.SynthModel(MOE, seed=4)
        if other_draft:
            rng = np.random.default_rng(17)
            m.mtp_fusion = synth.SynthMatrix(rng.normal(0, 0.02, (256, 512)).astype(np.float32))
        s = m.oracle_session()
        first = s.prefill(prompt, 5, rq)
        outs.append(_decode(s, rq, first, len(prompt), 20))
    assert outs[0] == outs[1]


# ------------------------------------------------------------------------------- GPU
@pytest.mark.gpu
@pytest.mark.parametrize("experts,top_k,scale", [(8, 2, 1.0), (128, 8, 2.5), (256, 8, 1.0), (40, 3, 1.0)])
def test_router_kernel_matches_the_oracle(experts, top_k, scale):
    import torch
    from quantum_llm_b200 import lib
    from tests.gpu_util import dev
    L = lib.load()
    rng = np.random.default_rng(experts + top_k)
    rows = 5
    logits = rng.normal(0, 2.0, (rows, experts)).astype(np.float32)
    logits[1, rng.integers(0, experts, 5)] = logits[1].max()     # ties
    logits[2] = 0.25                                               # everything ties
    d = dev(logits)
    idx = torch.zeros((rows, top_k), dtype=torch.int32, device="cuda")
    sc = torch.zeros((rows, top_k), dtype=torch.float32, device="cuda")
    rc = L.qllm_k_moe_route(d.data_ptr(), rows, experts, top_k, scale, idx.data_ptr(), sc.data_ptr(), None)
    assert rc == 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    for r in range(rows):
        want_idx, want_sc = _route_oracle(logits[r], top_k, scale)
        assert np.array_equal(idx[r].cpu().numpy().astype(np.uint32), want_idx)
        assert np.array_equal(sc[r].cpu().numpy(), want_sc)


@pytest.mark.gpu
@pytest.mark.parametrize("route_scale,graph,hidden,expert_ffn",
                         [(1.0, True, 256, 128), (2.5, False, 256, 128), (1.0, True, 192, 144)])
def test_routed_experts_step_equals_the_oracle(route_scale, graph, hidden, expert_ffn):
    # CUDA-core GEMV + scalar attention + exact expert arithmetic: the same bits as the oracle.
    # hidden 256 / width 128: expert weights staged through shared memory by bulk copies;
    # hidden 192 / width 144 (rows that are not whole 16-byte granules): the kernels that load
    # them straight into registers
    from tests.test_gpu_step import compare, run_cpu, run_gpu
    model = synth.SynthModel(dict(MOE, route_scale=route_scale, hidden=hidden, expert_ffn=expert_ffn), seed=5)
    prompt = synth.prompt(4096, 96, 5)
    gpu = run_gpu(model, prompt, 0, 24, graph=graph)
    cpu = run_cpu(model, prompt, 0, 24)
    c = compare(gpu, cpu, len(prompt))
    print("routed experts parity", c)
    assert gpu["drafts"] == cpu["drafts"]
    assert gpu["stream"] == cpu["stream"]
    assert c["exact"] == c["shared"] and c["shared"] >= 20
    # the first page holds prompt positions only (later pages also hold rows of rejected
    # speculative positions, which the two sides are free to leave in different states)
    p, st, o = gpu["provider"], gpu["state"], cpu["oracle"]
    want = o.page(0)
    assert np.array_equal(p.read_page(st, 0)[:want.size], want)
