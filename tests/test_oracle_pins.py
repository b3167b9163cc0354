"""Pins the CPU oracle to the reference: golden vectors produced by the
reference's own code (tests/golden/make_golden.py), the known-answer values of
the reference's unit tests, and, when oracle/_ref is present, the reference's
sampler itself run side by side."""
import json
import math
import os

import numpy as np
import pytest

from oracle import binding as ob


@pytest.fixture(scope="module")
def L():
    return ob.lib()


def test_e4m3_decode_matches_reference_table(L, golden_dir):
    table = json.load(open(os.path.join(golden_dir, "fp4_tables.json")))["e4m3fn_decode"]
    assert len(table) == 254
    for code, value in table.items():
        assert L.qo_e4m3_decode(int(code)) == value
    assert math.isnan(L.qo_e4m3_decode(0x7F)) and math.isnan(L.qo_e4m3_decode(0xFF))


def test_e2m1_decode_and_nibble_order_match_reference(L, golden_dir):
    table = json.load(open(os.path.join(golden_dir, "fp4_tables.json")))["e2m1_byte_decode_low_then_high"]
    for byte, (low, high) in enumerate(table):
        assert L.qo_e2m1_decode(byte & 15) == low and L.qo_e2m1_decode(byte >> 4) == high
    # tests/compiler/test_fp4_quant.py:337-339: 0.5 low nibble, -0.5 high nibble -> 0x91
    assert L.qo_e2m1_encode(0.5) | (L.qo_e2m1_encode(-0.5) << 4) == 0x01 | (0x09 << 4)
    assert L.qo_e2m1_encode(1.0) | (L.qo_e2m1_encode(-1.5) << 4) == 0x02 | (0x0B << 4)


def test_e4m3_encode_is_nearest_ties_to_even_code(L):
    # independent exhaustive nearest search (the method of
    # runtime/tools/native_nvfp4_cuda_smoke.cpp:98-116), not the encoder's own arithmetic
    values = np.array([L.qo_e4m3_decode(c) for c in range(0x7F)], np.float64)
    rng = np.random.default_rng(3)
    probes = np.concatenate([rng.uniform(0, 460, 4000), rng.uniform(0, 0.05, 2000),
                             (values[:-1] + values[1:]) / 2, values]).astype(np.float32)
    for x in probes:
        err = np.abs(values - np.float64(x))
        best = np.flatnonzero(err == err.min())
        want = best[0] if len(best) == 1 else [c for c in best if c % 2 == 0][0]
        assert L.qo_e4m3_encode(float(x)) == want, x
    assert L.qo_e4m3_encode(1e9) == 0x7E and L.qo_e4m3_encode(-1e9) == 0xFE


def test_e2m1_encode_thresholds(L):
    # transformer_kernels.cu:1917-1929: ties go to the even code
    cases = {0.25: 0, 0.26: 1, 0.75: 2, 1.25: 2, 1.26: 3, 1.75: 4, 2.5: 4, 2.51: 5, 3.5: 6, 5.0: 6, 5.01: 7, 100.0: 7}
    for x, code in cases.items():
        assert L.qo_e2m1_encode(x) == code and L.qo_e2m1_encode(-x) == (code | 8)


def test_bf16_and_f16_rounding(L):
    import torch
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-6, 500), rng.normal(0, 6e4, 500)]).astype(np.float32)
    want_bf = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    want_h = torch.from_numpy(x).to(torch.float16)
    for i, v in enumerate(x):
        assert L.qo_bf16_round(float(v)) == want_bf[i]
        if np.isfinite(want_h[i].item()):
            assert L.qo_f16_bits(float(v)) == int(want_h[i].view(torch.int16).item()) & 0xFFFF


def test_counter_uniform_matches_reference_vectors(L, golden_dir):
    for seed, pos, stream, index, want in json.load(open(os.path.join(golden_dir, "sampler_cases.json")))["counter_uniform"]:
        assert L.qo_counter_uniform(seed, pos, stream, index) == want


def test_distribution_matches_reference_vectors(golden_dir):
    for case in json.load(open(os.path.join(golden_dir, "sampler_cases.json")))["distributions"]:
        tokens, probs = ob.make_distribution(case["logits"], case["tokens"], case["temperature_ppm"],
                                             case["top_p_ppm"], case["min_p_ppm"])
        assert list(tokens) == case["out_tokens"]
        assert list(probs) == case["out_probabilities"]  # bit-exact doubles


def test_rejection_matches_reference_vectors(golden_dir):
    for case in json.load(open(os.path.join(golden_dir, "sampler_cases.json")))["rejections"]:
        r, token = ob.rejection_sample(case["proposal"], case["target"], case["draft"], case["ua"], case["uc"])
        assert (r, token) == (case["accepted"], case["token"])


def test_sample_token_matches_reference_vectors(golden_dir):
    """The scalar decode fallback's sampler (whole-row ordering, top_k 0 or above 64) against
    tokens produced by the reference's own distribution / sampling / counter functions."""
    cases = json.load(open(os.path.join(golden_dir, "sampler_cases.json")))["sample_token"]
    assert len(cases) >= 40
    for case in cases:
        logits = np.array(case["logits_f32_bits"], np.uint32).view(np.float32)
        rq = ob.Request(case["seed"], case["temperature_ppm"], case["top_p_ppm"], case["top_k"], case["min_p_ppm"],
                        0, 2000000)
        assert ob.sample_token(logits, rq, case["position"]) == case["token"]
    # what the reference throws on: no finite maximum, top_k beyond the row
    rq = ob.Request(1, 700000, 900000, 0, 0, 0, 2000000)
    assert ob.sample_token(np.full(100, -np.inf, np.float32), rq, 3) is None
    assert ob.sample_token(np.zeros(10, np.float32), ob.Request(1, 700000, 900000, 11, 0, 0, 2000000), 3) is None


def test_nucleus_known_answer():
    # runtime/tests/cache_state_test.cpp:105-114
    tokens, probs = ob.make_distribution([4.0, 3.0, 2.0, 1.0], [9, 5, 2, 1], 1_000_000, 800_000, 0)
    assert list(tokens) == [9, 5] and abs(probs[0] - 0.7310585786300049) < 1e-12


def test_rejection_mass_matches_closed_form(L):
    # runtime/tests/cache_state_test.cpp:57-103, with 100 000 trials
    target = ([3, 7, 11], [0.50, 0.30, 0.20])
    draft = ([3, 7, 13], [0.20, 0.70, 0.10])
    toks = [3, 7, 11, 13]
    p = dict(zip(*target)); q = dict(zip(*draft))
    rej = sum(q.get(t, 0) - min(p.get(t, 0), q.get(t, 0)) for t in toks)
    res = sum(max(0.0, p.get(t, 0) - q.get(t, 0)) for t in toks)
    expected = {t: min(p.get(t, 0), q.get(t, 0)) + rej * max(0.0, p.get(t, 0) - q.get(t, 0)) / res for t in toks}
    trials = 100_000
    seen = dict.fromkeys(toks, 0)
    dt = np.array(draft[0], np.uint32); dp = np.array(draft[1], np.float64)
    for trial in range(trials):
        proposal = L.qo_sample_distribution(ob._ptr(dt), ob._ptr(dp), 3, L.qo_counter_uniform(19, trial, 1, 0))
        _, token = ob.rejection_sample(proposal, target, draft, L.qo_counter_uniform(19, trial, 2, 0),
                                       L.qo_counter_uniform(19, trial, 3, 0))
        seen[token] += 1
    for t in toks:
        assert abs(seen[t] / trials - expected[t]) < 0.006


def test_sampler_side_by_side_with_reference_build():
    ref = ob.ref_sampler()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(11)
    for _ in range(300):
        k = int(rng.integers(1, 65))
        logits = np.sort(rng.normal(0, 3.0, k).astype(np.float32))[::-1].copy()
        tokens = np.sort(rng.permutation(100000)[:k]).astype(np.uint32)
        args = (logits, tokens, int(rng.integers(1, 2_000_001)), int(rng.integers(1, 1_000_001)), int(rng.integers(0, 200_000)))
        a, b = ob.make_distribution(*args), ob.make_distribution(*args, impl=ref)
        assert (a is None) == (b is None)
        if a is not None:
            assert list(a[0]) == list(b[0]) and list(a[1]) == list(b[1])
        s, p, st, i = (int(x) for x in rng.integers(0, 2**31, 4))
        assert ob.lib().qo_counter_uniform(s, p, st, i) == ref.ref_counter_uniform(s, p, st, i)


def test_nvfp4_fixture_of_reference_smoke_tool(L):
    # runtime/tools/native_nvfp4_cuda_smoke.cpp:181-205: deterministic codes, all local
    # scales 0x38 (= 1.0); the tool's gate is max-abs error 0 against its host oracle.
    hidden = 64
    seed = 3
    codes = np.zeros((hidden, hidden // 2), np.uint8)
    for row in range(hidden):
        for pair in range(hidden // 2):
            low = 1 + (seed + row + 3 * pair) % 7
            high = (1 + (seed + 2 * row + pair) % 7) | (8 if (seed + row + pair) & 1 else 0)
            codes[row, pair] = low | (high << 4)
    scales = np.full((hidden, hidden // 16), 0x38, np.uint8)
    divisor = np.float32(2.0)
    m = ob.matrix(codes, scales, np.float32(1.0) / divisor, np.float32(4.0))
    x = np.random.default_rng(2).normal(0, 1, (3, hidden)).astype(np.float32)
    y = ob.gemv(m, x)
    # independent float64 evaluation of the same definition
    levels = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6])
    w = np.empty((hidden, hidden))
    w[:, 0::2] = levels[codes & 15]
    w[:, 1::2] = levels[codes >> 4]
    w /= 2.0
    xq = np.empty_like(x)
    L.qo_nvfp4_fake_quant(ob._ptr(x), 3, hidden, np.float32(4.0), ob._ptr(xq))
    want = xq.astype(np.float64) @ w.T
    import torch
    want_bf = torch.from_numpy(want.astype(np.float32)).to(torch.bfloat16).float().numpy()
    assert np.abs(y - want_bf).max() <= np.abs(want_bf).max() * 2 ** -7  # at most one BF16 ulp
    assert (y == want_bf).mean() > 0.98
