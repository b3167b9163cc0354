"""Regenerates tests/golden/*.json.  Run where the reference tree is present (its location:
QLLM_REFERENCE, else a `reference` directory beside the repository); the parity tests only read the committed
JSON.

  fp4_tables.json     decode tables produced by importing the reference's Python
                      decoders (compiler/expert_pack/fp4_reference.py)
  sampler_cases.json  outputs of the reference's own sampler
                      (runtime/src/speculative_sampling.cpp through oracle/_ref)
                      on seeded inputs
"""
import ctypes as C
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle.binding import REFERENCE_DEFAULT  # noqa: E402
sys.path.insert(0, os.path.join(os.environ.get("QLLM_REFERENCE", REFERENCE_DEFAULT), "compiler"))


def fp4_tables():
    from expert_pack import fp4_reference as fr
    e4m3 = {}
    for code in range(256):
        if code & 0x7F == 0x7F:
            continue
        e4m3[str(code)] = fr.decode_fp8_e4m3fn(code)
    e2m1 = [list(fr.decode_fp4_e2m1_values(bytes([b]))) for b in range(256)]
    return {"e4m3fn_decode": e4m3, "e2m1_byte_decode_low_then_high": e2m1}


def sampler_cases():
    from oracle import binding as ob
    ref = ob.ref_sampler()
    assert ref is not None, "oracle/_ref was not built"
    rng = np.random.default_rng(7)
    uniforms = [[int(s), int(p), int(st), int(i), ref.ref_counter_uniform(int(s), int(p), int(st), int(i))]
                for s, p, st, i in zip(rng.integers(0, 2**63, 64), rng.integers(0, 2**31, 64),
                                       rng.integers(0, 400, 64), rng.integers(0, 8, 64))]
    dists, rejections = [], []
    for case in range(48):
        k = int(rng.integers(1, 65))
        logits = np.sort(rng.normal(0, 2.0, k).astype(np.float32))[::-1].copy()
        if case % 5 == 0 and k > 2:
            logits[1] = logits[0]
        tokens = rng.permutation(5000)[:k].astype(np.uint32)
        for i in range(1, k):  # equal logits must carry ascending ids
            if logits[i] == logits[i - 1] and tokens[i] < tokens[i - 1]:
                tokens[i - 1], tokens[i] = tokens[i], tokens[i - 1]
        t_ppm = int(rng.choice([300000, 700000, 1000000, 1500000]))
        p_ppm = int(rng.choice([500000, 800000, 950000, 1000000]))
        m_ppm = int(rng.choice([0, 0, 50000]))
        d = ob.make_distribution(logits, tokens, t_ppm, p_ppm, m_ppm, impl=ref)
        dists.append({"logits": [float(x) for x in logits], "tokens": [int(x) for x in tokens],
                      "temperature_ppm": t_ppm, "top_p_ppm": p_ppm, "min_p_ppm": m_ppm,
                      "out_tokens": [int(x) for x in d[0]], "out_probabilities": [float(x) for x in d[1]]})
    for case in range(200):
        a, b = dists[int(rng.integers(len(dists)))], dists[int(rng.integers(len(dists)))]
        target = (a["out_tokens"], a["out_probabilities"])
        draft = (b["out_tokens"], b["out_probabilities"])
        proposal = int(draft[0][int(rng.integers(len(draft[0])))])
        ua, uc = float(rng.random()), float(rng.random())
        r, token = ob.rejection_sample(proposal, target, draft, ua, uc, impl=ref)
        rejections.append({"proposal": proposal, "target": target, "draft": draft, "ua": ua, "uc": uc,
                           "accepted": r, "token": token})
    return {"counter_uniform": uniforms, "distributions": dists, "rejections": rejections,
            "sample_token": sample_token_cases(ref, ob)}


def sample_token_cases(ref, ob):
    """sample_token (runtime/tools/dense_fp4_provider.cpp:771-802) composed from the reference's own
    functions: numpy orders the ids by the reference's comparator (logit descending, NaN last, id
    ascending), the reference's make_sampling_distribution / sample_distribution /
    counter_uniform do the rest.  Rows carry ties, infinities and (some) NaNs."""
    rng = np.random.default_rng(21)
    cases = []
    for case in range(40):
        n = int(rng.integers(70, 400))
        logits = rng.normal(0, 2.5, n).astype(np.float32)
        logits[rng.integers(0, n, 6)] = logits[int(rng.integers(0, n))]       # ties
        if case % 4 == 1:
            logits[rng.integers(0, n, 3)] = -np.inf
        if case % 4 == 2:
            logits[rng.integers(0, n, 2)] = np.nan
        if case % 8 == 7:
            logits[int(rng.integers(0, n))] = 0.0
            logits[int(rng.integers(0, n))] = -0.0
        top_k = min(n, [0, 0, 65, 100, n][case % 5])
        t_ppm = int(rng.choice([300000, 700000, 1000000, 2000000]))
        p_ppm = int(rng.choice([500000, 900000, 1000000]))
        m_ppm = int(rng.choice([0, 0, 20000]))
        seed, position = int(rng.integers(0, 2**63)), int(rng.integers(0, 2**20))
        nan = np.isnan(logits)
        order = np.lexsort((np.arange(n), -np.where(nan, 0, logits).astype(np.float64), nan))
        keep = order[:top_k or n].astype(np.uint32)
        d = ob.make_distribution(logits[keep], keep, t_ppm, p_ppm, m_ppm, impl=ref)
        u = ref.ref_counter_uniform(seed, position, 0, 0)
        token = C.c_uint32(0)
        tt, tp = np.ascontiguousarray(d[0], np.uint32), np.ascontiguousarray(d[1], np.float64)
        assert ref.ref_sample_distribution(tt.ctypes.data, tp.ctypes.data, len(tt), u, C.byref(token)) == 0
        cases.append({"logits_f32_bits": [int(x) for x in logits.view(np.uint32)], "top_k": top_k,
                      "temperature_ppm": t_ppm, "top_p_ppm": p_ppm, "min_p_ppm": m_ppm, "seed": seed,
                      "position": position, "token": int(token.value), "retained": len(tt)})
    return cases


if __name__ == "__main__":
    with open(os.path.join(HERE, "fp4_tables.json"), "w") as f:
        json.dump(fp4_tables(), f)
    with open(os.path.join(HERE, "sampler_cases.json"), "w") as f:
        json.dump(sampler_cases(), f)
    print("golden vectors written")
