"""Two-layer models with the projection widths of the benchmarked configurations, built on the
host so that the CPU oracle and the CUDA provider consume the same bytes.

dense27b: hidden 5120, 40 q / 8 kv heads of 128, FFN 17408, vocabulary 151936 (draft 65536), Q4H
target cache, Q8 draft cache.  moe35b: hidden 2048, 32 q / 4 kv heads, 128 experts of width 768
(8 per token).  echo27b: dense27b with the attention and FFN output projections scaled to almost
nothing and a fusion matrix that passes the normalised embedding through, so that the draft head
can be right and acceptance lengths above zero occur (the construction of
tests/test_oracle_step.py::echo_model at full width).

Weights are N(0, 0.02) drawn in row blocks from counter-seeded generators (the same values
whatever the number of threads), the embedding of token t is the BF16 rounding of the head's master
row t + 9000 (so that the echo model walks through the vocabulary, in and out of the draft head's
65536 rows, and acceptance lengths vary), the draft block is the last target block plus N(0, 0.004).  tests/golden/
make_full_width_golden.py runs the oracle over these models once and stores what the GPU test
(tests/test_full_width_golden.py) compares against; the fixture also records SHA-256 digests of
the quantised weights, so a host that draws other numbers is reported as such, not as a parity
failure.
"""
import hashlib
import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from oracle import binding as ob
from tests import synth

DENSE = dict(layers=2, hidden=5120, q_heads=40, kv_heads=8, head_dim=128, ffn=17408, vocab=151936,
             draft_vocab=65536, rotary_dim=128, rope_theta=1e6, eps=1e-6, page_tokens=256,
             kv_encoding=ob.KV_Q4H, mtp_kv_encoding=ob.KV_Q8, activation_bf16=1, draft_depth=4,
             max_context=1024, split_tokens=512)
MOE = dict(layers=2, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, ffn=768, vocab=151936,
           draft_vocab=65536, rotary_dim=128, rope_theta=1e6, eps=1e-6, page_tokens=256,
           kv_encoding=ob.KV_Q4H, mtp_kv_encoding=ob.KV_Q8, activation_bf16=1, draft_depth=4,
           max_context=1024, split_tokens=256, experts=128, route_width=8, expert_ffn=768, route_scale=1.0)
CASES = {"dense27b": (DENSE, 3), "moe35b": (MOE, 4), "echo27b": (DENSE, 3)}
PROMPT_TOKENS, STEPS, PROMPT_SEED = 320, 6, 11
SAMPLE_STRIDE = 128          # every 128th logit of a verify row is stored next to its top 64
_BLOCK_ROWS = 512
EMBEDDING_SHIFT = 9000
_POOL = ThreadPoolExecutor(max_workers=min(32, os.cpu_count() or 8))


def normal_rows(rows, cols, std, key, base=None, noise=0.0):
    """[rows, cols] float32 N(0, std) (or base + N(0, noise)).  Drawing a billion normals takes
    minutes on a host, so a tall matrix is drawn as its first eighth only -- block b of 512 rows from
    default_rng([key..., b]), the same values whatever the number of threads -- and part k of the
    other seven is that eighth rotated by 16 k columns, negated for odd k: rows with the same
    statistics that compute different functions of their input."""
    out = np.empty((rows, cols), np.float32)
    parts = 8 if rows >= 4096 and rows % 8 == 0 else 1
    drawn = rows // parts

    def fill(b):
        r0, r1 = b * _BLOCK_ROWS, min(drawn, (b + 1) * _BLOCK_ROWS)
        g = np.random.default_rng(list(key) + [b])
        g.standard_normal(out=out[r0:r1], dtype=np.float32)
        out[r0:r1] *= np.float32(std if base is None else noise)

    list(_POOL.map(fill, range((drawn + _BLOCK_ROWS - 1) // _BLOCK_ROWS)))

    def derive(k):
        part = out[k * drawn:(k + 1) * drawn]
        shift = (16 * k) % cols
        part[:, shift:] = out[:drawn, :cols - shift]
        part[:, :shift] = out[:drawn, cols - shift:]
        if k & 1:
            np.negative(part, out=part)

    list(_POOL.map(derive, range(1, parts)))
    if base is not None:
        out += base
    return out


class _Block:
    pass


def _quantized(w, input_scale=synth.INPUT_SCALE):
    """synth.SynthMatrix(w) without the full-size temporaries (per-tensor scale 448*6/absmax)."""
    m = synth.SynthMatrix.__new__(synth.SynthMatrix)
    amax = np.float32(max(float(w.max()), -float(w.min())))
    m.divisor = np.float32(448.0 * 6.0) / amax
    m.weight_scale = np.float32(1.0) / m.divisor
    m.input_scale = np.float32(input_scale)
    m.codes, m.scales = ob.quantize_weights(w, m.divisor)
    m.rows, m.cols = w.shape
    return m


def _bf16_bits(w):
    import torch
    return torch.from_numpy(w).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def _dense_block(cfg, seed, index, digest, keep_master=False, base=None):
    H, F = cfg["hidden"], cfg["ffn"]
    qkv_rows = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"]
    shapes = dict(qkv=(qkv_rows, H), o=(H, cfg["q_heads"] * cfg["head_dim"]))
    experts = int(cfg.get("experts", 0))
    if not experts:
        shapes.update(gate_up=(2 * F, H), down=(H, F))
    b = _Block()
    b.experts = experts
    b.master = {}
    for j, (name, (rows, cols)) in enumerate(shapes.items()):
        w = normal_rows(rows, cols, 0.02, (seed, index, j)) if base is None else \
            normal_rows(rows, cols, 0.0, (seed, index, j), base=base.master[name], noise=0.004)
        setattr(b, name, _quantized(w))
        digest.update(getattr(b, name).codes[::97].tobytes())
        if keep_master:
            b.master[name] = w
    b.input_norm = np.ones(H, np.float32)
    b.post_norm = np.ones(H, np.float32)
    b.router = None
    if experts:
        W = cfg["expert_ffn"]
        b.gate_up = b.down = synth.SynthMatrix(np.ones((16, 16), np.float32))   # unused by a routed block
        w = normal_rows(experts, H, 0.2, (seed, index, 4)) if base is None else \
            normal_rows(experts, H, 0.0, (seed, index, 4), base=base.master["router"], noise=0.004)
        b.router = _quantized(w)
        if keep_master:
            b.master["router"] = w
        groups = {}
        for j, (name, rows, cols, scale0, step) in enumerate((("gate", W, H, synth.INPUT_SCALE, 0.0),
                                                              ("up", W, H, 300.0, 4.0), ("down", H, W, 2000.0, 16.0))):
            w = normal_rows(experts * rows, cols, 0.02, (seed, index, 5 + j)) if base is None else \
                normal_rows(experts * rows, cols, 0.0, (seed, index, 5 + j), base=base.master[name], noise=0.004)
            # every expert projection has its own tensor scale and its own activation scale
            groups[name] = [_quantized(w[e * rows:(e + 1) * rows], scale0 + step * e) for e in range(experts)]
            digest.update(groups[name][0].codes.tobytes())
            if keep_master:
                b.master[name] = w
        b.expert_gate, b.expert_up, b.expert_down = groups["gate"], groups["up"], groups["down"]
    b.oracle = synth.SynthBlock.oracle.__get__(b)
    return b


def _rescaled(matrix, factor):
    """The same quantised bytes with the per-tensor multiplier scaled (an output that is `factor` as large)."""
    m = synth._matrix_from(matrix.codes, matrix.scales, matrix)
    m.weight_scale = np.float32(matrix.weight_scale * np.float32(factor))
    return m


_BUILT = {}


def _echo_variant(model):
    """The same weights with o and down scaled to almost nothing and a pass-through fusion matrix."""
    import copy
    m = copy.copy(model)
    H = m.cfg["hidden"]

    def quiet(block):
        b = copy.copy(block)
        b.o, b.down = _rescaled(block.o, 1e-4), _rescaled(block.down, 1e-4)
        b.oracle = synth.SynthBlock.oracle.__get__(b)
        return b

    m.layers = [quiet(b) for b in model.layers]
    m.mtp_block = quiet(model.mtp_block)
    fusion = np.zeros((H, 2 * H), np.float32)
    fusion[np.arange(H), np.arange(H)] = 1.0
    m.mtp_fusion = synth.SynthMatrix(fusion)
    return m


def build(case):
    """-> (SynthModel-compatible model, SHA-256 hex digest over samples of its quantised weights).
    Models are kept for the life of the process (echo27b shares dense27b's weights)."""
    if case in _BUILT:
        return _BUILT[case]
    if case == "echo27b":
        dense, digest = build("dense27b")
        _BUILT[case] = (_echo_variant(dense), digest)
        return _BUILT[case]
    cfg, seed = CASES[case]
    cfg = dict(cfg)
    digest = hashlib.sha256()
    m = synth.SynthModel.__new__(synth.SynthModel)
    m.cfg = cfg
    H, V = cfg["hidden"], cfg["vocab"]
    head_master = normal_rows(V, H, 0.02, (seed, 100))
    # token t embeds as the head row of token t + EMBEDDING_SHIFT: tied weights would make every
    # token its own most likely successor
    m.embedding = np.roll(_bf16_bits(head_master), -EMBEDDING_SHIFT, axis=0)
    m.head = _quantized(head_master)
    del head_master
    digest.update(m.head.codes[::997].tobytes())
    m.layers = [_dense_block(cfg, seed, l, digest, keep_master=(l == cfg["layers"] - 1)) for l in range(cfg["layers"])]
    m.final_norm = np.ones(H, np.float32)
    m.mtp_embedding_norm = np.ones(H, np.float32)
    m.mtp_hidden_norm = np.ones(H, np.float32)
    m.mtp_draft_norm = np.ones(H, np.float32)
    m.mtp_block = _dense_block(cfg, seed + 1000, 0, digest, base=m.layers[-1])
    m.layers[-1].master = {}
    m.mtp_fusion = _quantized(normal_rows(H, 2 * H, 0.02, (seed, 101)))
    digest.update(m.mtp_fusion.codes[::97].tobytes())
    _BUILT[case] = (m, digest.hexdigest())
    return _BUILT[case]


def prompt(case):
    return synth.prompt(CASES[case][0]["vocab"], PROMPT_TOKENS, PROMPT_SEED)


def row_summary(row):
    """What the fixture keeps of one logits row: its 64 largest entries (ties to the lower id) and a
    strided sample, enough for a max-abs / relative-RMS comparison without storing 151936 floats."""
    order = np.lexsort((np.arange(row.size), -row.astype(np.float64)))[:64]
    return order.astype(np.uint32), row[order].astype(np.float32), row[::SAMPLE_STRIDE].astype(np.float32)


def committed_page_bytes(page, cfg, layer_offsets, page_index, committed):
    """The bytes of one cache page that belong to positions below `committed` (all layers: target
    layers then the draft layer), as one array.  Slots past the accepted prefix hold speculative
    rows that are overwritten before any read, and the provider's fixed-width draft pass also
    stores padding rows there, so only committed positions are comparable."""
    pt, kv, hd = cfg["page_tokens"], cfg["kv_heads"], cfg["head_dim"]
    n = max(0, min(pt, committed - page_index * pt))
    parts = []
    for layer in range(cfg["layers"] + 1):
        enc = cfg["kv_encoding"] if layer < cfg["layers"] else cfg["mtp_kv_encoding"]
        lo = layer_offsets[layer]
        if enc == ob.KV_Q4H:      # [K codes kv,pt,hd/2][K scales kv,pt f16][V codes][V scales]
            codes, scales = kv * pt * (hd // 2), kv * pt * 2
            for _ in range(2):
                parts.append(page[lo:lo + codes].reshape(kv, pt, hd // 2)[:, :n].reshape(-1))
                parts.append(page[lo + codes:lo + codes + scales].reshape(kv, pt, 2)[:, :n].reshape(-1))
                lo += codes + scales
        else:                     # token-major records: [K: pt records of kv heads][V: ...]
            record = kv * (hd + 2 if enc == ob.KV_Q8 else 2 * hd)
            for _ in range(2):
                parts.append(page[lo:lo + n * record])
                lo += pt * record
    return np.concatenate(parts)
