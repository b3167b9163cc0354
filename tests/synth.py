"""Seeded synthetic models and prompts for the parity tests.

The reference ships no NVFP4 weight quantiser (it copies checkpoint payloads),
so the harness owns one: the reference's NVFP4 activation-quantiser formula
(runtime/src/cuda/transformer_kernels.cu:1960-1967) applied to weight rows with a
per-tensor scale 448*6/absmax.  Both the oracle and the CUDA path consume the
same bytes produced here.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import binding as ob  # noqa: E402

INPUT_SCALE = 448.0 * 6.0 / 8.0  # activation global scale, fixed per tensor

TINY = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=1024, vocab=4096,
            draft_vocab=4096, rotary_dim=64, rope_theta=1e6, eps=1e-6, page_tokens=64,
            kv_encoding=ob.KV_F16, mtp_kv_encoding=ob.KV_Q8, activation_bf16=1, draft_depth=4,
            max_context=256, split_tokens=64)


def bf16_bits(x):
    x = np.ascontiguousarray(x, np.float32)
    b = x.view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFF + ((b >> 16) & 1)) >> 16
    return b.astype(np.uint16)


class SynthMatrix:
    def __init__(self, w, input_scale=INPUT_SCALE):
        w = np.ascontiguousarray(w, np.float32)
        amax = np.float32(np.abs(w).max())
        self.divisor = np.float32(448.0 * 6.0) / amax  # stored divisor g
        self.weight_scale = np.float32(1.0) / self.divisor
        self.input_scale = np.float32(input_scale)
        self.codes, self.scales = ob.quantize_weights(w, self.divisor)
        self.rows, self.cols = w.shape

    def oracle(self):
        return ob.matrix(self.codes, self.scales, self.weight_scale, self.input_scale)


class SynthBlock:
    def __init__(self, cfg, rng, base=None, noise=0.0):
        H, F = cfg["hidden"], cfg["ffn"]
        qkv_rows = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"]
        shapes = dict(qkv=(qkv_rows, H), o=(H, cfg["q_heads"] * cfg["head_dim"]),
                      gate_up=(2 * F, H), down=(H, F))
        self.experts = int(cfg.get("experts", 0))
        if self.experts:   # routed experts: separate gate / up / down matrices per expert
            W = cfg["expert_ffn"]
            shapes["router"] = (self.experts, H)
            for e in range(self.experts):
                shapes[f"gate{e}"], shapes[f"up{e}"], shapes[f"down{e}"] = (W, H), (W, H), (H, W)
        self.master = {}
        for name, shape in shapes.items():
            if base is None:
                std = 0.2 if name == "router" else 0.02   # router logits spread over a few units
                w = rng.normal(0.0, std, shape).astype(np.float32)
            else:
                w = base.master[name] + rng.normal(0.0, noise, shape).astype(np.float32)
            self.master[name] = w
        self.qkv, self.o, self.gate_up, self.down = (SynthMatrix(self.master[n]) for n in
                                                     ("qkv", "o", "gate_up", "down"))
        self.input_norm = np.ones(H, np.float32)
        self.post_norm = np.ones(H, np.float32)
        self.router = None
        if self.experts:
            # every projection has its own activation scale, as in the checkpoint format
            self.router = SynthMatrix(self.master["router"])
            self.expert_gate = [SynthMatrix(self.master[f"gate{e}"], INPUT_SCALE) for e in range(self.experts)]
            self.expert_up = [SynthMatrix(self.master[f"up{e}"], 300.0 + 4.0 * e) for e in range(self.experts)]
            self.expert_down = [SynthMatrix(self.master[f"down{e}"], 2000.0 + 16.0 * e) for e in range(self.experts)]

    def oracle(self):
        if not self.experts:
            return ob.Block(ob._ptr(self.input_norm), self.qkv.oracle(), self.o.oracle(),
                            ob._ptr(self.post_norm), self.gate_up.oracle(), self.down.oracle())
        arrays = [(ob.Matrix * self.experts)(*[m.oracle() for m in group])
                  for group in (self.expert_gate, self.expert_up, self.expert_down)]
        self._oracle_arrays = arrays   # keep the ctypes arrays alive
        return ob.Block(ob._ptr(self.input_norm), self.qkv.oracle(), self.o.oracle(),
                        ob._ptr(self.post_norm), self.gate_up.oracle(), self.down.oracle(),
                        self.router.oracle(), arrays[0], arrays[1], arrays[2])


class SynthModel:
    """Random-init decoder + one MTP block = last target block + N(0, 0.004)."""

    def __init__(self, cfg, seed=0):
        self.cfg = dict(cfg)
        rng = np.random.default_rng(seed)
        H, V = cfg["hidden"], cfg["vocab"]
        self.embedding = bf16_bits(rng.normal(0.0, 0.02, (V, H)).astype(np.float32))
        self.layers = [SynthBlock(cfg, rng) for _ in range(cfg["layers"])]
        self.final_norm = np.ones(H, np.float32)
        self.head = SynthMatrix(rng.normal(0.0, 0.02, (V, H)).astype(np.float32))
        self.mtp_embedding_norm = np.ones(H, np.float32)
        self.mtp_hidden_norm = np.ones(H, np.float32)
        self.mtp_draft_norm = np.ones(H, np.float32)
        self.mtp_fusion = SynthMatrix(rng.normal(0.0, 0.02, (H, 2 * H)).astype(np.float32))
        self.mtp_block = SynthBlock(cfg, rng, base=self.layers[-1], noise=0.004)

    def oracle_config(self):
        c = ob.Config()
        for k, v in self.cfg.items():
            setattr(c, k, v)
        return c

    def oracle_session(self):
        blocks = (ob.Block * len(self.layers))(*[b.oracle() for b in self.layers])
        w = ob.Weights(ob._ptr(self.embedding), blocks, ob._ptr(self.final_norm), self.head.oracle(),
                       ob._ptr(self.mtp_embedding_norm), ob._ptr(self.mtp_hidden_norm),
                       self.mtp_fusion.oracle(), self.mtp_block.oracle(), ob._ptr(self.mtp_draft_norm))
        return ob.Session(self.oracle_config(), w, (self, blocks))


def _matrix_from(codes, scales, like):
    m = SynthMatrix.__new__(SynthMatrix)
    m.codes, m.scales = np.ascontiguousarray(codes), np.ascontiguousarray(scales)
    m.divisor, m.weight_scale, m.input_scale = like.divisor, like.weight_scale, like.input_scale
    m.rows, m.cols = m.codes.shape[0], m.codes.shape[1] * 2
    return m


def _take_rows(m, ranges):
    return _matrix_from(np.concatenate([m.codes[a:b] for a, b in ranges]),
                        np.concatenate([m.scales[a:b] for a, b in ranges]), m)


def _take_columns(m, start, stop):
    return _matrix_from(m.codes[:, start // 2:stop // 2], m.scales[:, start // 16:stop // 16], m)


def shard_model(model, rank, ranks):
    """Tensor-parallel shard `rank` of a dense SynthModel: the rank's q/k/v head rows and gate/up
    rows, the matching K columns of o and down (slices of the same quantised tensors);
    everything else is shared with `model`.  `cfg` carries the local head and FFN counts."""
    import copy
    c = model.cfg
    QH, KV, HD, F = c["q_heads"], c["kv_heads"], c["head_dim"], c["ffn"]
    assert QH % ranks == 0 and KV % ranks == 0 and F % (16 * ranks) == 0 and not c.get("experts", 0)
    q, kv, f = QH // ranks * HD, KV // ranks * HD, F // ranks
    k0, v0 = QH * HD, (QH + KV) * HD

    def shard_block(b):
        s = copy.copy(b)
        s.qkv = _take_rows(b.qkv, [(rank * q, (rank + 1) * q), (k0 + rank * kv, k0 + (rank + 1) * kv),
                                   (v0 + rank * kv, v0 + (rank + 1) * kv)])
        s.o = _take_columns(b.o, rank * q, (rank + 1) * q)
        s.gate_up = _take_rows(b.gate_up, [(rank * f, (rank + 1) * f), (F + rank * f, F + (rank + 1) * f)])
        s.down = _take_columns(b.down, rank * f, (rank + 1) * f)
        return s

    out = copy.copy(model)
    out.cfg = dict(c, q_heads=QH // ranks, kv_heads=KV // ranks, ffn=F // ranks)
    out.layers = [shard_block(b) for b in model.layers]
    out.mtp_block = shard_block(model.mtp_block)
    return out


def prompt(vocab, count, seed):
    return np.random.default_rng(seed).integers(0, vocab, count, dtype=np.uint32)


def request(seed=1234, temperature_ppm=0, top_p_ppm=950000, top_k=20, min_p_ppm=0, context_limit=256,
            presence_penalty_ppm=0, first_output_position=0):
    return ob.Request(seed, temperature_ppm, top_p_ppm, top_k, min_p_ppm, context_limit,
                      2000000 + presence_penalty_ppm, first_output_position)
