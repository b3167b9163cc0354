"""Seeded random-init models built directly in device memory, for benchmarks and
large-shape property tests.  Weights are N(0, 0.02) quantised to NVFP4 by the
library's own device quantiser (per-tensor scale 448*6/absmax); the draft block is
the last target block plus N(0, 0.004).  torch is used for device memory and the
random generator only.
"""
import ctypes as C

import torch

from . import lib as _l
from .provider import Nvfp4MtpProvider

INPUT_SCALE = 448.0 * 6.0 / 8.0

# 27B-class dense target of the headline benchmark (64 layers, hidden 5120, 40q/8kv,
# head_dim 128, FFN 17408, vocab 151936), Q4H target cache, Q8 draft cache.
DENSE_27B = dict(layers=64, hidden=5120, q_heads=40, kv_heads=8, head_dim=128, ffn=17408, vocab=151936,
                 draft_vocab=65536, rotary_dim=128, rope_theta=1e6, eps=1e-6, page_tokens=256,
                 kv_encoding=_l.KV_Q4H, mtp_kv_encoding=_l.KV_Q8, activation_bf16=1, draft_depth=4,
                 max_context=33792, split_tokens=512)


# 35B-A3B-class sparse target (48 layers, hidden 2048, 32q/4kv, head_dim 128, 128 routed experts of
# width 768, 8 selected per token, no shared expert), Q4H target cache, Q8 draft cache.  `ffn` is
# unused by a routed model (kept non-zero for buffer sizing).
MOE_35B = dict(layers=48, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, ffn=768, vocab=151936,
               draft_vocab=65536, rotary_dim=128, rope_theta=1e6, eps=1e-6, page_tokens=256,
               kv_encoding=_l.KV_Q4H, mtp_kv_encoding=_l.KV_Q8, activation_bf16=1, draft_depth=4,
               max_context=9216, split_tokens=256, experts=128, route_width=8, expert_ffn=768, route_scale=1.0)


class DeviceMatrix:
    def __init__(self, codes, scales, weight_scale, rows, cols):
        self.codes, self.scales, self.weight_scale, self.rows, self.cols = codes, scales, weight_scale, rows, cols

    def c(self):
        return _l.Matrix(self.codes.data_ptr(), self.scales.data_ptr(), self.weight_scale, INPUT_SCALE,
                         self.rows, self.cols)

    def nbytes(self):
        return self.codes.numel() + self.scales.numel()

    def take_rows(self, ranges):
        """The output rows of the given (start, stop) ranges, in that order (same tensor scale)."""
        codes = torch.cat([self.codes[a:b] for a, b in ranges]).contiguous()
        scales = torch.cat([self.scales[a:b] for a, b in ranges]).contiguous()
        return DeviceMatrix(codes, scales, self.weight_scale, codes.shape[0], self.cols)

    def take_columns(self, start, stop):
        """Input columns [start, stop) (multiples of 16): a K-slice of the same quantised tensor."""
        assert start % 16 == 0 and stop % 16 == 0
        return DeviceMatrix(self.codes[:, start // 2:stop // 2].contiguous(),
                            self.scales[:, start // 16:stop // 16].contiguous(), self.weight_scale, self.rows,
                            stop - start)


def _random_rows(rows, cols, seed, device, std=0.02, base_seed=None, noise=0.0):
    gen = torch.Generator(device=device)
    gen.manual_seed(seed if base_seed is None else base_seed)
    w = torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * std
    if base_seed is not None:
        gen.manual_seed(seed)
        w += torch.randn((rows, cols), generator=gen, device=device, dtype=torch.float32) * noise
    return w


def quantize(w):
    """fp32 device tensor [rows, cols] -> DeviceMatrix (library quantiser)."""
    L = _l.load()
    rows, cols = w.shape
    divisor = float(448.0 * 6.0 / w.abs().max().item())
    codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((rows, cols // 16), dtype=torch.uint8, device=w.device)
    stream = torch.cuda.current_stream(w.device).cuda_stream
    _l.check(L.qllm_k_nvfp4_quantize_weights(w.data_ptr(), rows, cols, divisor, codes.data_ptr(), scales.data_ptr(),
                                              C.c_void_p(stream)))
    torch.cuda.current_stream(w.device).synchronize()
    weight_scale = float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(divisor, dtype=torch.float32))
    return DeviceMatrix(codes, scales, weight_scale, rows, cols)


def shard_block(m, cfg, rank, ranks):
    """Tensor-parallel shard of a dense block's projections: q/k/v head rows and gate/up rows of
    the rank (column split of the outputs), the matching K columns of o and down."""
    QH, KV, HD, F = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], cfg["ffn"]
    assert QH % ranks == 0 and KV % ranks == 0 and F % (16 * ranks) == 0 and not cfg.get("experts", 0)
    q, kv, f = QH // ranks * HD, KV // ranks * HD, F // ranks
    k0, v0 = QH * HD, (QH + KV) * HD
    return dict(
        qkv=m["qkv"].take_rows([(rank * q, (rank + 1) * q), (k0 + rank * kv, k0 + (rank + 1) * kv),
                                (v0 + rank * kv, v0 + (rank + 1) * kv)]),
        o=m["o"].take_columns(rank * q, (rank + 1) * q),
        gate_up=m["gate_up"].take_rows([(rank * f, (rank + 1) * f), (F + rank * f, F + (rank + 1) * f)]),
        down=m["down"].take_columns(rank * f, (rank + 1) * f))


def gather_handles(mine, ranks, group=None):
    """All ranks' exchange-area handles concatenated in rank order (what tp_attach takes)."""
    if ranks == 1:
        return bytes(mine)
    import torch.distributed as dist
    handles = [None] * ranks
    dist.all_gather_object(handles, bytes(mine), group=group)
    assert all(len(h) == _l.TP_HANDLE_BYTES for h in handles)
    return b"".join(handles)


class DeviceBlock:
    SHAPES = ("qkv", "o", "gate_up", "down")

    def __init__(self, cfg, seed, device, base_seed=None, tp=None):
        """`tp` = (rank, ranks): keep this rank's shard of every projection.  The full matrices are
        generated and quantised exactly as without `tp`, then sliced, so the ranks together hold
        the bytes of the unsharded model."""
        H, F = cfg["hidden"], cfg["ffn"]
        qkv_rows = (cfg["q_heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"]
        shapes = dict(qkv=(qkv_rows, H), o=(H, cfg["q_heads"] * cfg["head_dim"]), gate_up=(2 * F, H), down=(H, F))
        self.experts = int(cfg.get("experts", 0))
        names = self.SHAPES if not self.experts else ("qkv", "o")
        self.m = {}
        for i, name in enumerate(names):
            rows, cols = shapes[name]
            w = _random_rows(rows, cols, seed * 16 + i, device,
                             base_seed=None if base_seed is None else base_seed * 16 + i, noise=0.004)
            self.m[name] = quantize(w)
            del w
        if tp is not None:
            self.m = shard_block(self.m, cfg, *tp)
        self.input_norm = torch.ones(H, dtype=torch.float32, device=device)
        self.post_norm = torch.ones(H, dtype=torch.float32, device=device)
        if self.experts:
            W = cfg["expert_ffn"]
            base = None if base_seed is None else base_seed * 16
            self.router = quantize(_random_rows(self.experts, H, seed * 16 + 4, device, std=0.2,
                                                base_seed=None if base is None else base + 4, noise=0.004))
            self.expert = {}
            for j, (name, rows, cols) in enumerate((("gate", W, H), ("up", W, H), ("down", H, W))):
                # one draw for all experts of a role, then one quantisation (own scale) per expert
                w = _random_rows(self.experts * rows, cols, seed * 16 + 5 + j, device,
                                 base_seed=None if base is None else base + 5 + j, noise=0.004)
                self.expert[name] = [quantize(w[e * rows:(e + 1) * rows]) for e in range(self.experts)]
                del w

    def c(self):
        if not self.experts:
            return _l.Block(self.input_norm.data_ptr(), self.m["qkv"].c(), self.m["o"].c(), self.post_norm.data_ptr(),
                            self.m["gate_up"].c(), self.m["down"].c())
        self._arrays = [(_l.Matrix * self.experts)(*[m.c() for m in self.expert[name]])
                        for name in ("gate", "up", "down")]   # host descriptor arrays, kept alive here
        return _l.Block(self.input_norm.data_ptr(), self.m["qkv"].c(), self.m["o"].c(), self.post_norm.data_ptr(),
                        _l.Matrix(), _l.Matrix(), self.router.c(), self._arrays[0], self._arrays[1], self._arrays[2])

    def nbytes(self):
        """Bytes one pass streams from this block (dense), or its attention + router part (routed)."""
        return sum(x.nbytes() for x in self.m.values()) + (self.router.nbytes() if self.experts else 0)

    def expert_nbytes(self):
        return sum(self.expert[name][0].nbytes() for name in ("gate", "up", "down")) if self.experts else 0


class DeviceModel:
    def __init__(self, cfg, seed=0, device="cuda:0", tp=None):
        """`cfg` is the whole model's geometry.  With `tp` = (rank, ranks) this object holds that
        rank's tensor-parallel shard and `self.cfg` its local head / FFN counts."""
        self.global_cfg = dict(cfg)
        self.cfg = dict(cfg)
        self.tp = tp
        if tp is not None:
            for key in ("q_heads", "kv_heads", "ffn"):
                self.cfg[key] = cfg[key] // tp[1]
        self.device = torch.device(device)
        H, V = cfg["hidden"], cfg["vocab"]
        with torch.cuda.device(self.device):
            gen = torch.Generator(device=self.device)
            gen.manual_seed(seed * 1000 + 1)
            self.embedding = (torch.randn((V, H), generator=gen, device=self.device, dtype=torch.float32) * 0.02
                              ).to(torch.bfloat16)
            self.layers = [DeviceBlock(cfg, seed * 1000 + 10 + l, self.device, tp=tp) for l in range(cfg["layers"])]
            self.final_norm = torch.ones(H, dtype=torch.float32, device=self.device)
            self.head = quantize(_random_rows(V, H, seed * 1000 + 2, self.device))
            self.mtp_norms = [torch.ones(H, dtype=torch.float32, device=self.device) for _ in range(3)]
            self.mtp_fusion = quantize(_random_rows(H, 2 * H, seed * 1000 + 3, self.device))
            self.mtp_block = DeviceBlock(cfg, seed * 1000 + 4, self.device,
                                         base_seed=seed * 1000 + 10 + cfg["layers"] - 1, tp=tp)
            torch.cuda.empty_cache()

    def config(self):
        c = _l.Config()
        for k, v in self.cfg.items():
            setattr(c, k, v)
        return c

    def provider(self):
        blocks = (_l.Block * len(self.layers))(*[b.c() for b in self.layers])
        w = _l.Weights(self.embedding.data_ptr(), blocks, self.final_norm.data_ptr(), self.head.c(),
                       self.mtp_norms[0].data_ptr(), self.mtp_norms[1].data_ptr(), self.mtp_fusion.c(),
                       self.mtp_block.c(), self.mtp_norms[2].data_ptr())
        return Nvfp4MtpProvider(self.config(), w, weights_on_device=True, device=self.device.index or 0,
                                keepalive=(self, blocks))

    def echo_variant(self):
        """The same weights as a model whose drafts can be right (dense, unsharded): the attention
        and FFN output projections are scaled to almost nothing, so the next token is a function of
        the current token alone, and the fusion matrix passes the normalised embedding through,
        so the draft block sees what the target saw.  Shares every weight tensor with `self`
        (only the per-tensor multipliers of o / down and the fusion matrix differ)."""
        import copy
        assert self.tp is None and not self.cfg.get("experts", 0)
        m = copy.copy(self)

        def quiet(block):
            b = copy.copy(block)
            b.m = dict(block.m)
            for name in ("o", "down"):
                src = block.m[name]
                b.m[name] = DeviceMatrix(src.codes, src.scales, src.weight_scale * 1e-4, src.rows, src.cols)
            return b

        m.layers = [quiet(b) for b in self.layers]
        m.mtp_block = quiet(self.mtp_block)
        H = self.cfg["hidden"]
        with torch.cuda.device(self.device):
            fusion = torch.zeros((H, 2 * H), dtype=torch.float32, device=self.device)
            fusion[torch.arange(H), torch.arange(H)] = 1.0
            m.mtp_fusion = quantize(fusion)
        return m

    def tensor_parallel_provider(self, group=None):
        """Provider of this rank's shard with the exchange areas of all ranks attached: the
        inter-process handles travel through `torch.distributed` (all-gather over `group`)."""
        rank, ranks = self.tp
        provider = self.provider()
        provider.set_gemv_impl(1)
        provider.tp_attach(gather_handles(provider.tp_export(rank, ranks), ranks, group))
        return provider

    # ---- algorithmic bytes (weights streamed once per pass; scales included)
    def verify_weight_bytes(self):
        return sum(b.nbytes() for b in self.layers) + self.head.nbytes()

    def draft_pass_weight_bytes(self):
        V, H = self.cfg["draft_vocab"], self.cfg["hidden"]
        return self.mtp_block.nbytes() + self.mtp_fusion.nbytes() + V * H // 2 + V * H // 16

    def kv_bytes_per_token(self):
        L = _l.load()
        c = self.cfg
        target = L.qllm_k_kv_layer_bytes(c["kv_encoding"], c["page_tokens"], c["kv_heads"], c["head_dim"])
        draft = L.qllm_k_kv_layer_bytes(c["mtp_kv_encoding"], c["page_tokens"], c["kv_heads"], c["head_dim"])
        return target * c["layers"] // c["page_tokens"], draft // c["page_tokens"]

    def expected_distinct_experts(self, rows):
        """Expected number of distinct experts `rows` tokens touch under uniform routing."""
        e, k = self.cfg.get("experts", 0), self.cfg.get("route_width", 0)
        return e * (1.0 - (1.0 - k / e) ** rows) if e else 0.0

    def step_bytes(self, context):
        """Algorithmic bytes of one MTP-4 step at `context` cached tokens: one verify pass
        (all layer weights + head + target cache) and draft_depth draft passes.  For a routed
        model the expert bytes of a pass are those of the distinct experts its rows touch
        (expectation under uniform routing: 5 rows in the verify pass, 1 in a draft pass)."""
        target_kv, draft_kv = self.kv_bytes_per_token()
        verify = self.verify_weight_bytes() + target_kv * context
        draft = self.draft_pass_weight_bytes() + draft_kv * context
        if self.cfg.get("experts", 0):
            per_expert = self.layers[0].expert_nbytes()
            verify += int(self.cfg["layers"] * per_expert * self.expected_distinct_experts(5))
            draft += int(per_expert * self.expected_distinct_experts(1))
        return verify + self.cfg["draft_depth"] * draft, verify
