"""runtime-model.tsv parsing and capability negotiation (host code of the library, no GPU):
every text of the corpus gets the verdict of the reference's own parser (golden file written
by tests/golden/make_descriptor_golden.py), accepted texts the same canonical dump."""
import ctypes as C
import hashlib
import json
import os
import re

import pytest

from quantum_llm_b200 import lib as ql
from tests import descriptor_text as dt

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "descriptor_cases.json")


def parse(text):
    L = ql.load()
    raw = text.encode()
    handle = C.c_void_p()
    rc = L.qllm_descriptor_parse(raw, len(raw), C.byref(handle))
    if rc != 0:
        assert not handle.value
        return None, L.qllm_last_error().decode()
    return handle, ""


def dump(handle):
    L = ql.load()
    n = L.qllm_descriptor_dump(handle, None, 0)
    out = C.create_string_buffer(n + 1)
    L.qllm_descriptor_dump(handle, out, n + 1)
    return out.value.decode()


def test_corpus_gets_the_reference_parser_s_verdicts():
    golden = json.load(open(GOLDEN))
    cases = dt.all_cases()
    assert [g["name"] for g in golden] == list(cases)
    L = ql.load()
    accepted = 0
    for g in golden:
        text = cases[g["name"]]
        assert hashlib.sha256(text.encode()).hexdigest() == g["sha256"], g["name"]   # same input as the generator's
        handle, message = parse(text)
        assert (handle is not None) == g["accepted"], (g["name"], message, g.get("answer"))
        if handle is None:
            assert message == g["answer"], g["name"]    # same rule, same line number
            continue
        accepted += 1
        got = dump(handle)
        L.qllm_descriptor_destroy(handle)
        if "answer" in g:
            assert got == g["answer"], g["name"]
        else:
            assert hashlib.sha256(got.encode()).hexdigest() == g["answer_sha256"], g["name"]
    assert accepted >= 60 and len(golden) - accepted >= 200


def negotiate(text, **preset):
    L = ql.load()
    handle, message = parse(text)
    assert handle is not None, message
    c = ql.Config()
    for k, v in preset.items():
        setattr(c, k, v)
    rc = L.qllm_descriptor_negotiate(handle, C.byref(c))
    return rc, c, handle


def test_negotiation_fills_the_geometry_of_the_dense_model():
    L = ql.load()
    assert L.qllm_capability_name().decode() == dt.CAPABILITY and L.qllm_capability_abi() == dt.ABI
    rc, c, h = negotiate(dt.text(dt.records(layers=3)), kv_encoding=ql.KV_Q4H, page_tokens=256, split_tokens=256,
                         max_context=32768)
    assert rc == 0, L.qllm_last_error().decode()
    assert (c.layers, c.hidden, c.vocab, c.q_heads, c.kv_heads, c.head_dim, c.rotary_dim) == (3, 256, 4096, 4, 2, 64, 64)
    assert (c.draft_depth, c.draft_vocab, c.ffn, c.activation_bf16, c.mtp_kv_encoding) == (4, 4096, 1024, 1, ql.KV_Q8)
    assert c.eps == pytest.approx(1e-6, rel=1e-6) and c.rope_theta == 1e6
    assert (c.kv_encoding, c.page_tokens, c.split_tokens) == (ql.KV_Q4H, 256, 256)   # the caller's
    assert c.max_context == 8192          # clamped to the model's
    assert c.experts == 0
    assert L.qllm_descriptor_tensor(h, b"fusion_projection") == b"mtp.fc.weight"
    assert L.qllm_descriptor_tensor(h, b"layer.0.query_projection") == b"mtp.layers.0.self_attn.q_proj.weight"
    assert L.qllm_descriptor_tensor(h, b"final_norm") == b"model.norm.weight"     # model-level role
    assert L.qllm_descriptor_tensor(h, b"no_such_role") is None
    L.qllm_descriptor_destroy(h)


def test_negotiation_reads_the_routed_component():
    L = ql.load()
    rc, c, h = negotiate(dt.text(dt.records(routed=True)), max_context=4096)
    assert rc == 0, L.qllm_last_error().decode()
    assert (c.experts, c.route_width, c.expert_ffn, c.route_scale, c.max_context) == (8, 2, 128, 1.0, 4096)
    L.qllm_descriptor_destroy(h)


def _with(recs, kind, n, **changes):
    return dt.text(dt.edit(recs, kind, n, **changes))


@pytest.mark.parametrize("name,text", [
    # the capability has to be the artifact's exact-decode program and a required kernel, with this ABI
    ("other capability", dt.text(dt.records()).replace(dt.CAPABILITY, "decode.mtp.dense-full-attention.fp4-block32.exact.v2")),
    ("no exact-decode program", dt.text([r for r in dt.records() if not r[0].startswith("exact_decode")])),
    # contract of the program's parameters
    ("two source layers", _with(dt.records(), "exact_decode_parameter", 0, f2=2)),
    ("depth differs from emitted - 1", _with(dt.records(), "exact_decode_parameter", 1, f2=3)),
    ("depth above the row limit", dt.text(dt.records(depth=7))),
    ("draft vocabulary above the vocabulary", _with(dt.records(), "exact_decode_parameter", 2, f2=5000)),
    ("draft vocabulary zero", _with(dt.records(), "exact_decode_parameter", 2, f2=0)),
    ("draft cache not Q8", _with(dt.records(), "exact_decode_parameter", 3, f2=0)),
    ("embedding not first", _with(dt.records(), "exact_decode_parameter", 4, f2=0)),
    ("no post norm", _with(dt.records(), "exact_decode_parameter", 5, f2=0)),
    ("parameter missing", dt.text(dt.drop(dt.records(), "exact_decode_parameter", 5))),
    # geometry attributes
    ("no head count", dt.text(dt.drop(dt.records(), "attribute", 0))),
    ("two draft layers", _with(dt.records(), "attribute", 7, f2=2)),
    ("zero-centred norm", dt.text(dt.add_after(dt.records(), "attribute", ["attribute", "zero_centered_norm", 1]))),
    ("shared expert", _with(dt.records(routed=True), "component", 0, f6=1)),
])
def test_negotiation_rejects_contracts_the_provider_does_not_implement(name, text):
    L = ql.load()
    rc, c, h = negotiate(text, max_context=1024, layers=99)
    assert rc == -4, name              # QLLM_INVALID_ARGUMENT, as the reference's prepare step answers
    assert c.layers == 99, name        # the configuration is untouched on refusal
    assert re.search("declare|contract|attribute|supported", L.qllm_last_error().decode()), name
    L.qllm_descriptor_destroy(h)
