"""Builders of runtime-model.tsv texts for the descriptor tests and their golden generator:
a dense and a routed NVFP4 MTP model in the record grammar of the reference's
runtime/src/model_descriptor.cpp:492-746 (schema 3: layer program, operation program with
explicit data flow, program endpoints, exact_decode program)."""
import struct

CAPABILITY = "decode.mtp.dense-full-attention.nvfp4-block16.exact.v1"
ABI = 2


def f32_bits(x):
    return struct.unpack("<I", struct.pack("<f", x))[0]


def records(layers=2, routed=False, schema=3, depth=4, vocab=4096, hidden=256, draft_vocab=4096):
    """List of records (each a list of fields); join with tabs and newlines via text()."""
    r = [["model", schema, "synthetic.dense.nvfp4", vocab, 8192, hidden],
         ["attribute", "attention_heads", 4], ["attribute", "kv_heads", 2], ["attribute", "head_dim", 64],
         ["attribute", "rotary_dimension", 64], ["attribute", "norm_epsilon_f32_bits", f32_bits(1e-6)],
         ["attribute", "rope_theta_f32_bits", f32_bits(1e6)], ["attribute", "activation_bf16", 1],
         ["attribute", "mtp_layers", 1], ["attribute", "intermediate_size", 1024],
         ["model_tensor", "token_embedding", "model.embed_tokens.weight"],
         ["model_tensor", "final_norm", "model.norm.weight"],
         ["model_tensor", "output_head", "lm_head.weight"],
         ["kernel", "embedding.lookup.v1", 1], ["kernel", "block.full-attention.standard-gqa.v1", 1],
         ["kernel", "ffn.swiglu.nvfp4-block16.v1", 1], ["kernel", "head.linear.v1", 1], ["kernel", CAPABILITY, ABI]]
    if routed:
        r += [["kernel", "router.softmax-topk.v1", 1], ["kernel", "moe.nvfp4-block16.v1", 1],
              ["component", "main", 0, layers, 8, 2, 0, hidden, 128, "moe.nvfp4-block16.v1", 1, 5, 5, "nvfp4-block16"],
              ["component_attribute", "main", "route_scale_f32_bits", f32_bits(1.0)],
              ["router", "main", "router.softmax-topk.v1", 1], ["router_parameter", "main", "normalize", 1]]
    if schema >= 3:
        r += [["program_input", "tokens", "v.tokens", "u32"], ["program_output", "logits", "v.logits", "f32"]]
    for l in range(layers):
        r.append(["layer", l, "block.full-attention.standard-gqa.v1", 1, "main" if routed else "-", l if routed else 0])
        r.append(["layer_parameter", l, "window", 0])
    op = 0
    flows = schema >= 3

    def operation(layer, capability, component="-", component_layer=0, source=None, target=None, tensors=()):
        nonlocal op
        out = [["operation", op, "-" if layer is None else layer, capability, 1, component, component_layer]]
        out.append(["operation_parameter", op, "rows", 5])
        for role, name in tensors:
            out.append(["operation_tensor", op, role, name])
        if flows:
            out.append(["operation_input", op, "x", source[0], source[1]])
            out.append(["operation_output", op, "y", target[0], target[1]])
        op += 1
        return out

    value = ("v.tokens", "u32")
    if schema >= 3:
        r += operation(None, "embedding.lookup.v1", source=value, target=("v.h0", "f32"),
                       tensors=[("table", "model.embed_tokens.weight")])
        value = ("v.h0", "f32")
    for l in range(layers):
        nxt = (f"v.attn{l}", "f32")
        r += operation(l, "block.full-attention.standard-gqa.v1", source=value, target=nxt,
                       tensors=[("query_projection", f"model.layers.{l}.self_attn.q_proj.weight")])
        value = nxt
        if routed:
            nxt = (f"v.route{l}", "f32")
            r += operation(l, "router.softmax-topk.v1", "main", l, source=value, target=nxt)
            value = nxt
            nxt = (f"v.moe{l}", "f32")
            r += operation(l, "moe.nvfp4-block16.v1", "main", l, source=value, target=nxt)
        else:
            nxt = (f"v.ffn{l}", "f32")
            r += operation(l, "ffn.swiglu.nvfp4-block16.v1", source=value, target=nxt)
        value = nxt
    if schema >= 3:
        r += operation(None, "head.linear.v1", source=value, target=("v.logits", "f32"))
        r += [["exact_decode", CAPABILITY, ABI, depth + 1],
              ["exact_decode_parameter", "source_mtp_layers", 1], ["exact_decode_parameter", "draft_depth", depth],
              ["exact_decode_parameter", "draft_vocabulary_size", draft_vocab],
              ["exact_decode_parameter", "mtp_kv_encoding", 1], ["exact_decode_parameter", "embedding_first", 1],
              ["exact_decode_parameter", "post_norm", 1],
              ["exact_decode_tensor", "token_embedding", "model.embed_tokens.weight"],
              ["exact_decode_tensor", "output_head", "lm_head.weight"],
              ["exact_decode_tensor", "fusion_projection", "mtp.fc.weight"],
              ["exact_decode_tensor", "embedding_norm", "mtp.pre_fc_norm_embedding.weight"],
              ["exact_decode_tensor", "hidden_norm", "mtp.pre_fc_norm_hidden.weight"],
              ["exact_decode_tensor", "draft_norm", "mtp.norm.weight"],
              ["exact_decode_tensor", "layer.0.query_projection", "mtp.layers.0.self_attn.q_proj.weight"]]
    return r


def text(recs, newline="\n"):
    return newline.join(["expert-runtime-model-v1"] + ["\t".join(str(f) for f in rec) for rec in recs]) + newline


# ---- test corpus: named edits of the two base texts, and seeded random edits --------------------
import random  # noqa: E402


def edit(recs, kind, n=0, **changes):
    """Copy of recs with field edits on the n-th record of a kind ({field index: value})."""
    out, seen = [list(r) for r in recs], 0
    for r in out:
        if r[0] == kind:
            if seen == n:
                for index, value in changes.items():
                    r[int(index[1:])] = value
                return out
            seen += 1
    raise KeyError(kind)


def drop(recs, kind, n=0):
    out, seen = [], 0
    for r in recs:
        if r[0] == kind:
            seen += 1
            if seen == n + 1:
                continue
        out.append(list(r))
    return out


def add_after(recs, kind, new, n=0):
    out, seen = [], 0
    for r in recs:
        out.append(list(r))
        if r[0] == kind:
            if seen == n:
                out.append(list(new))
            seen += 1
    return out


def named_cases():
    d, m = records(), records(routed=True)
    T = text
    cases = {
        "dense": T(d), "routed": T(m), "dense_crlf": T(d, "\r\n"), "dense_blank_lines": T(d).replace("\n", "\n\n"),
        "schema1": T(records(schema=1)[:-0 or None]), "schema2_dense": T(records(schema=2)),
        "schema2_routed": T(records(schema=2, routed=True)),
        "depth1": T(records(depth=1)), "eight_layers": T(records(layers=8)),
        "empty": "", "header_only": "expert-runtime-model-v1\n", "wrong_header": T(d).replace("model-v1", "model-v2", 1),
        "no_header": T(d).split("\n", 1)[1], "no_model": T(drop(d, "model")),
        "two_models": T(add_after(d, "model", d[0])), "model_short": T([d[0][:5]] + d[1:]),
        "model_schema_4": T(edit(d, "model", f1=4)), "model_schema_0": T(edit(d, "model", f1=0)),
        "model_vocab_0": T(edit(d, "model", f3=0)), "model_vocab_overflow": T(edit(d, "model", f3=2 ** 32)),
        "model_hidden_text": T(edit(d, "model", f5="wide")), "model_plus_sign": T(edit(d, "model", f3="+4096")),
        "model_negative": T(edit(d, "model", f3="-1")), "model_hex": T(edit(d, "model", f3="0x10")),
        "model_space": T(edit(d, "model", f3=" 4096")), "architecture_empty": T(edit(d, "model", f2="")),
        "attribute_duplicate": T(add_after(d, "attribute", d[1])), "attribute_text": T(edit(d, "attribute", f2="many")),
        "attribute_u64_max": T(edit(d, "attribute", f2=2 ** 64 - 1)), "attribute_u64_overflow": T(edit(d, "attribute", f2=2 ** 64)),
        "attribute_extra_field": T(edit(d, "attribute", f2="4\t5")), "attribute_trailing_tab": T(edit(d, "attribute", f2="4\t")),
        "attribute_before_model": T([d[1], d[0]] + d[2:]),
        "tensor_duplicate_role": T(add_after(d, "model_tensor", d[10])), "tensor_empty_name": T(edit(d, "model_tensor", f2="")),
        "unknown_record": T(add_after(d, "model", ["comment", "x"])), "lower_case_kind": T(edit(d, "kernel", f0="Kernel")),
        "kernel_abi_0": T(edit(d, "kernel", f2=0)), "kernel_duplicate": T(add_after(d, "kernel", d[13])),
        "kernel_same_name_other_abi": T(add_after(d, "kernel", ["kernel", "embedding.lookup.v1", 2])),
        "no_kernels": T([r for r in d if r[0] != "kernel"]),
        "exact_twice": T(add_after(d, "exact_decode", [r for r in d if r[0] == "exact_decode"][0])),
        "exact_emitted_1": T(edit(d, "exact_decode", f3=1)), "exact_abi_0": T(edit(d, "exact_decode", f2=0)),
        "exact_unlisted_capability": T(edit(d, "exact_decode", f1="decode.other.v1")),
        "exact_unlisted_abi": T(edit(d, "exact_decode", f2=3)),
        "exact_in_schema_2": T(edit(d, "model", f1=2)),
        "exact_parameter_duplicate": T(add_after(d, "exact_decode_parameter", ["exact_decode_parameter", "draft_depth", 4], 1)),
        "exact_parameter_first": T(add_after(d, "model", ["exact_decode_parameter", "draft_depth", 4])),
        "exact_tensor_first": T(add_after(d, "model", ["exact_decode_tensor", "output_head", "lm_head.weight"])),
        "exact_tensor_duplicate": T(add_after(d, "exact_decode_tensor", ["exact_decode_tensor", "output_head", "other"], 1)),
        "no_layers": T([r for r in d if not r[0].startswith("layer")]),
        "layer_gap": T(edit(d, "layer", 1, f1=2)), "layer_reversed": T(edit(edit(d, "layer", 0, f1=1), "layer", 1, f1=0)),
        "layer_unlisted_block": T(edit(d, "layer", f2="block.other.v1")), "layer_abi_0": T(edit(d, "layer", f3=0)),
        "layer_dense_component_index": T(edit(d, "layer", f5=1)), "layer_unknown_component": T(edit(d, "layer", f4="draft")),
        "layer_parameter_unknown_layer": T(edit(d, "layer_parameter", f1=7)),
        "layer_parameter_duplicate": T(add_after(d, "layer_parameter", ["layer_parameter", 0, "window", 1])),
        "no_operations": T([r for r in d if not r[0].startswith("operation")]),
        "operation_gap": T(edit(d, "operation", 2, f1=9)),
        "operation_layer_backwards": T(edit(edit(d, "operation", 1, f2=1), "operation", 3, f2=0)),
        "operation_layer_uncovered": T(edit(edit(d, "operation", 3, f2=0), "operation", 4, f2=0)),
        "operation_unknown_layer": T(edit(d, "operation", 1, f2=5)),
        "operation_unlisted": T(edit(d, "operation", 1, f3="block.other.v1")),
        "operation_dense_component_index": T(edit(d, "operation", 1, f6=1)),
        "operation_model_level_component": T(edit(m, "operation", 0, f5="main")),
        "operation_parameter_unknown": T(edit(d, "operation_parameter", f1=77)),
        "operation_tensor_duplicate": T(add_after(d, "operation_tensor", ["operation_tensor", 0, "table", "again"])),
        "operation_input_duplicate_port": T(add_after(d, "operation_input", ["operation_input", 0, "x", "v.tokens", "u32"])),
        "operation_no_flow": T([r for r in d if not (r[0] in ("operation_input", "operation_output") and r[1] == 1)]),
        "operation_input_unavailable": T(edit(d, "operation_input", 1, f3="v.nothing")),
        "operation_input_wrong_abi": T(edit(d, "operation_input", 1, f4="f16")),
        "operation_input_from_later": T(edit(d, "operation_input", 1, f3="v.ffn1")),
        "operation_two_producers": T(edit(d, "operation_output", 2, f3="v.attn0")),
        "operation_overwrites_input": T(edit(d, "operation_output", 2, f3="v.tokens", f4="u32")),
        "no_program_input": T(drop(d, "program_input")), "no_program_output": T(drop(d, "program_output")),
        "program_output_unavailable": T(edit(d, "program_output", f2="v.none")),
        "program_output_wrong_abi": T(edit(d, "program_output", f3="f16")),
        "program_input_duplicate_value": T(add_after(d, "program_input", ["program_input", "again", "v.tokens", "u32"])),
        "program_input_duplicate_role": T(add_after(d, "program_input", ["program_input", "tokens", "v.other", "u32"])),
        "schema2_with_endpoints": T(add_after(records(schema=2), "model", ["program_input", "tokens", "v.tokens", "u32"])),
        "schema2_model_level_operation": T(edit(records(schema=2), "operation", 0, f2="-")),
        "schema1_without_operations": T([r for r in records(schema=1) if not r[0].startswith("operation")]),
        "schema2_without_operations": T([r for r in records(schema=2) if not r[0].startswith("operation")]),
        "component_route_wider_than_experts": T(edit(m, "component", f5=9)),
        "component_hidden_mismatch": T(edit(m, "component", f7=128)), "component_layers_0": T(edit(m, "component", f3=0)),
        "component_source_abi_0": T(edit(m, "component", f11=0)), "component_short": T([r[:13] if r[0] == "component" else r for r in m]),
        "component_offset_overflow": T(edit(m, "component", f2=2 ** 64 - 1)), "component_offset_max_ok": T(edit(m, "component", f2=2 ** 64 - 2)),
        "component_twice": T(add_after(m, "component", [r for r in m if r[0] == "component"][0])),
        "component_same_namespace": T(add_after(m, "component", ["component", "draft", 0, 2, 8, 2, 0, 256, 128, "moe.nvfp4-block16.v1", 1, 5, 5, "nvfp4-block16"])),
        "component_unlisted_execution": T(edit(m, "component", f9="moe.other.v1")),
        "component_without_router": T([r for r in m if not r[0].startswith("router")]),
        "router_twice": T(add_after(m, "router", ["router", "main", "router.softmax-topk.v1", 1])),
        "router_unlisted": T(edit(m, "router", f2="router.other.v1")), "router_abi_0": T(edit(m, "router", f3=0)),
        "router_unknown_component": T(edit(m, "router", f1="draft")),
        "router_parameter_before_router": T([r for r in m if r[0] != "router"]),
        "component_attribute_unknown": T(edit(m, "component_attribute", f1="draft")),
        "routed_layer_index_out_of_range": T(edit(m, "layer", 1, f5=2)),
        "routed_layer_without_router_operation": T(edit(m, "operation", 2, f3="ffn.swiglu.nvfp4-block16.v1", f5="-", f6=0)),
        "routed_operation_index_out_of_range": T(edit(m, "operation", 2, f6=5)),
    }
    return cases


def random_cases(count=240, seed=11):
    rng = random.Random(seed)
    cases = {}
    for i in range(count):
        recs = [list(r) for r in records(layers=rng.choice([1, 2, 3]), routed=rng.random() < 0.5,
                                           schema=rng.choice([2, 3, 3, 3]))]
        for _ in range(rng.choice([1, 1, 2])):
            how = rng.choice(["drop", "duplicate", "swap", "number", "field"])
            a = rng.randrange(len(recs))
            if how == "drop":
                del recs[a]
            elif how == "duplicate":
                recs.insert(rng.randrange(len(recs)), list(recs[a]))
            elif how == "swap":
                b = rng.randrange(len(recs))
                recs[a], recs[b] = recs[b], recs[a]
            elif how == "number":
                numeric = [k for k, f in enumerate(recs[a]) if isinstance(f, int)]
                if numeric:
                    k = rng.choice(numeric)
                    recs[a][k] = rng.choice([0, 1, 2, 3, recs[a][k] + 1, 2 ** 32 - 1, 2 ** 32])
            else:
                k = rng.randrange(1, len(recs[a]))
                recs[a][k] = rng.choice(["-", "main", "", "v.h0", "f32", recs[a][k]])
        cases[f"random_{i:03d}"] = text(recs)
    return cases


def all_cases():
    """name -> text, in a fixed order."""
    return {**named_cases(), **random_cases()}
