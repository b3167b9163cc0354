"""Generates tests/golden/dense_pack.bin and dense_pack.json: a small dense QPack written by the
REFERENCE's own writer (compiler/expert_pack/writer.py, write_dense_record) from a hand-made
SafeTensors checkpoint: two native NVFP4 matrices (ABI 5; FP32 and BF16 activation divisor), a
raw F32 vector and a raw BF16 matrix (ABI 0).  The JSON holds what the writer reported for each
record (offset, sizes, sections, payload hash) plus the source bytes' digests, i.e. the answers
the library's reader has to reproduce.

    python tests/golden/make_pack_golden.py        # needs the reference tree

"""
import hashlib
import json
import os
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle.binding import REFERENCE_DEFAULT  # noqa: E402
REFERENCE = Path(os.environ.get("QLLM_REFERENCE", REFERENCE_DEFAULT))


def bf16_bytes(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)).tobytes()


def build_checkpoint(root, rng):
    """model.safetensors by hand: 8-byte header length, JSON header, tensor bytes."""
    tensors = {}

    def nvfp4(name, rows, cols, input_dtype):
        tensors[f"{name}.weight"] = ("U8", [rows, cols // 2], rng.integers(0, 256, rows * cols // 2, dtype=np.uint8).tobytes())
        scales = rng.integers(0x18, 0x58, rows * cols // 16, dtype=np.uint8).tobytes()   # finite positive E4M3
        tensors[f"{name}.weight_scale"] = ("F8_E4M3", [rows, cols // 16], scales)
        tensors[f"{name}.weight_scale_2"] = ("F32", [1], struct.pack("<f", 448.0 * 6.0 / float(rng.uniform(0.05, 0.2))))
        divisor = 336.0 if input_dtype == "F32" else 320.0      # 320 is exact in BF16
        raw = struct.pack("<f", divisor) if input_dtype == "F32" else bf16_bytes(np.array([divisor]))
        tensors[f"{name}.input_scale"] = (input_dtype, [1], raw)

    nvfp4("model.layers.0.mlp.down_proj", 48, 64, "F32")
    nvfp4("model.layers.0.self_attn.o_proj", 32, 512, "BF16")
    tensors["model.norm.weight"] = ("F32", [64], rng.normal(1.0, 0.1, 64).astype(np.float32).tobytes())
    tensors["model.embed_tokens.weight"] = ("BF16", [16, 64], bf16_bytes(rng.normal(0, 0.02, (16, 64))))
    header, blob = {}, b""
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    text = json.dumps(header).encode()
    (root / "model.safetensors").write_bytes(struct.pack("<Q", len(text)) + text + blob)
    (root / "config.json").write_text("{}")
    return {name: raw for name, (_, _, raw) in tensors.items()}


# header field -> (byte offset, struct code); the 256-byte header is "<8sHHIIIIIIIIQQQQQ32s32s" + zeros
FIELDS = {"magic": (0, "8s"), "version": (8, "H"), "header_bytes": (10, "H"), "flags": (12, "I"), "quant_abi": (16, "I"),
          "rank": (20, "I"), "dim0": (24, "I"), "dim1": (28, "I"), "dim4": (40, "I"), "record_bytes": (44, "Q"),
          "data_offset": (52, "Q"), "data_bytes": (60, "Q"), "scale_offset": (68, "Q"), "scale_bytes": (76, "Q"),
          "name_hash": (84, "32s"), "payload_hash": (116, "32s"), "padding": (200, "B")}


def corruptions(entries):
    """(name, record index, [(offset inside the record, bytes)], {index entry overrides})"""
    def field(name, value):
        offset, code = FIELDS[name]
        return (offset, struct.pack("<" + code, value))
    nv, nv_bf16, f32, bf16 = 0, 1, 2, 3
    local0 = 48 * 64 // 16
    scale0 = entries[nv]["sections"]["scales"]["offset"]
    scale1 = entries[nv_bf16]["sections"]["scales"]["offset"]
    local1 = 32 * 512 // 16
    out = [("intact", i, [], {}) for i in range(4)]
    out += [
        ("magic", nv, [field("magic", b"EPDENS02")], {}), ("version 2", nv, [field("version", 2)], {}),
        ("header bytes 512", nv, [field("header_bytes", 512)], {}), ("padding byte set", f32, [field("padding", 1)], {}),
        ("not row-major", nv, [field("flags", 4)], {}), ("not symmetric", nv, [field("flags", 1)], {}),
        ("abi 3 on an NVFP4 record", nv, [field("quant_abi", 3)], {}), ("abi 1 on an NVFP4 record", nv, [field("quant_abi", 1)], {}),
        ("abi 6 on a raw record", f32, [field("quant_abi", 6)], {}), ("abi 5 on a raw record", bf16, [field("quant_abi", 5)], {}),
        ("abi 0 on an NVFP4 record", nv, [field("quant_abi", 0)], {}), ("abi 9", f32, [field("quant_abi", 9)], {}),
        ("rank 0", f32, [field("rank", 0)], {}), ("rank 6", f32, [field("rank", 6)], {}),
        ("rank 3 of a matrix", nv, [field("rank", 3)], {}), ("dim4 set", bf16, [field("dim4", 7)], {}),
        ("rows differ", nv, [field("dim0", 47)], {}), ("columns differ", nv, [field("dim1", 80)], {}),
        ("record bytes differ", nv, [field("record_bytes", 8192)], {}),
        ("data offset inside the header", f32, [field("data_offset", 128)], {"sections.data.offset": 128}),
        ("data bytes differ", nv, [field("data_bytes", 1537)], {}),
        ("data bytes differ, index agrees", nv, [field("data_bytes", 1024)], {"sections.data.bytes": 1024}),
        ("data past the record", f32, [field("data_bytes", 8192)], {"sections.data.bytes": 8192}),
        ("scale offset unaligned", nv, [field("scale_offset", scale0 + 16)], {"sections.scales.offset": scale0 + 16}),
        ("scale bytes + 1", nv, [field("scale_bytes", local0 + 9)], {"sections.scales.bytes": local0 + 9}),
        ("scale bytes - 2 (BF16 divisor form)", nv, [field("scale_bytes", local0 + 6)], {"sections.scales.bytes": local0 + 6}),
        ("raw record with a scale section", f32, [field("scale_offset", 512), field("scale_bytes", 4)],
         {"sections.scales.offset": 512, "sections.scales.bytes": 4}),
        ("name hash", nv, [field("name_hash", b"\1" * 32)], {}), ("payload hash", nv, [field("payload_hash", b"\2" * 32)], {}),
        ("payload byte flipped", nv, [(300, b"\xff")], {}), ("padding after the scales flipped", nv, [(4000, b"\x01")], {}),
        ("NaN block scale", nv, [(scale0 + 5, b"\x7f")], {}), ("negative NaN block scale", nv, [(scale0 + 6, b"\xff")], {}),
        ("zero weight divisor", nv, [(scale0 + local0, struct.pack("<f", 0.0))], {}),
        ("negative weight divisor", nv, [(scale0 + local0, struct.pack("<f", -3.0))], {}),
        ("infinite activation divisor", nv, [(scale0 + local0 + 4, struct.pack("<f", float("inf")))], {}),
        ("NaN BF16 activation divisor", nv_bf16, [(scale1 + local1 + 4, b"\xc0\x7f")], {}),
        ("zero BF16 activation divisor", nv_bf16, [(scale1 + local1 + 4, b"\x00\x00")], {}),
        ("other tensor name", nv, [], {"name": "model.layers.1.mlp.down_proj.weight"}),
        ("index shape differs", nv, [], {"source_shape": [64, 48]}), ("index rank differs", f32, [], {"source_shape": [8, 8]}),
        ("index offset unaligned", f32, [], {"offset": 16384 + 256}), ("index size differs", f32, [], {"stored_bytes": 8192}),
        ("index size unaligned", f32, [], {"stored_bytes": 4000}), ("index size tiny", f32, [], {"stored_bytes": 128}),
        ("record of another tensor", bf16, [], {"offset": 16384}),
        ("index data section differs", bf16, [], {"sections.data.bytes": 2047}),
        ("index dtype I64 for F32 bytes", f32, [], {"stored_dtype": "I64", "decoded_bytes": 512}),
        ("index dtype unknown", f32, [], {"stored_dtype": "F16"}),
        ("index payload hash differs", bf16, [], {"payload_sha256": "00" * 32}),
        ("past the end of the pack", bf16, [], {"offset": 24576}),
    ]
    return out


def apply_overrides(entry, overrides):
    e = json.loads(json.dumps(entry))
    for key, value in overrides.items():
        node, parts = e, key.split(".")
        for part in parts[:-1]:
            node = node[part]
        node[parts[-1]] = value
    return e


def corruption_verdicts(pack_path, entries):
    from compiler.expert_pack.errors import ValidationError
    from compiler.expert_pack.validate import validate_dense_record
    original = pack_path.read_bytes()
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "dense.qpack"
        for name, index, patches, overrides in corruptions(entries):
            data = bytearray(original)
            base = entries[index]["offset"]
            for offset, raw in patches:
                data[base + offset:base + offset + len(raw)] = raw
            path.write_bytes(bytes(data))
            entry = apply_overrides(entries[index], overrides)
            try:
                validate_dense_record(path, entry, 4096)
                verdict, message = True, ""
            except ValidationError as error:
                verdict, message = False, str(error)
            out.append({"name": name, "record": index, "patches": [[o, r.hex()] for o, r in patches],
                        "overrides": overrides, "accepted": verdict, "message": message})
    return out


def main():
    sys.path.insert(0, str(REFERENCE))
    from compiler.expert_pack import constants
    from compiler.expert_pack.adapters import NativeNvfp4MatrixSource
    from compiler.expert_pack.safetensors import SafeTensorCheckpoint
    from compiler.expert_pack.writer import write_dense_record

    rng = np.random.default_rng(2024)
    out_bin = ROOT / "tests" / "golden" / "dense_pack.bin"
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp)
        raw = build_checkpoint(root, rng)
        checkpoint = SafeTensorCheckpoint(root)
        T = checkpoint.tensors
        entries = []
        with open(out_bin, "w+b") as handle:
            for base in ("model.layers.0.mlp.down_proj", "model.layers.0.self_attn.o_proj"):
                weight = T[f"{base}.weight"]
                source = NativeNvfp4MatrixSource(weight, T[f"{base}.weight_scale"], T[f"{base}.weight_scale_2"],
                                                 T[f"{base}.input_scale"], (weight.shape[0], weight.shape[1] * 2))
                r = write_dense_record(handle, checkpoint, weight, "dense.qpack", quant_abi=constants.NVFP4_QUANT_ABI_ID,
                                       native_nvfp4=source)
                entries.append(r.entry)
            r = write_dense_record(handle, checkpoint, T["model.norm.weight"], "dense.qpack", preserve_float32=True)
            entries.append(r.entry)
            r = write_dense_record(handle, checkpoint, T["model.embed_tokens.weight"], "dense.qpack",
                                   preserve_bfloat16=True)
            entries.append(r.entry)
    for e in entries:
        name = e["name"]
        e["data_sha256"] = hashlib.sha256(raw[name]).hexdigest()
        if e["quant_abi"] == constants.NVFP4_QUANT_ABI_ID:
            base = name[:-len(".weight")]
            e["scale_sha256"] = hashlib.sha256(raw[f"{base}.weight_scale"]).hexdigest()
            e["weight_divisor"] = struct.unpack("<f", raw[f"{base}.weight_scale_2"])[0]
            divisor = raw[f"{base}.input_scale"]
            e["input_divisor"] = struct.unpack("<f", divisor if len(divisor) == 4 else b"\0\0" + divisor)[0]
    verdicts = corruption_verdicts(out_bin, entries)
    meta = {"corruptions": verdicts, "pack_bytes": out_bin.stat().st_size, "pack_sha256": hashlib.sha256(out_bin.read_bytes()).hexdigest(),
            "header_struct": constants.DENSE_HEADER_STRUCT.format, "records": entries}
    (ROOT / "tests" / "golden" / "dense_pack.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    print(f"{len(entries)} records, {meta['pack_bytes']} bytes -> {out_bin}")


if __name__ == "__main__":
    main()
