"""Generates tests/golden/expert_pack.bin and expert_pack.json: routed-expert QPack records written
by the REFERENCE's own writer (compiler/expert_pack/writer.py, write_expert_record, native NVFP4 /
ABI 5) from a hand-made SafeTensors checkpoint: two experts of hidden 64, intermediate 32.  The
JSON holds the writer's index entries, the digests and divisors of the source tensors, and the
verdict of the reference's validator (compiler/expert_pack/validate.py, validate_expert_record)
on every corruption listed below: the answers the library's reader has to reproduce.

    python tests/golden/make_expert_pack_golden.py        # needs the reference tree

"""
import hashlib
import json
import struct
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
from make_pack_golden import REFERENCE, ROOT, apply_overrides  # noqa: E402

HIDDEN, INTERMEDIATE, EXPERTS, LAYER = 64, 32, 2, 3
ROLES = (("gate", "gate_proj", INTERMEDIATE, HIDDEN), ("up", "up_proj", INTERMEDIATE, HIDDEN),
         ("down", "down_proj", HIDDEN, INTERMEDIATE))


def tensor_base(expert, projection):
    return f"model.layers.{LAYER}.mlp.experts.{expert}.{projection}"


def build_checkpoint(root, rng):
    tensors = {}
    for expert in range(EXPERTS):
        for _, projection, rows, cols in ROLES:
            base = tensor_base(expert, projection)
            tensors[f"{base}.weight"] = ("U8", [rows, cols // 2], rng.integers(0, 256, rows * cols // 2, dtype=np.uint8).tobytes())
            tensors[f"{base}.weight_scale"] = ("F8_E4M3", [rows, cols // 16],
                                               rng.integers(0x18, 0x58, rows * cols // 16, dtype=np.uint8).tobytes())
            tensors[f"{base}.weight_scale_2"] = ("F32", [1], struct.pack("<f", 448.0 * 6.0 / float(rng.uniform(0.05, 0.2))))
            tensors[f"{base}.input_scale"] = ("F32", [1], struct.pack("<f", float(rng.uniform(200.0, 400.0))))
    header, blob = {}, b""
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = {"dtype": dtype, "shape": shape, "data_offsets": [len(blob), len(blob) + len(raw)]}
        blob += raw
    text = json.dumps(header).encode()
    (root / "model.safetensors").write_bytes(struct.pack("<Q", len(text)) + text + blob)
    (root / "config.json").write_text("{}")
    return {name: raw for name, (_, _, raw) in tensors.items()}


# header field -> (byte offset, struct code) of the 256-byte expert header
FIELDS = {"magic": (0, "8s"), "version": (8, "H"), "header_bytes": (10, "H"), "flags": (12, "I"), "quant_abi": (16, "I"),
          "layer": (20, "I"), "expert": (24, "I"), "hidden": (28, "I"), "intermediate": (32, "I"), "fused_rows": (36, "I"),
          "reserved": (40, "I"), "record_bytes": (44, "Q"), "gate_up_q_offset": (52, "Q"), "gate_up_q_bytes": (60, "Q"),
          "gate_up_scales_offset": (68, "Q"), "gate_up_scales_bytes": (76, "Q"), "down_q_offset": (84, "Q"),
          "down_q_bytes": (92, "Q"), "down_scales_offset": (100, "Q"), "down_scales_bytes": (108, "Q"),
          "payload_hash": (116, "32s"), "padding": (180, "B")}


def corruptions(entries):
    """(name, record index, [(offset inside the record, bytes)], {index entry overrides})"""
    def field(name, value):
        offset, code = FIELDS[name]
        return (offset, struct.pack("<" + code, value))
    s = entries[0]["sections"]
    local = HIDDEN * INTERMEDIATE // 16
    gus, ds, dq = s["gate_up_scales"]["offset"], s["down_scales"]["offset"], s["down_q"]["offset"]
    out = [("intact", i, [], {}) for i in range(EXPERTS)]
    out += [
        ("magic", 0, [field("magic", b"EPDENS01")], {}), ("version 2", 0, [field("version", 2)], {}),
        ("header bytes 512", 0, [field("header_bytes", 512)], {}), ("reserved set", 0, [field("reserved", 1)], {}),
        ("padding byte set", 1, [field("padding", 1)], {}),
        ("per-row flag set", 0, [field("flags", 1 | 2 | 4 | 8)], {}), ("not fused", 0, [field("flags", 1 | 4)], {}),
        ("abi 9", 0, [field("quant_abi", 9)], {}), ("abi 0", 0, [field("quant_abi", 0)], {}),
        ("abi 1 with NVFP4 flags", 0, [field("quant_abi", 1)], {}), ("abi 3 with NVFP4 flags", 0, [field("quant_abi", 3)], {}),
        ("abi 4 with NVFP4 flags", 0, [field("quant_abi", 4)], {}),
        ("layer differs", 0, [field("layer", LAYER + 1)], {}), ("expert differs", 1, [field("expert", 0)], {}),
        ("index layer differs", 0, [], {"layer": 0}), ("index expert differs", 0, [], {"expert": 1}),
        ("record bytes differ", 0, [field("record_bytes", 8192)], {}),
        ("fused rows differ", 0, [field("fused_rows", INTERMEDIATE)], {}),
        ("hidden not block-aligned", 0, [field("hidden", 72)], {}), ("hidden differs", 0, [field("hidden", 128)], {}),
        ("intermediate differs", 0, [field("intermediate", 16), field("fused_rows", 32)], {}),
        ("gate+up bytes differ", 0, [field("gate_up_q_bytes", 2047)], {"sections.gate_up_q.bytes": 2047}),
        ("gate+up scale bytes differ", 0, [field("gate_up_scales_bytes", 2 * local + 8)],
         {"sections.gate_up_scales.bytes": 2 * local + 8}),
        ("down bytes differ", 0, [field("down_q_bytes", 2048)], {"sections.down_q.bytes": 2048}),
        ("down scale bytes differ", 0, [field("down_scales_bytes", local)], {"sections.down_scales.bytes": local}),
        ("index section differs", 0, [], {"sections.down_q.offset": dq + 256}),
        ("header section differs", 0, [field("down_q_offset", dq + 256)], {}),
        ("section unaligned", 0, [field("gate_up_scales_offset", gus + 16)], {"sections.gate_up_scales.offset": gus + 16}),
        ("sections overlap", 0, [field("gate_up_scales_offset", 1024)], {"sections.gate_up_scales.offset": 1024}),
        ("sections out of order", 0, [field("down_q_offset", 256)], {"sections.down_q.offset": 256}),
        ("section past the record", 0, [field("down_scales_offset", 4096)], {"sections.down_scales.offset": 4096}),
        ("payload hash", 0, [field("payload_hash", b"\2" * 32)], {}), ("payload byte flipped", 1, [(300, b"\xff")], {}),
        ("padding after the last section flipped", 0, [(ds + local + 8, b"\x01")], {}),
        ("NaN gate block scale", 0, [(gus + 3, b"\x7f")], {}), ("NaN up block scale", 0, [(gus + local + 8 + 3, b"\xff")], {}),
        ("NaN down block scale", 1, [(ds + 7, b"\x7f")], {}),
        ("zero gate weight divisor", 0, [(gus + local, struct.pack("<f", 0.0))], {}),
        ("negative up weight divisor", 0, [(gus + local + 8 + local, struct.pack("<f", -1.0))], {}),
        ("infinite down weight divisor", 0, [(ds + local, struct.pack("<f", float("inf")))], {}),
        ("NaN gate activation divisor", 0, [(gus + local + 4, struct.pack("<f", float("nan")))], {}),
        ("zero up activation divisor", 0, [(gus + local + 8 + local + 4, struct.pack("<f", 0.0))], {}),
        ("negative down activation divisor", 0, [(ds + local + 4, struct.pack("<f", -2.0))], {}),
        ("index decoded bytes differ", 0, [], {"decoded_bytes": 2 * HIDDEN * INTERMEDIATE * 4}),
        ("index payload hash differs", 1, [], {"payload_sha256": "00" * 32}),
        ("index offset unaligned", 1, [], {"offset": 256}), ("index size differs", 0, [], {"stored_bytes": 8192}),
        ("index size unaligned", 0, [], {"stored_bytes": 4000}), ("index size tiny", 0, [], {"stored_bytes": 128}),
        ("record of the other expert", 0, [], {"offset": entries[1]["offset"]}),
        ("past the end of the pack", 1, [], {"offset": entries[1]["offset"] + entries[1]["stored_bytes"]}),
    ]
    return out


def corruption_verdicts(pack_path, entries):
    from compiler.expert_pack.errors import ValidationError
    from compiler.expert_pack.validate import validate_expert_record
    original = pack_path.read_bytes()
    out = []
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "experts.qpack"
        for name, index, patches, overrides in corruptions(entries):
            data = bytearray(original)
            base = entries[index]["offset"]
            for offset, raw in patches:
                data[base + offset:base + offset + len(raw)] = raw
            path.write_bytes(bytes(data))
            entry = apply_overrides(entries[index], overrides)
            try:
                validate_expert_record(path, entry, 4096)
                verdict, message = True, ""
            except ValidationError as error:
                verdict, message = False, str(error)
            out.append({"name": name, "record": index, "patches": [[o, r.hex()] for o, r in patches],
                        "overrides": overrides, "accepted": verdict, "message": message})
    return out


def main():
    sys.path.insert(0, str(REFERENCE))
    from compiler.expert_pack import constants
    from compiler.expert_pack.adapters import ExpertSource, NativeNvfp4MatrixSource
    from compiler.expert_pack.safetensors import SafeTensorCheckpoint
    from compiler.expert_pack.writer import write_expert_record

    rng = np.random.default_rng(2025)
    out_bin = ROOT / "tests" / "golden" / "expert_pack.bin"
    with tempfile.TemporaryDirectory() as tmp:
        root = Path(tmp)
        raw = build_checkpoint(root, rng)
        checkpoint = SafeTensorCheckpoint(root)
        T = checkpoint.tensors
        entries = []
        with open(out_bin, "w+b") as handle:
            for expert in range(EXPERTS):
                native = {}
                for role, projection, rows, cols in ROLES:
                    base = tensor_base(expert, projection)
                    native[role] = NativeNvfp4MatrixSource(T[f"{base}.weight"], T[f"{base}.weight_scale"],
                                                           T[f"{base}.weight_scale_2"], T[f"{base}.input_scale"], (rows, cols))
                source = ExpertSource(LAYER, expert, native["gate"].weight, native["up"].weight, native["down"].weight,
                                      native["gate"], native["up"], native["down"])
                r = write_expert_record(handle, checkpoint, source, "experts.qpack", HIDDEN, INTERMEDIATE,
                                        quant_abi=constants.NVFP4_QUANT_ABI_ID)
                entries.append(r.entry)
    for e in entries:
        e["golden"] = {}
        for role, projection, rows, cols in ROLES:
            base = tensor_base(e["expert"], projection)
            e["golden"][role] = {"codes_sha256": hashlib.sha256(raw[f"{base}.weight"]).hexdigest(),
                                 "scale_sha256": hashlib.sha256(raw[f"{base}.weight_scale"]).hexdigest(),
                                 "weight_divisor": struct.unpack("<f", raw[f"{base}.weight_scale_2"])[0],
                                 "input_divisor": struct.unpack("<f", raw[f"{base}.input_scale"])[0],
                                 "shape": [rows, cols]}
    verdicts = corruption_verdicts(out_bin, entries)
    meta = {"corruptions": verdicts, "pack_bytes": out_bin.stat().st_size,
            "pack_sha256": hashlib.sha256(out_bin.read_bytes()).hexdigest(),
            "header_struct": constants.EXPERT_HEADER_STRUCT.format, "records": entries}
    (ROOT / "tests" / "golden" / "expert_pack.json").write_text(json.dumps(meta, indent=1, sort_keys=True))
    print(f"{len(entries)} records, {meta['pack_bytes']} bytes -> {out_bin}")
    for v in verdicts:
        print(f"  {'ok ' if v['accepted'] else 'BAD'} {v['name']}: {v['message']}")


if __name__ == "__main__":
    main()
