"""Dense QPack records (host code of the library, no GPU): a pack written by the reference's own
writer is read back, and every corruption of it gets the verdict of the reference's validator
(tests/golden/dense_pack.bin / .json, written by tests/golden/make_pack_golden.py)."""
import ctypes as C
import hashlib
import json
import os

import numpy as np
import pytest

from quantum_llm_b200 import lib as ql

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
META = json.load(open(os.path.join(GOLDEN, "dense_pack.json")))
PACK = open(os.path.join(GOLDEN, "dense_pack.bin"), "rb").read()


def entry_of(e):
    """The index entry as the C structure (a dict shaped like the reference manifest's)."""
    shape = (C.c_uint32 * 5)(*e["source_shape"])
    digest = (C.c_uint8 * 32)(*bytes.fromhex(e["payload_sha256"]))
    return ql.PackEntry(e["name"].encode(), e["offset"], e["stored_bytes"], len(e["source_shape"]), shape,
                        e["sections"]["data"]["offset"], e["sections"]["data"]["bytes"],
                        e["sections"]["scales"]["offset"], e["sections"]["scales"]["bytes"],
                        ql.PACK_DTYPES.get(e["stored_dtype"], 99), digest)


def check(pack, e, verify=1):
    L = ql.load()
    buffer = C.create_string_buffer(pack, len(pack))
    entry = entry_of(e)
    rc = L.qllm_pack_check_dense(buffer, len(pack), C.byref(entry), verify)
    return rc, L.qllm_last_error().decode()


def test_sha256_matches_hashlib():
    L = ql.load()
    rng = np.random.default_rng(0)
    for n in (0, 1, 55, 56, 63, 64, 65, 119, 120, 1000, 4096 + 3):
        data = rng.integers(0, 256, n, dtype=np.uint8).tobytes()
        out = (C.c_uint8 * 32)()
        L.qllm_sha256(C.create_string_buffer(data, max(n, 1)), n, out)
        assert bytes(out) == hashlib.sha256(data).digest(), n
    assert hashlib.sha256(PACK).hexdigest() == META["pack_sha256"] and len(PACK) == META["pack_bytes"]


def test_records_of_the_reference_writer_are_accepted_and_decoded():
    L = ql.load()
    buffer = C.create_string_buffer(PACK, len(PACK))
    base = C.addressof(buffer)
    seen = 0
    for e in META["records"]:
        rc, message = check(PACK, e)
        assert rc == 0, (e["name"], message)
        start = e["offset"] + e["sections"]["data"]["offset"]
        assert hashlib.sha256(PACK[start:start + e["sections"]["data"]["bytes"]]).hexdigest() == e["data_sha256"]
        if e["quant_abi"] != 5:
            continue
        seen += 1
        m, entry = ql.Matrix(), entry_of(e)
        assert L.qllm_pack_nvfp4_matrix(buffer, len(PACK), C.byref(entry), 1, C.byref(m)) == 0, L.qllm_last_error()
        rows, cols = e["source_shape"]
        assert (m.rows, m.cols) == (rows, cols)
        assert m.codes - base == start                     # pointers into the pack, nothing copied
        scales = m.scales - base
        assert scales == e["offset"] + e["sections"]["scales"]["offset"]
        assert hashlib.sha256(PACK[scales:scales + rows * cols // 16]).hexdigest() == e["scale_sha256"]
        # weight scale = 1 / stored divisor (FP32 division), activation scale = stored divisor
        assert np.float32(m.weight_scale) == np.float32(1.0) / np.float32(e["weight_divisor"])
        assert m.input_scale == e["input_divisor"]
    assert seen == 2
    raw = entry_of(META["records"][2])
    m = ql.Matrix()
    assert L.qllm_pack_nvfp4_matrix(buffer, len(PACK), C.byref(raw), 1, C.byref(m)) == -4     # not an NVFP4 record


@pytest.mark.parametrize("case", META["corruptions"], ids=lambda c: c["name"].replace(" ", "_"))
def test_corruptions_get_the_reference_validator_s_verdict(case):
    data = bytearray(PACK)
    base = META["records"][case["record"]]["offset"]
    for offset, raw in case["patches"]:
        raw = bytes.fromhex(raw)
        data[base + offset:base + offset + len(raw)] = raw
    e = json.loads(json.dumps(META["records"][case["record"]]))
    for key, value in case["overrides"].items():
        node, parts = e, key.split(".")
        for part in parts[:-1]:
            node = node[part]
        node[parts[-1]] = value
    rc, message = check(bytes(data), e)
    assert (rc == 0) == case["accepted"], (case["name"], message, case["message"])
    if rc != 0:
        assert rc == -4
        other_encoding = "flags are incomplete" in case["message"] and "NVFP4" not in case["message"]
        if not other_encoding and case["name"] != "abi 9":
            # same rule as the reference (encodings this provider does not read are refused as such)
            assert case["message"].startswith(message), (case["name"], message, case["message"])


def test_payload_check_is_optional():
    bad = bytearray(PACK)
    bad[300] ^= 0xFF
    e = META["records"][0]
    assert check(bytes(bad), e, verify=1)[0] == -4
    assert check(bytes(bad), e, verify=0)[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("impl", [0, 1])
def test_matrix_read_from_the_pack_runs_through_the_gemv(impl):
    # the record's bytes go to the device as they are; the CUDA GEMV over them equals the oracle's
    # GEMV over the same bytes (bit-exact on the CUDA-core path)
    import torch
    from oracle import binding as ob
    L = ql.load()
    e = META["records"][1]    # 32 x 512, BF16 activation divisor
    buffer = C.create_string_buffer(PACK, len(PACK))
    m, entry = ql.Matrix(), entry_of(e)
    assert L.qllm_pack_nvfp4_matrix(buffer, len(PACK), C.byref(entry), 1, C.byref(m)) == 0
    rows, cols = m.rows, m.cols
    base = C.addressof(buffer)
    codes = np.frombuffer(PACK, np.uint8, rows * cols // 2, m.codes - base).reshape(rows, cols // 2).copy()
    scales = np.frombuffer(PACK, np.uint8, rows * cols // 16, m.scales - base).reshape(rows, cols // 16).copy()
    x = np.random.default_rng(3).normal(0, 1, (5, cols)).astype(np.float32)
    want = ob.gemv(ob.matrix(codes, scales, m.weight_scale, m.input_scale), x)
    dc, ds, dx = (torch.from_numpy(a).cuda() for a in (codes, scales, x))
    y = torch.empty((5, rows), dtype=torch.float32, device="cuda")
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(5, rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    cm = ql.Matrix(dc.data_ptr(), ds.data_ptr(), m.weight_scale, m.input_scale, rows, cols)
    rc = L.qllm_k_nvfp4_gemv(C.byref(cm), 0, rows, dx.data_ptr(), y.data_ptr(), 5, ws.data_ptr(), ws_bytes, impl, None)
    assert rc == 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    if impl == 0:
        assert np.array_equal(got, want)
    else:   # tensor-core path: FP32 accumulation order differs -> at most one BF16 step on single values
        assert np.max(np.abs(got - want)) <= 2e-2 * max(1.0, float(np.abs(want).max()))


# ------------------------------------------------------------------ routed-expert records
EXPERT_META = json.load(open(os.path.join(GOLDEN, "expert_pack.json")))
EXPERT_PACK = open(os.path.join(GOLDEN, "expert_pack.bin"), "rb").read()
SECTIONS = ("gate_up_q", "gate_up_scales", "down_q", "down_scales")


def expert_entry_of(e):
    offsets = (C.c_uint64 * 4)(*[e["sections"][s]["offset"] for s in SECTIONS])
    sizes = (C.c_uint64 * 4)(*[e["sections"][s]["bytes"] for s in SECTIONS])
    digest = (C.c_uint8 * 32)(*bytes.fromhex(e["payload_sha256"]))
    return ql.PackExpertEntry(e["layer"], e["expert"], e["offset"], e["stored_bytes"], offsets, sizes,
                              e["decoded_bytes"], digest)


def expert_matrices(pack, e, verify=1):
    L = ql.load()
    buffer = C.create_string_buffer(pack, len(pack))
    entry = expert_entry_of(e)
    gate, up, down = ql.Matrix(), ql.Matrix(), ql.Matrix()
    rc = L.qllm_pack_nvfp4_expert(buffer, len(pack), C.byref(entry), verify, C.byref(gate), C.byref(up), C.byref(down))
    return rc, buffer, {"gate": gate, "up": up, "down": down}


def test_expert_records_of_the_reference_writer_are_accepted_and_decoded():
    assert hashlib.sha256(EXPERT_PACK).hexdigest() == EXPERT_META["pack_sha256"]
    for e in EXPERT_META["records"]:
        rc, buffer, matrices = expert_matrices(EXPERT_PACK, e)
        assert rc == 0, ql.load().qllm_last_error()
        base = C.addressof(buffer)
        for role, m in matrices.items():
            g = e["golden"][role]
            rows, cols = g["shape"]
            assert (m.rows, m.cols) == (rows, cols)
            codes, scales = m.codes - base, m.scales - base
            assert hashlib.sha256(EXPERT_PACK[codes:codes + rows * cols // 2]).hexdigest() == g["codes_sha256"]
            assert hashlib.sha256(EXPERT_PACK[scales:scales + rows * cols // 16]).hexdigest() == g["scale_sha256"]
            assert np.float32(m.weight_scale) == np.float32(1.0) / np.float32(g["weight_divisor"])
            assert m.input_scale == g["input_divisor"]


@pytest.mark.parametrize("case", EXPERT_META["corruptions"], ids=lambda c: c["name"].replace(" ", "_"))
def test_expert_corruptions_get_the_reference_validator_s_verdict(case):
    L = ql.load()
    data = bytearray(EXPERT_PACK)
    base = EXPERT_META["records"][case["record"]]["offset"]
    for offset, raw in case["patches"]:
        raw = bytes.fromhex(raw)
        data[base + offset:base + offset + len(raw)] = raw
    e = json.loads(json.dumps(EXPERT_META["records"][case["record"]]))
    for key, value in case["overrides"].items():
        node, parts = e, key.split(".")
        for part in parts[:-1]:
            node = node[part]
        node[parts[-1]] = value
    buffer = C.create_string_buffer(bytes(data), len(data))
    entry = expert_entry_of(e)
    rc = L.qllm_pack_check_expert(buffer, len(data), C.byref(entry), 1)
    message = L.qllm_last_error().decode()
    assert (rc == 0) == case["accepted"], (case["name"], message, case["message"])
    if rc != 0:
        assert rc == -4
        if not case["name"].startswith(("abi 1", "abi 3", "abi 4")):     # other providers' encodings: refused as such
            assert case["message"].startswith(message), (case["name"], message, case["message"])


def test_expert_payload_check_is_optional():
    bad = bytearray(EXPERT_PACK)
    bad[300] ^= 0xFF
    e = EXPERT_META["records"][0]
    assert expert_matrices(bytes(bad), e, verify=1)[0] == -4
    assert expert_matrices(bytes(bad), e, verify=0)[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("role", ["gate", "up", "down"])
def test_expert_matrices_read_from_the_pack_run_through_the_gemv(role):
    # each projection of a record goes to the device as it lies in the pack; the CUDA-core GEMV
    # over it equals the oracle's GEMV over the same bytes
    import torch
    from oracle import binding as ob
    L = ql.load()
    rc, buffer, matrices = expert_matrices(EXPERT_PACK, EXPERT_META["records"][1])
    assert rc == 0
    m, base = matrices[role], C.addressof(buffer)
    rows, cols = m.rows, m.cols
    codes = np.frombuffer(EXPERT_PACK, np.uint8, rows * cols // 2, m.codes - base).reshape(rows, cols // 2).copy()
    scales = np.frombuffer(EXPERT_PACK, np.uint8, rows * cols // 16, m.scales - base).reshape(rows, cols // 16).copy()
    x = np.random.default_rng(5).normal(0, 1, (5, cols)).astype(np.float32)
    want = ob.gemv(ob.matrix(codes, scales, m.weight_scale, m.input_scale), x)
    dc, ds, dx = (torch.from_numpy(a).cuda() for a in (codes, scales, x))
    y = torch.empty((5, rows), dtype=torch.float32, device="cuda")
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(5, rows, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    cm = ql.Matrix(dc.data_ptr(), ds.data_ptr(), m.weight_scale, m.input_scale, rows, cols)
    rc = L.qllm_k_nvfp4_gemv(C.byref(cm), 0, rows, dx.data_ptr(), y.data_ptr(), 5, ws.data_ptr(), ws_bytes, 0, None)
    assert rc == 0, L.qllm_last_error().decode()
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), want)
