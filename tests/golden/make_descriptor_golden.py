"""Generates tests/golden/descriptor_cases.json: runtime-model.tsv texts with the verdict (and,
when accepted, the canonical dump) of the REFERENCE's own parser, compiled from the reference
tree into oracle/_ref/libqllm_ref_descriptor.so by `make -C oracle ref`.

    python tests/golden/make_descriptor_golden.py

Run where the reference tree is present; the JSON it writes is what the tests use."""
import ctypes as C
import json
import os
import hashlib
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from tests import descriptor_text as dt  # noqa: E402


def reference_verdict(lib, text):
    raw = text.encode()
    out = C.create_string_buffer(1 << 16)
    rc = lib.qref_descriptor_parse(raw, len(raw), out, len(out))
    return rc == 0, out.value.decode()


def main():
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libqllm_ref_descriptor.so"))
    lib.qref_descriptor_parse.argtypes = [C.c_char_p, C.c_ulong, C.c_char_p, C.c_ulong]
    out = []
    for name, text in dt.all_cases().items():
        ok, answer = reference_verdict(lib, text)
        # the texts are rebuilt by tests/descriptor_text.py; the digest pins them
        case = {"name": name, "sha256": hashlib.sha256(text.encode()).hexdigest(), "accepted": ok}
        if ok and name.startswith("random_"):   # accepted random edits: the dump's digest is enough
            case["answer_sha256"] = hashlib.sha256(answer.encode()).hexdigest()
        else:
            case["answer"] = answer
        out.append(case)
    path = os.path.join(ROOT, "tests", "golden", "descriptor_cases.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=0, sort_keys=True)
    accepted = sum(c["accepted"] for c in out)
    print(f"{len(out)} cases ({accepted} accepted by the reference) -> {path}")


if __name__ == "__main__":
    main()
