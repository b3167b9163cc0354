"""Writes tests/golden/full_width_<case>.npz: the CPU oracle's run over the two-layer full-width
models of tests/full_width.py (a 320-token prompt through prefill and draft priming, then six
speculative steps, greedy).  Stored per step: emitted tokens, next token, the drafts proposed for
the following step, and of each of the five verify rows the 64 largest logits (ids and values)
plus every 128th logit; at the end the SHA-256 of every cache page's committed positions.  The GPU test
tests/test_full_width_golden.py replays the same model through the CUDA provider and compares.

    python tests/golden/make_full_width_golden.py [dense27b moe35b echo27b]

Needs about 20 GB of host memory and a few minutes per case; it is not run by the test suite.
"""
import hashlib
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from tests import full_width as fw  # noqa: E402
from tests import synth  # noqa: E402


def run(case):
    t0 = time.time()
    model, digest = fw.build(case)
    cfg = model.cfg
    print(case, "weights", round(time.time() - t0, 1), "s", digest[:16], flush=True)
    session = model.oracle_session()
    request = synth.request(context_limit=cfg["max_context"])
    prompt = fw.prompt(case)
    first = session.prefill(prompt, 8, request)
    print(case, "prefill", round(time.time() - t0, 1), "s first token", first, flush=True)
    out = dict(page_bytes=np.uint64(session.page(0).size), weights_sha256=np.frombuffer(bytes.fromhex(digest), np.uint8), first_token=np.uint32(first),
               initial_drafts=session.drafts().astype(np.uint32), prompt_sha256=np.frombuffer(
                   hashlib.sha256(prompt.tobytes()).digest(), np.uint8))
    emitted, counts, nexts, drafts, top_ids, top_values, samples = [], [], [], [], [], [], []
    position, token = len(prompt), first
    for step in range(fw.STEPS):
        r = session.execute_exact_decode(request, token, position)
        logits = session.last_logits(5)
        e = np.zeros(8, np.uint32)
        e[:r.emitted_count] = r.emitted[:r.emitted_count]
        emitted.append(e)
        counts.append(r.emitted_count)
        nexts.append(r.next_token)
        d = np.zeros(4, np.uint32)
        got = session.drafts()
        d[:len(got)] = got
        drafts.append(d)
        summaries = [fw.row_summary(logits[i]) for i in range(5)]
        top_ids.append(np.stack([s[0] for s in summaries]))
        top_values.append(np.stack([s[1] for s in summaries]))
        samples.append(np.stack([s[2] for s in summaries]))
        position += r.positions_advanced
        token = r.next_token
        print(case, "step", step, "emitted", list(e[:r.emitted_count]), "next", r.next_token, round(time.time() - t0, 1),
              "s", flush=True)
    pages = (position + cfg["page_tokens"] - 1) // cfg["page_tokens"]
    offsets = [session.layer_offset(l) for l in range(cfg["layers"] + 1)]
    out.update(emitted=np.stack(emitted), emitted_count=np.array(counts, np.uint32), next_token=np.array(nexts, np.uint32),
               drafts=np.stack(drafts), top_ids=np.stack(top_ids), top_values=np.stack(top_values),
               samples=np.stack(samples),
               committed=np.uint32(position),
               page_sha256=np.stack([np.frombuffer(hashlib.sha256(fw.committed_page_bytes(
                   session.page(i), cfg, offsets, i, position).tobytes()).digest(), np.uint8) for i in range(pages)]))
    path = os.path.join(ROOT, "tests", "golden", f"full_width_{case}.npz")
    np.savez_compressed(path, **out)
    print(case, "written", path, os.path.getsize(path), "bytes; accepted per step",
          [int(c) - 1 for c in counts], flush=True)


if __name__ == "__main__":
    for name in (sys.argv[1:] or list(fw.CASES)):
        run(name)
