"""Host logic of the provider mirror's prompt driver (no GPU): the call order of the reference
runner (moe_vm_runner.cpp:679-778) — a target chunk, then the synchronisation batch that shifts
the same positions by one token, the head's first token before the last batch, drafts produced
by the last batch only — for every way of cutting the prompt."""
import numpy as np
import pytest

from quantum_llm_b200.provider import Nvfp4MtpProvider


class Recorder(Nvfp4MtpProvider):
    def __init__(self, first_token):      # no library, no device
        self.calls, self.first = [], first_token

    def prefill_chunk(self, state, tokens, first_position):
        self.calls.append(("chunk", list(map(int, tokens)), first_position))

    def first_token(self, state, request, sample_position):
        self.calls.append(("first", sample_position))
        return self.first

    def synchronize_exact_decode_batch(self, state, request, next_tokens, first_target_position, produce_final_draft):
        self.calls.append(("sync", list(map(int, next_tokens)), first_target_position, bool(produce_final_draft)))

    def __del__(self):
        pass


@pytest.mark.parametrize("count,chunk_rows,first_position", [(13, 5, 0), (40, 8, 100), (97, 40, 0), (97, 128, 7), (1, 5, 0),
                                                             (128, 128, 0), (129, 128, 0)])
def test_prompt_is_cut_into_chunks_each_followed_by_its_shifted_batch(count, chunk_rows, first_position):
    tokens = np.arange(1000, 1000 + count, dtype=np.uint32)
    p = Recorder(first_token=77)
    assert p.prefill(None, None, tokens, first_position=first_position, chunk_rows=chunk_rows) == 77
    calls, covered = list(p.calls), 0
    while calls:
        kind, chunk, at = calls.pop(0)
        assert kind == "chunk" and at == first_position + covered and 1 <= len(chunk) <= chunk_rows
        assert chunk == list(tokens[covered:covered + len(chunk)])
        last = covered + len(chunk) == count
        if last:
            assert calls.pop(0) == ("first", first_position + count - 1)
        kind, shifted, sync_at, produce = calls.pop(0)
        assert kind == "sync" and sync_at == at and produce == last and len(shifted) == len(chunk)
        want = list(tokens[covered + 1:covered + len(chunk) + 1])
        if last:
            want.append(77)          # the token the head chose closes the shifted stream
        assert shifted == [int(t) for t in want]
        covered += len(chunk)
        assert last or len(chunk) == chunk_rows       # only the last chunk is ragged
    assert covered == count
