"""Full-width checks on the GPU: the 27B projection widths (hidden 5120, FFN 17408, 40 q / 8 kv
heads of 128, vocabulary 151936) with two layers, where the CPU oracle would take minutes.  The
CUDA-core GEMV (exact integer block arithmetic, bit-equal to the oracle at the small sizes) is
the reference here; the tensor-core GEMV, the CUDA graph and the tensor-core attention have to
agree with it within the stated tolerance, and speculation must not change greedy output."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CONTEXT, REAL, STEPS = 320, 40, 6


def _model(seed=3, layers=2, routed=False):
    from quantum_llm_b200.synthetic import DENSE_27B, MOE_35B, DeviceModel
    cfg = dict(MOE_35B if routed else DENSE_27B, layers=layers, max_context=1024)
    return DeviceModel(cfg, seed=seed), cfg


def _decode(model, cfg, gemv_impl, attention_impl, graph, steps=STEPS):
    from quantum_llm_b200.provider import RequestParameters
    provider = model.provider()
    provider.set_gemv_impl(gemv_impl)
    provider.set_attention_impl(attention_impl)
    provider.set_graph_mode(graph)
    state = provider.create_request_state()
    request = RequestParameters(sampling_seed=7, sampling_temperature_ppm=0, reserved_context_tokens=cfg["max_context"])
    prompt = np.random.default_rng(11).integers(0, cfg["vocab"], CONTEXT, dtype=np.uint32)
    provider.fill_synthetic_kv(state, 0, CONTEXT - REAL, seed=99)
    token = provider.prefill(state, request, prompt[CONTEXT - REAL:], first_position=CONTEXT - REAL, chunk_rows=5)
    position, stream, rows = CONTEXT, [token], []
    for _ in range(steps):
        r = provider.execute_exact_decode(state, request, token, position, cfg["max_context"])
        rows.append(provider.read_logits(5)[0].copy())     # the guaranteed token's row
        stream += r.emitted_tokens[1:] + [r.next_token]
        position += r.positions_advanced
        token = r.next_token
    return stream, np.stack(rows)


@pytest.mark.parametrize("routed", [False, True], ids=["dense27b", "moe35b"])
def test_tensor_core_paths_agree_with_the_exact_path_at_full_width(routed):
    # routed: 128 experts of width 768 at hidden 2048, 32 q / 4 kv heads (group 8)
    model, cfg = _model(routed=routed)
    exact_stream, exact_rows = _decode(model, cfg, gemv_impl=0, attention_impl=0, graph=False)
    # same arithmetic replayed from a CUDA graph: the same bits
    graph_stream, graph_rows = _decode(model, cfg, gemv_impl=0, attention_impl=0, graph=True)
    assert graph_stream == exact_stream and np.array_equal(graph_rows, exact_rows)
    # tcgen05 GEMV + tensor-core attention: 2e-2 max-abs, 1e-3 relative RMS on the logits of the first
    # step (later steps may follow another token after a near-tie)
    # (routed model: the attention stays on the exact kernel here.  Top-8 of 128 router logits is a
    # discontinuous function: a last-bit difference in the attention output that flips one
    # selection moves the logits by tenths, which says nothing about either kernel; the
    # tensor-core attention at this head geometry is checked against the oracle on a dense
    # model in tests/test_gpu_step.py)
    fast_stream, fast_rows = _decode(model, cfg, gemv_impl=1, attention_impl=0 if routed else 1, graph=True)
    assert fast_stream[0] == exact_stream[0]
    a, b = exact_rows[0], fast_rows[0]
    assert np.max(np.abs(a - b)) <= 2e-2
    assert np.sqrt(np.mean((a - b) ** 2)) <= 1e-3 * np.sqrt(np.mean(a ** 2)) + 1e-6
    shared = 0
    while shared < len(exact_stream) and exact_stream[shared] == fast_stream[shared]:
        shared += 1
    assert shared >= 2, (exact_stream, fast_stream)


def test_greedy_output_does_not_depend_on_the_draft_model_at_27b_width():
    from quantum_llm_b200.synthetic import DeviceBlock
    model, cfg = _model()
    want, _ = _decode(model, cfg, gemv_impl=1, attention_impl=1, graph=True)
    # another draft block: other drafts, other accepted counts, the same emitted tokens
    model.mtp_block = DeviceBlock(cfg, 4242, model.device)
    got, _ = _decode(model, cfg, gemv_impl=1, attention_impl=1, graph=True)
    n = min(len(want), len(got))
    assert got[:n] == want[:n]
