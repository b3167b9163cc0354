"""Tensor-parallel verify: sharding of the projections (CPU), the exchange path with a single
rank (one GPU, bit-exact against the plain path) and two ranks on two GPUs (child processes)."""
import os
import subprocess
import sys

import numpy as np
import pytest

from oracle import binding as ob
from tests import synth

# head_dim 128 and widths such that the local K of o (q_heads/2 * 128) and down (ffn/2) are
# multiples of 256, the tensor-core GEMV's K tile
TP_MODEL = dict(synth.TINY, head_dim=128, rotary_dim=128, q_heads=4, kv_heads=2, ffn=1024, kv_encoding=ob.KV_Q4H)
TP_PROMPT = (96, 7)   # tokens, seed
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shards_partition_the_projections():
    model = synth.SynthModel(TP_MODEL, seed=3)
    c = model.cfg
    q, kv = c["q_heads"] * c["head_dim"], c["kv_heads"] * c["head_dim"]
    shards = [synth.shard_model(model, r, 2) for r in range(2)]
    for s in shards:
        assert s.cfg["q_heads"] == 2 and s.cfg["kv_heads"] == 1 and s.cfg["ffn"] == 512
        assert s.head is model.head and s.mtp_fusion is model.mtp_fusion
    for full, parts in [(model.layers[1], [s.layers[1] for s in shards]),
                        (model.mtp_block, [s.mtp_block for s in shards])]:
        for name in ("codes", "scales"):
            per = 2 if name == "codes" else 16
            a = getattr(full.qkv, name)
            got = [getattr(p.qkv, name) for p in parts]
            assert np.array_equal(np.concatenate([g[:q // 2] for g in got]), a[:q])
            assert np.array_equal(np.concatenate([g[q // 2:q // 2 + kv // 2] for g in got]), a[q:q + kv])
            assert np.array_equal(np.concatenate([g[q // 2 + kv // 2:] for g in got]), a[q + kv:])
            assert np.array_equal(np.concatenate([getattr(p.o, name) for p in parts], axis=1), getattr(full.o, name))
            assert np.array_equal(np.concatenate([getattr(p.down, name) for p in parts], axis=1),
                                  getattr(full.down, name))
            f = c["ffn"]
            gu = getattr(full.gate_up, name)
            assert np.array_equal(np.concatenate([getattr(p.gate_up, name)[:f // 2] for p in parts]), gu[:f])
            assert np.array_equal(np.concatenate([getattr(p.gate_up, name)[f // 2:] for p in parts]), gu[f:])
            assert getattr(parts[0].o, name).shape[1] * per == q // 2
        assert all(p.o.weight_scale == full.o.weight_scale and p.down.weight_scale == full.down.weight_scale
                   for p in parts)


def test_device_shards_match_the_host_rule():
    # the bench's device-side sharding slices the same rows and columns
    import torch
    from quantum_llm_b200 import synthetic
    rng = np.random.default_rng(0)
    cfg = dict(q_heads=4, kv_heads=2, head_dim=32, ffn=64, hidden=32)
    shapes = dict(qkv=(8 * 32, 32), o=(32, 128), gate_up=(128, 32), down=(32, 64))
    full = {}
    for name, (rows, cols) in shapes.items():
        codes = torch.from_numpy(rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8))
        scales = torch.from_numpy(rng.integers(0, 120, (rows, cols // 16), dtype=np.uint8))
        full[name] = synthetic.DeviceMatrix(codes, scales, 0.5, rows, cols)
    parts = [synthetic.shard_block(full, cfg, r, 2) for r in range(2)]
    assert torch.equal(torch.cat([p["o"].codes for p in parts], dim=1), full["o"].codes)
    assert torch.equal(torch.cat([p["down"].scales for p in parts], dim=1), full["down"].scales)
    assert torch.equal(torch.cat([p["qkv"].codes[:64] for p in parts]), full["qkv"].codes[:128])
    assert torch.equal(torch.cat([p["qkv"].codes[64:96] for p in parts]), full["qkv"].codes[128:192])
    assert torch.equal(torch.cat([p["qkv"].codes[96:] for p in parts]), full["qkv"].codes[192:])
    assert torch.equal(torch.cat([p["gate_up"].codes[32:] for p in parts]), full["gate_up"].codes[64:])
    assert parts[1]["o"].cols == 64 and parts[1]["gate_up"].rows == 64 and parts[0]["o"].weight_scale == 0.5


def test_two_gloo_ranks_gather_the_handles_in_rank_order(tmp_path):
    # host side of the attach step on CPU: every rank ends up with [handle of rank 0 | handle of rank 1]
    import json
    import socket
    import textwrap
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import json, os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        from quantum_llm_b200 import synthetic
        from tests import synth
        from tests.test_tensor_parallel import TP_MODEL
        rank = int(os.environ["RANK"])
        dist.init_process_group("gloo")
        mine = bytes([17 * (rank + 1)]) * 64
        both = synthetic.gather_handles(mine, 2)
        shard = synth.shard_model(synth.SynthModel(TP_MODEL, seed=3), rank, 2)
        dist.barrier()
        dist.destroy_process_group()
        print(json.dumps({{"rank": rank, "handles": list(both), "o_cols": shard.layers[0].o.cols,
                          "kv_heads": shard.cfg["kv_heads"]}}))
    """))
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    for proc in procs:
        out, err = proc.communicate(timeout=300)
        assert proc.returncode == 0, err[-2000:]
        got = json.loads(out.strip().splitlines()[-1])
        assert got["handles"] == [17] * 64 + [34] * 64
        assert got["o_cols"] == 256 and got["kv_heads"] == 1


def test_single_rank_gather_needs_no_process_group():
    from quantum_llm_b200 import synthetic
    assert synthetic.gather_handles(b"\x05" * 64, 1) == b"\x05" * 64


def _decode(p, model, generate, graph=True):
    from tests.gpu_util import request_pair
    prq, _ = request_pair(seed=1234, temperature_ppm=0, context_limit=model.cfg["max_context"])
    p.set_graph_mode(graph)
    st = p.create_request_state()
    prompt = synth.prompt(model.cfg["vocab"], *TP_PROMPT)
    first = p.prefill(st, prq, prompt, chunk_rows=5)
    stream, rows, pos, tok = [first], [], len(prompt), first
    while len(stream) < generate + 1:
        r = p.execute_exact_decode(st, prq, tok, pos, prq.reserved_context_tokens)
        rows.append(p.read_logits(5)[0].copy())
        stream += r.emitted_tokens[1:] + [r.next_token]
        pos += r.positions_advanced
        tok = r.next_token
    return stream[:generate + 1], np.stack(rows), [int(t) for t in p.read_drafts(st)]


@pytest.mark.gpu
def test_single_rank_exchange_equals_the_plain_path():
    # ranks = 1: the o and down partials go through the inbox, tickets and sequence counter,
    # with no peer to wait for -> the same bits as the provider without an exchange area
    from tests.gpu_util import provider_from_synth
    model = synth.SynthModel(TP_MODEL, seed=3)
    plain = provider_from_synth(model)
    plain.set_gemv_impl(1)
    want = _decode(plain, model, 24)
    p = provider_from_synth(synth.shard_model(model, 0, 1))
    p.set_gemv_impl(1)
    handle = p.tp_export(0, 1)
    assert len(handle) == 64
    p.tp_attach(handle)
    got = _decode(p, model, 24)
    assert got[0] == want[0] and got[2] == want[2]
    assert np.array_equal(got[1], want[1])


@pytest.mark.gpu
def test_a_peer_that_never_delivers_ends_the_step_with_an_error_not_a_hang():
    # two ranks, one GPU: the "peer" is a zeroed buffer that nobody writes, so the consumer of the
    # first exchange polls until its limit (about a second), sets the kernel error word and every
    # later wait gives up at once.  The step reports QLLM_INTERNAL; the context stays usable.
    import time
    import torch
    from quantum_llm_b200.lib import QllmError
    from tests.gpu_util import provider_from_synth, request_pair
    model = synth.SynthModel(TP_MODEL, seed=3)
    p = provider_from_synth(synth.shard_model(model, 0, 2))
    p.set_gemv_impl(1)
    p.tp_export(0, 2)
    silent = torch.zeros(p.tp_area_bytes(), dtype=torch.uint8, device="cuda")
    p.tp_attach_local([0, silent.data_ptr()])
    prq, _ = request_pair(context_limit=model.cfg["max_context"])
    st = p.create_request_state()
    t0 = time.time()
    with pytest.raises(QllmError) as failure:
        p.prefill(st, prq, synth.prompt(model.cfg["vocab"], *TP_PROMPT), chunk_rows=5)
    assert time.time() - t0 < 60.0
    assert "device" in str(failure.value) or "failed" in str(failure.value)
    # the device still answers: a plain provider on the same GPU decodes as usual
    torch.cuda.synchronize()
    plain = provider_from_synth(model)
    plain.set_gemv_impl(1)
    stream, _, _ = _decode(plain, model, 4)
    assert len(stream) == 5


@pytest.mark.gpu
def test_exchange_needs_the_tensor_core_gemv_and_an_attached_area():
    from quantum_llm_b200.lib import QllmError
    from tests.gpu_util import provider_from_synth
    model = synth.SynthModel(TP_MODEL, seed=3)
    p = provider_from_synth(synth.shard_model(model, 0, 2))
    p.set_gemv_impl(1)
    p.tp_export(0, 2)
    with pytest.raises(QllmError):   # peers not attached
        _decode(p, model, 4, graph=False)
    with pytest.raises(QllmError):   # second area
        p.tp_export(0, 2)


@pytest.mark.gpu
def test_two_ranks_on_two_gpus_agree_with_one_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from tests.gpu_util import provider_from_synth
    generate = 24
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29731", os.path.join(ROOT, "tests", "tp_worker.py"), str(tmp_path),
           str(generate)]
    done = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(2)]
    # every rank sums the same partials in the same order: identical rows, tokens and drafts
    assert np.array_equal(ranks[0]["stream"], ranks[1]["stream"])
    assert np.array_equal(ranks[0]["rows"], ranks[1]["rows"])
    assert np.array_equal(ranks[0]["drafts"], ranks[1]["drafts"])
    # against the unsharded model on one GPU: other FP32 summation order inside o and down ->
    # logits within 2e-2 max-abs and 1e-3 relative RMS while the token streams agree
    model = synth.SynthModel(TP_MODEL, seed=3)
    plain = provider_from_synth(model)
    plain.set_gemv_impl(1)
    stream, rows, _ = _decode(plain, model, generate)
    shared = 0
    while shared < len(stream) and stream[shared] == ranks[0]["stream"][shared]:
        shared += 1
    assert shared >= 8, (stream, ranks[0]["stream"])
    # the first step's first row has the same inputs on both sides (same first token, same cache).
    # Both sides round to BF16 after sums taken in different orders, so single values move by a
    # BF16 step: each is within the parity tolerance of the oracle, the two of each other within
    # 2e-2 max-abs and a few 1e-3 relative RMS.
    assert stream[0] == ranks[0]["stream"][0]
    a, b = rows[0], ranks[0]["rows"][0]
    assert np.max(np.abs(a - b)) <= 2e-2
    assert np.sqrt(np.mean((a - b) ** 2)) <= 5e-3 * np.sqrt(np.mean(a ** 2))
