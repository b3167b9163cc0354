"""One tensor-parallel rank of tests/test_tensor_parallel.py (launched by torch.distributed.run,
one process per GPU): decodes with its shard of a synthetic model and writes what it produced
to <out_dir>/rank<r>.npz.  The handles of the exchange areas travel over a gloo group."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main(out_dir, generate):
    import torch
    import torch.distributed as dist
    from tests import synth
    from tests.gpu_util import provider_from_synth, request_pair
    from tests.test_tensor_parallel import TP_MODEL, TP_PROMPT
    rank, ranks = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    model = synth.SynthModel(TP_MODEL, seed=3)
    shard = synth.shard_model(model, rank, ranks)
    p = provider_from_synth(shard, device=local)
    p.set_gemv_impl(1)
    mine = p.tp_export(rank, ranks)
    handles = [None] * ranks
    dist.all_gather_object(handles, mine)
    p.tp_attach(b"".join(handles))
    p.set_graph_mode(True)
    prq, _ = request_pair(seed=1234, temperature_ppm=0, context_limit=TP_MODEL["max_context"])
    st = p.create_request_state()
    prompt = synth.prompt(TP_MODEL["vocab"], *TP_PROMPT)
    dist.barrier()   # every rank has mapped its peers before the first exchange
    first = p.prefill(st, prq, prompt, chunk_rows=5)
    stream, rows, pos, tok = [first], [], len(prompt), first
    while len(stream) < generate + 1:
        r = p.execute_exact_decode(st, prq, tok, pos, prq.reserved_context_tokens)
        rows.append(p.read_logits(5)[0].copy())   # the guaranteed token's row: its input is always emitted
        stream += r.emitted_tokens[1:] + [r.next_token]
        pos += r.positions_advanced
        tok = r.next_token
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), stream=np.array(stream[:generate + 1], np.int64),
             rows=np.stack(rows), drafts=np.array([int(t) for t in p.read_drafts(st)], np.int64))
    dist.barrier()   # no rank leaves while a peer may still store into its memory
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1], int(sys.argv[2]))
