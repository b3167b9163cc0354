"""The multi-replica plumbing of bench.py on CPU: two gloo ranks reduce their timings and
token counts the way a --gpus N run does (slowest rank's time, sum of the units), and the
reference arm prints its line on rank 0 only."""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_gloo_ranks_reduce_times_by_max_and_units_by_sum(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import json, os, sys
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        import bench
        rank = int(os.environ["RANK"])
        dist.init_process_group("gloo")
        times, counts = bench.reduce_over_ranks([10.0 + rank, 7.0 - rank], [100.0 * (rank + 1), 3.0], "cpu")
        dist.barrier()
        dist.destroy_process_group()
        print(json.dumps({{"rank": rank, "times": times, "counts": counts}}))
    """))
    port = _free_port()
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        got = json.loads(out.strip().splitlines()[-1])
        assert got["times"] == [11.0, 7.0]      # max over ranks
        assert got["counts"] == [300.0, 6.0]    # sum over ranks


def test_single_process_reduction_is_the_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_over_ranks([1.5, 2.5], [4.0], "cpu") == ([1.5, 2.5], [4.0])


def test_reference_arm_prints_on_rank_zero_only():
    # --no-cpu-full-step: the arm's one whole 64-layer step takes minutes on a small host
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1",
           "--warmup", "0", "--no-cpu-full-step"]
    quiet = subprocess.run(cmd, env=dict(os.environ, RANK="1", WORLD_SIZE="2"), capture_output=True, text=True,
                           timeout=300, cwd=ROOT)
    assert quiet.returncode == 0 and quiet.stdout.strip() == ""
    first = subprocess.run(cmd, env=dict(os.environ, RANK="0", WORLD_SIZE="2"), capture_output=True, text=True,
                           timeout=300, cwd=ROOT)
    assert first.returncode == 0, first.stderr[-2000:]
    line = json.loads(first.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["unit"] == "tok/s"
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] == line["value"] > 0
    assert line["cpu_baseline"]["whole_model_step"] is None
    assert line["e2e"] == {"value": line["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
