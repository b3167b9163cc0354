"""Benchmark of the MTP-4 speculative decode step on B200.

Workload (N=1): 27B-class dense target, NVFP4 weights, one stream, 32768 cached
tokens, Q4H target cache + Q8 draft cache, 4 drafts per step.  One "step" is one
execute_exact_decode: verify 5 rows, accept/rollback on the device, 4 draft passes.
`value` is decode tok/s with everything resident in HBM (steps enqueued back to back,
one read at the end); `e2e` is the same through the provider's per-step call with the
invocation cursor uploaded and the result record read back every step.
N>1 runs N independent replicas (one stream per GPU, data parallel, no collective).
`--model moe35b` runs the same step on the 35B-A3B-class routed model (48 layers, 128 experts,
8 per token) at 8192 cached tokens; `--streams S` steps S independent requests in turn on each
GPU (their rows are not batched into one pass).  `--parallelism tp` shards ONE stream's model
over the N GPUs instead (q/k/v heads and FFN columns per rank, partial sums of the o and down
projections exchanged through peer memory inside the GEMV kernel).

N > 1 on the dense model with one stream defaults to the tensor-parallel form; `--parallelism dp`
asks for replicas.  The line also carries `verify_step` (the verify pass alone against the HBM
roofline, the quantity the 60 % target is stated on) and `echo_model_leg` (the same step on a model
whose drafts can be accepted).

`--microbench` times the tensor-core GEMV alone on the verify-step projection shapes at
M = 5, 40, 128, 160, 640 rows (one JSON line per shape and M).  `--prefill-bench TOKENS` times the
prompt path (target chunks of `--chunk-rows` rows + draft priming, host tokens in, first token out).

  python bench.py --gpus N --steps K --warmup W [--impl reference]
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONTEXT = 32768          # cached tokens when the timed region starts
MOE_CONTEXT = 8192       # the routed model's configuration
REAL_PREFILL = 40        # last prompt tokens run through the real prefill path
METRIC = "decode_tok_per_s_mtp4_q4h_32k"
VERIFY_TARGET_FRAC = 0.60   # the stated target: the verify pass at 60 % of the HBM roofline


def captured_dram_bytes(n, k, m):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch of the tensor-core GEMV on an
    N x K matrix at M rows, from the committed table of ncu captures (profiles/, rows
    `| N | K | M | bytes | ...`); None when that shape was never captured."""
    try:
        text = open(os.path.join(ROOT, "profiles", "nvfp4_gemv_dram_traffic_by_shape.md")).read()
    except OSError:
        return None
    for row in text.splitlines():
        cells = [c.strip() for c in row.strip().strip("|").split("|")]
        if len(cells) >= 4 and cells[0].isdigit():
            if (int(cells[0]), int(cells[1]), int(cells[2])) == (n, k, m):
                return float(cells[3].replace(" ", "").replace(",", ""))
    return None


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemv-impl", type=int, default=int(os.environ.get("QLLM_GEMV_IMPL", "1")))
    ap.add_argument("--attention-impl", type=int, default=int(os.environ.get("QLLM_ATTENTION_IMPL", "1")),
                    help="Q4H attention kernel: 1 = INT8 mma.sync, 2 = tcgen05 with tensor-memory accumulators")
    ap.add_argument("--small", action="store_true", help="4-layer model for profiler captures")
    ap.add_argument("--model", default="dense27b", choices=["dense27b", "moe35b"],
                    help="dense27b: the headline workload; moe35b: the routed 35B-A3B-class target")
    ap.add_argument("--parallelism", default=None, choices=["dp", "tp"],
                    help="N > 1: tp = ONE stream whose model is sharded over the N GPUs (tensor parallel, strong "
                         "scaling; the default for dense27b with one stream, N = 2, 4 or 8); dp = N independent "
                         "replicas (weak scaling; the default for the routed model and for several streams)")
    ap.add_argument("--no-echo-leg", action="store_true",
                    help="skip the extra leg on the echo model (drafts that can be accepted)")
    ap.add_argument("--streams", type=int, default=1, help="independent requests per GPU, stepped in turn")
    ap.add_argument("--context", type=int, default=0, help="cached tokens (0: 32768 dense, 8192 routed)")
    ap.add_argument("--kv-encoding", default="q4h", choices=["q4h", "f16"],
                    help="target KV cache: Q4H (the headline metric) or exact F16 (metric ..._f16kv_32k)")
    ap.add_argument("--split-tokens", type=int, default=0,
                    help="cached tokens per attention CTA (multiple of 64; 0 = the model configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cpu-full-step", action="store_true",
                    help="skip the one whole 64-layer step of the CPU port (half a minute of host time)")
    ap.add_argument("--microbench", action="store_true",
                    help="kernel microbenchmark of the NVFP4 GEMV on the verify-step shapes at M = 5, 40, 128, 160, 640")
    ap.add_argument("--prefill-bench", type=int, default=0, metavar="TOKENS",
                    help="time the prompt path (target chunks + draft priming) over TOKENS prompt tokens")
    ap.add_argument("--chunk-rows", type=int, default=128, help="rows per prompt chunk of --prefill-bench (1..128)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step kernel by kernel instead of replaying a CUDA graph (profiler captures)")
    args = ap.parse_args()
    if not args.context:
        args.context = CONTEXT if args.model == "dense27b" else MOE_CONTEXT
    if args.parallelism is None:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        args.parallelism = "tp" if (world in (2, 4, 8) and args.model == "dense27b" and args.streams == 1 and
                                    args.gemv_impl == 1) else "dp"
    return args


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = max(mx, float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


class OracleSteps:
    """The CPU arm's bounded sample of the workload: REAL speculative steps of the reference's
    arithmetic (the oracle port: verify over 5 rows, acceptance, rollback, 4 draft passes) on a
    model with the workload's widths, vocabulary, context length and cache encodings, but `layers`
    of its target layers (a full 64-layer step takes minutes on the host).  Weights are random
    NVFP4 bytes (valid E2M1 codes, E4M3 scales in [0.125, 2)), the cached prefix is the seeded
    synthetic records the GPU arm uses, the last 8 prompt tokens run for real.  Nothing is scaled:
    the reported rate is that of the sliced model, and the slice is named in the JSON line."""

    def __init__(self, cfg, context, layers=2, threads=None, share_layer_bytes=False):
        import numpy as np
        from oracle import binding as ob
        self.ob, self.O = ob, ob.lib()
        # explicit: launchers such as torchrun export OMP_NUM_THREADS=1
        self.O.qo_set_threads(threads or len(os.sched_getaffinity(0)) or 1)
        self.threads = int(self.O.qo_max_threads())
        rng = np.random.default_rng(0)
        self.cfg = dict(cfg, layers=layers, max_context=context + 1024)
        c = self.cfg
        H, F, V = c["hidden"], c["ffn"], c["vocab"]
        keep = self.keep = []

        def matrix(rows, cols):
            codes = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
            scales = rng.integers(0x20, 0x40, (rows, cols // 16), dtype=np.uint8)
            keep.extend((codes, scales))
            return ob.matrix(codes, scales, 2e-3, 336.0)

        def ones():
            v = np.ones(H, np.float32)
            keep.append(v)
            return ob._ptr(v)

        def block():
            qkv_rows = (c["q_heads"] + 2 * c["kv_heads"]) * c["head_dim"]
            return ob.Block(ones(), matrix(qkv_rows, H), matrix(H, c["q_heads"] * c["head_dim"]), ones(),
                            matrix(2 * F, H), matrix(H, F))

        # BF16 embedding rows of magnitude ~0.01 with random signs
        embedding = (rng.integers(0x3c00, 0x3d00, (V, H), dtype=np.uint16) |
                     (rng.integers(0, 2, (V, H), dtype=np.uint16) << 15))
        keep.append(embedding)
        # share_layer_bytes: every target layer points at ONE layer's random bytes.  The arithmetic and
        # the memory traffic per layer are those of distinct layers (a layer is 186 MB, far beyond any
        # last-level cache), the host needs 0.2 GB instead of 12 GB and no minute of random-number
        # generation -- which is what lets a whole 64-layer step be timed for real.
        if share_layer_bytes:
            one = block()
            blocks = (ob.Block * layers)(*[one for _ in range(layers)])
        else:
            blocks = (ob.Block * layers)(*[block() for _ in range(layers)])
        weights = ob.Weights(ob._ptr(embedding), blocks, ones(), matrix(V, H), ones(), ones(), matrix(H, 2 * H),
                             block(), ones())
        config = ob.Config()
        for k, v in c.items():
            if hasattr(config, k):
                setattr(config, k, v)
        self.session = ob.Session(config, weights, (keep, blocks))
        self.request = ob.Request(1, 0, 950000, 20, 0, c["max_context"], 2000000)
        real = 8
        self.session.fill_synthetic_kv(0, context - real, 1234)
        prompt = rng.integers(0, V, real, dtype=np.uint32)
        self.token = self.session.prefill_at(prompt, context - real, 8, self.request)
        self.position = context
        self.context = context
        self.description = (f"real speculative steps of the oracle port on a {layers}-layer slice of the "
                            f"{cfg['layers']}-layer model (full widths, vocabulary and {context}-token Q4H/Q8 caches; "
                            f"nothing scaled)") if layers != cfg["layers"] else (
            f"a real speculative step of the oracle port on all {layers} layers (full widths, vocabulary and "
            f"{context}-token Q4H/Q8 caches; the layers share one layer's random weight bytes, 186 MB per layer "
            f"streamed from memory each time)")

    def step(self):
        """One speculative step; returns (seconds, tokens emitted)."""
        t0 = time.perf_counter()
        r = self.session.execute_exact_decode(self.request, self.token, self.position)
        seconds = time.perf_counter() - t0
        self.position += r.positions_advanced
        self.token = r.next_token
        return seconds, int(r.positions_advanced)


def reference_cpu_ffn(cfg, threads):
    """Second CPU figure: the reference's OWN host code (Fp4HostExecutor, runtime/src/cpu/
    fp4_host_executor.cpp, compiled unmodified into oracle/_ref) running one FFN layer of the
    workload's widths over the 5 verify rows.  Its weight format is the reference's CPU-lane FP4
    (E2M1 with one UE8M0 scale per 32 values, Q8 activations), not NVFP4 block-16, so this is a
    throughput figure for the same layer shape, not the same arithmetic.  None when not built."""
    import ctypes as C
    from oracle import binding as ob
    R = ob.ref_fp4_host()
    if R is None:
        return None
    H, F, rows, threads = cfg["hidden"], cfg["ffn"], cfg["draft_depth"] + 1, max(1, min(int(threads), 64))
    checksum = C.c_double(0.0)
    seconds = R.ref_fp4_host_ffn_seconds(H, F, rows, threads, 20, 7, C.byref(checksum))
    if not seconds > 0.0:
        return None
    layer_bytes = 3 * H * F * 17 // 32          # 4-bit codes + one scale byte per 32
    return {"kind": "_ref", "what": "Fp4HostExecutor, one SwiGLU FFN layer (gate, up, down) of the workload's widths, "
            f"{rows} rows, FP4 block-32 weights (the reference's CPU lane format), mean of 20 runs",
            "ms_per_ffn_layer": seconds * 1e3, "gb_per_s": layer_bytes / seconds / 1e9, "cores": threads,
            "gpu_ffn_layer_note": "the GPU path's FFN layer at the same widths is the gate/up GEMV + SiLU + down GEMV"}


def reference_cpu_acceptance():
    """The reference's OWN sampler code (runtime/src/speculative_sampling.cpp, compiled unmodified
    into oracle/_ref) making the acceptance decisions of a speculative step on the host: five target
    and four draft distributions over 20 sorted candidates, up to four rejection decisions, the bonus
    sample.  The GPU path does this in one kernel on the device.  None when not built."""
    import ctypes as C
    from oracle import binding as ob
    R = ob.ref_sampler()
    if R is None or not hasattr(R, "ref_acceptance_seconds_per_step"):
        return None
    accepted = C.c_uint64(0)
    seconds = R.ref_acceptance_seconds_per_step(20000, 20, 7, C.byref(accepted))
    if not seconds > 0.0:
        return None
    return {"kind": "_ref", "what": "make_sampling_distribution x 9 + rejection_sample x <= 4 + bonus sample per step, "
            "top_k 20, 20000 steps on one thread", "us_per_step": seconds * 1e6, "cores": 1,
            "accepted_per_step": accepted.value / 20000.0}


def algorithmic_step_bytes(cfg, context):
    """Bytes one MTP-4 step must read: verify weights + target KV + 4 draft passes."""
    nv = lambda r, c: r * c * 9 // 16   # NVFP4: 4-bit codes + one E4M3 scale per 16
    per_layer = (nv((cfg["q_heads"] + 2 * cfg["kv_heads"]) * cfg["head_dim"], cfg["hidden"]) +
                 nv(cfg["hidden"], cfg["q_heads"] * cfg["head_dim"]) + nv(2 * cfg["ffn"], cfg["hidden"]) +
                 nv(cfg["hidden"], cfg["ffn"]))
    head = nv(cfg["vocab"], cfg["hidden"])
    kv = 2 * (cfg["head_dim"] // 2 + 2) * cfg["kv_heads"] * cfg["layers"] * context
    draft = per_layer + nv(cfg["hidden"], 2 * cfg["hidden"]) + nv(cfg["draft_vocab"], cfg["hidden"]) \
        + 2 * (cfg["head_dim"] + 2) * cfg["kv_heads"] * context
    return per_layer * cfg["layers"] + head + kv + 4 * draft


def workload_name(context, kv="q4h", model="dense27b", streams=1):
    arch = ("27B dense (64L, h5120, 40q/8kv, hd128, ffn17408, vocab151936)" if model == "dense27b" else
            "35B-A3B routed (48L, h2048, 32q/4kv, hd128, 128 experts x ffn768, 8 per token, vocab151936)")
    per_gpu = "1 stream/GPU" if streams == 1 else f"{streams} streams/GPU stepped in turn (rows not batched)"
    return (f"{arch}, {per_gpu}, "
            f"{context} cached tokens, {'exact F16' if kv == 'f16' else 'Q4H'} target KV + Q8 draft KV, MTP-4, greedy")


REFERENCE_LAYERS = 2     # target layers of the slice the CPU arm steps through


def reference_arm(args):
    """Reference arm: the reference's arithmetic for this path on the host cores.  The reference's
    own provider needs a CUDA device and a compiled model artifact, so its CPU implementation of
    the path is the oracle port (kind "port").  Every step is a real speculative step of the
    sliced model (OracleSteps); `value` is what was measured, for the slice named in `config`."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    assert args.model == "dense27b" and args.streams == 1, "the reference arm times the headline workload only"
    from quantum_llm_b200.synthetic import DENSE_27B
    sample = OracleSteps(DENSE_27B, args.context, REFERENCE_LAYERS)
    for _ in range(args.warmup):
        sample.step()
    seconds, tokens = 0.0, 0
    for _ in range(args.steps):
        s, n = sample.step()
        seconds += s
        tokens += n
    value = tokens / seconds
    text = f"{sample.description}; {args.steps} timed steps on {sample.threads} threads"
    threads = sample.threads
    del sample
    whole_step = None
    if not args.no_cpu_full_step:   # one whole step of all 64 layers, measured
        whole_model = OracleSteps(DENSE_27B, args.context, DENSE_27B["layers"], share_layer_bytes=True)
        step_seconds, step_tokens = whole_model.step()
        whole_step = {"value": step_tokens / step_seconds, "unit": "tok/s", "seconds_per_step": step_seconds,
                      "cores": whole_model.threads, "kind": "port", "sample": whole_model.description}
        del whole_model
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4xnvfp4->f32",
            "data": "synthetic",
            "config": {"workload": workload_name(args.context), "layers": REFERENCE_LAYERS,
                       "layers_of_the_model": DENSE_27B["layers"],
                       "parallelism": "host cores of rank 0", "implementation": "CPU port of the reference arithmetic"},
            "accepted_len_per_step": tokens / args.steps,
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": text,
                             "whole_model_step": whole_step,
                             "reference_ffn": reference_cpu_ffn(DENSE_27B, threads),
                             "reference_acceptance": reference_cpu_acceptance()},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def reduce_over_ranks(times_ms, counts, device):
    """Whole-job figures of a replica run: the slowest rank's device times (MAX) and the
    units all ranks processed (SUM).  A single process returns its own numbers."""
    import torch
    import torch.distributed as dist
    t = torch.tensor(times_ms, dtype=torch.float64, device=device)
    c = torch.tensor(counts, dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(c, op=dist.ReduceOp.SUM)
    return [float(x) for x in t.cpu()], [float(x) for x in c.cpu()]


def gemv_kernel_leg(model, provider, gemv_impl, rows=5, repeats=3, name="gate_up"):
    """Average duration of the dominant kernel (gate/up NVFP4 GEMV, 34816x5120, 5 rows) over
    all layers' weights back to back (6.4 GB, far beyond L2), timed with CUDA events on the
    launching stream.  (`name` picks another of the layers' matrices.)"""
    import torch
    from quantum_llm_b200 import lib as ql
    L = ql.load()
    dev = model.device
    mats = [b.m[name] for b in model.layers]
    rows_w, cols = mats[0].rows, mats[0].cols
    x = torch.randn((rows, cols), device=dev, dtype=torch.float32)
    y = torch.empty((rows, rows_w), device=dev, dtype=torch.float32)
    ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(rows, rows_w, cols)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(device=dev)
    handles = []
    for m in mats:   # load-time preparation (TMA descriptor, re-tiled scales), outside the timing
        h, cm = C.c_void_p(), m.c()
        ql.check(L.qllm_k_matrix_prepare(C.byref(cm), C.c_void_p(stream.cuda_stream), C.byref(h)))
        handles.append(h)
    stream.synchronize()
    best = None
    sp = C.c_void_p(stream.cuda_stream)
    with torch.cuda.stream(stream):
        # one full call quantises the activations into the workspace; the timed launches are
        # the GEMV kernel alone (tensor-core path), as it runs between the fused kernels
        ql.check(L.qllm_k_nvfp4_gemv_prepared(handles[0], x.data_ptr(), y.data_ptr(), rows, ws.data_ptr(), ws_bytes,
                                             gemv_impl, sp))
        for rep in range(repeats + 1):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for h in handles:
                if gemv_impl == 1:
                    ql.check(L.qllm_k_nvfp4_gemv_prepared_core(h, rows, ws.data_ptr(), ws_bytes, sp))
                else:
                    ql.check(L.qllm_k_nvfp4_gemv_prepared(h, x.data_ptr(), y.data_ptr(), rows, ws.data_ptr(),
                                                         ws_bytes, gemv_impl, sp))
            stop.record(stream)
            stop.synchronize()
            ms = start.elapsed_time(stop) / len(handles)
            if rep > 0:
                best = ms if best is None else min(best, ms)
    for h in handles:
        L.qllm_k_matrix_release(h)
    algorithmic = mats[0].nbytes() + rows * cols * 2 + rows * rows_w * 4  # weights + bf16-valued rows in + fp32 out
    return best, algorithmic


def ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from quantum_llm_b200 import build as qbuild
    if local == 0:
        qbuild.build()
    if world > 1:
        dist.barrier()
    from quantum_llm_b200.provider import RequestParameters
    from quantum_llm_b200.synthetic import DENSE_27B, MOE_35B, DeviceModel

    routed = args.model == "moe35b"
    cfg = dict(MOE_35B if routed else DENSE_27B)
    tensor_parallel = args.parallelism == "tp"   # world == 1: the exchange path without peers
    assert not (tensor_parallel and (routed or args.gemv_impl != 1)), "tensor parallelism: dense27b, tcgen05 GEMV"
    # tensor parallel: every rank works on the same request (same seeds); replicas: one per rank
    replica = 0 if tensor_parallel else rank
    if args.small:
        cfg["layers"] = 4
    context = args.context
    cfg["max_context"] = context + 1024
    if args.split_tokens:
        cfg["split_tokens"] = args.split_tokens
    if args.kv_encoding == "f16":   # exact-F16 target cache (262144 B/token instead of 67584)
        from quantum_llm_b200 import lib as _ql
        cfg["kv_encoding"] = _ql.KV_F16
    steps_total = args.warmup + 2 * args.steps + 32
    assert context + 5 * steps_total + 16 < cfg["max_context"], "too many steps for the context reserve"
    if tensor_parallel:
        model = DeviceModel(cfg, seed=0, device=f"cuda:{local}", tp=(rank, world))
        provider = model.tensor_parallel_provider()
        if world > 1:
            dist.barrier()   # every rank has mapped its peers' exchange areas
    else:
        model = DeviceModel(cfg, seed=rank, device=f"cuda:{local}")
        provider = model.provider()
    provider.set_gemv_impl(args.gemv_impl)
    provider.set_attention_impl(args.attention_impl)
    request = RequestParameters(sampling_seed=1 + replica, sampling_temperature_ppm=0,
                                reserved_context_tokens=cfg["max_context"])
    synthetic = context - REAL_PREFILL

    class Stream:
        """One independent request: its own caches, cursor and (per-state) step graph."""
        def __init__(self, index):
            # prompt: seeded uniform ids; the first context-REAL_PREFILL positions are represented by
            # seeded synthetic cache records, the tail goes through the real prefill + draft priming
            seed = 1 + replica * args.streams + index
            prompt = np.random.default_rng(seed).integers(0, cfg["vocab"], context, dtype=np.uint32)
            self.state = provider.create_request_state()
            provider.fill_synthetic_kv(self.state, 0, synthetic, seed=1233 + seed)
            self.token = provider.prefill(self.state, request, prompt[synthetic:], first_position=synthetic,
                                          chunk_rows=5)
            self.position = context

        def step(self, parameters=request):
            r = provider.execute_exact_decode(self.state, parameters, self.token, self.position, cfg["max_context"])
            self.position += r.positions_advanced
            self.token = r.next_token
            return r.positions_advanced

        def steps(self, n):
            advanced = 0
            for r in provider.execute_exact_decode_steps(self.state, request, cfg["max_context"], n):
                advanced += r.positions_advanced
                self.position += r.positions_advanced
                self.token = r.next_token
            return advanced

    streams = [Stream(i) for i in range(args.streams)]
    stream = torch.cuda.ExternalStream(provider.stream(), device=f"cuda:{local}")
    launches0 = provider.telemetry(streams[0].state)["kernel_launches"]
    provider.set_graph_mode(False)
    streams[0].step()
    launches_per_step = provider.telemetry(streams[0].state)["kernel_launches"] - launches0
    provider.set_graph_mode(not args.no_graph)
    for _ in range(max(args.warmup, 3)):
        for s in streams:
            s.step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: steps enqueued back to back, device-resident, one read per batch of 32
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tokens_a, accepted_a = 0, 0
    with ClockSampler(local) as clocks:
        start.record(stream)
        done = 0
        while done < args.steps:
            n = min(32 if args.streams == 1 else 4, args.steps - done)
            for s in streams:
                advanced = s.steps(n)
                tokens_a += advanced
                accepted_a += advanced - n
            done += n
        stop.record(stream)
        stop.synchronize()
        barrier()
    ms_value = start.elapsed_time(stop)
    # ---- e2e: one provider call per step, cursor uploaded and result read back every step
    barrier()
    tokens_b = 0
    start.record(stream)
    for _ in range(args.steps):
        for s in streams:
            tokens_b += s.step()
    stop.record(stream)
    stop.synchronize()
    barrier()
    ms_e2e = start.elapsed_time(stop)
    # ---- the same step with temperature rejection sampling (T 0.7, top-p 0.95, top-k 20):
    # exact top-k of the 5 logits rows, device-side acceptance/residual sampling
    sampled = RequestParameters(sampling_seed=1 + replica, sampling_temperature_ppm=700000, sampling_top_p_ppm=950000,
                                sampling_top_k=20, sampling_min_p_ppm=0, reserved_context_tokens=cfg["max_context"])
    sampled_steps = min(16, args.steps)
    tokens_c = 0
    for timed in (False, True):   # the first round captures the sampled step's graph
        barrier()
        start.record(stream)
        for _ in range(sampled_steps if timed else 3):
            for s in streams:
                advanced = s.step(sampled)
                tokens_c += advanced if timed else 0
        stop.record(stream)
        stop.synchronize()
    barrier()
    ms_sampled = start.elapsed_time(stop)

    # ---- the verify pass alone (target forward over 5 rows, head, candidate selection): CUDA events
    # around 8 back-to-back repeats of its launch sequence (replayed from a graph like the step)
    barrier()
    ms_verify = provider.time_verify(streams[0].state, request, repeats=8)
    barrier()

    (ms_value, ms_e2e, ms_sampled, ms_verify), (tokens_a, tokens_b, accepted_a, tokens_c) = reduce_over_ranks(
        [ms_value, ms_e2e, ms_sampled, ms_verify], [tokens_a, tokens_b, accepted_a, tokens_c], f"cuda:{local}")
    if tensor_parallel:   # every rank emitted the same tokens: count them once
        tokens_a, tokens_b, accepted_a, tokens_c = (x / world for x in (tokens_a, tokens_b, accepted_a, tokens_c))
    jobs = 1 if tensor_parallel else world
    if rank != 0:
        if world > 1:
            dist.barrier()   # tensor parallel: no rank unmaps its exchange area while a peer may still run
            dist.destroy_process_group()
        return

    # ---- extra leg: the same step on the echo model (same weights, o/down scaled to almost nothing,
    # pass-through fusion matrix), whose drafts are right whenever the target's token lies in the draft
    # vocabulary: acceptance lengths 0..4, partial-accept rollback and bonus tokens at full size
    echo_leg = None
    if world == 1 and not routed and not tensor_parallel and not args.no_echo_leg and not args.small:
        echo_provider = model.echo_variant().provider()
        echo_provider.set_gemv_impl(args.gemv_impl)
        echo_provider.set_attention_impl(args.attention_impl)
        echo_provider.set_graph_mode(not args.no_graph)
        es = echo_provider.create_request_state()
        prompt = np.random.default_rng(77).integers(0, cfg["vocab"], context, dtype=np.uint32)
        echo_provider.fill_synthetic_kv(es, 0, synthetic, seed=4321)
        token = echo_provider.prefill(es, request, prompt[synthetic:], first_position=synthetic, chunk_rows=5)
        position = context
        for _ in range(3):
            r = echo_provider.execute_exact_decode(es, request, token, position, cfg["max_context"])
            position, token = position + r.positions_advanced, r.next_token
        echo_stream = torch.cuda.ExternalStream(echo_provider.stream(), device=f"cuda:{local}")
        echo_steps, echo_tokens = min(32, args.steps), 0
        torch.cuda.synchronize()
        start.record(echo_stream)
        for r in echo_provider.execute_exact_decode_steps(es, request, cfg["max_context"], echo_steps):
            echo_tokens += r.positions_advanced
        stop.record(echo_stream)
        stop.synchronize()
        echo_ms = start.elapsed_time(stop)
        t = echo_provider.telemetry(es)
        echo_leg = {"model": "echo variant of the same weights (drafts can be right)", "steps": echo_steps,
                    "accepted_len_per_step": echo_tokens / echo_steps, "value": echo_tokens / (echo_ms * 1e-3),
                    "unit": "tok/s", "ms_per_step": echo_ms / echo_steps,
                    "accepted_depth_calls": [int(x) for x in t["accepted_depth_calls"]]}
        es.close()
        del echo_provider

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if peaks else "fallback"
    # the dominant kernel: the dense model's gate/up GEMV; for the routed model the largest
    # tensor-core GEMV of a layer (fused q/k/v projection) stands in, the expert kernels being
    # selected per token
    kernel_name = "qkv" if routed else "gate_up"
    kernel_ms, kernel_bytes = gemv_kernel_leg(model, provider, args.gemv_impl, name=kernel_name)
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    step_bytes, verify_bytes = model.step_bytes(context)
    ms_per_step = ms_value / (args.steps * args.streams)   # per step of one stream
    kernel_shape = model.layers[0].m[kernel_name]
    metric = METRIC if not routed else "decode_tok_per_s_mtp4_q4h_8k_moe35b"
    step_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9
    value = tokens_a / (ms_value * 1e-3)
    e2e = tokens_b / (ms_e2e * 1e-3)
    line = {
        "metric": metric if args.kv_encoding == "q4h" else metric.replace("q4h", "f16kv"), "value": value,
        "unit": "tok/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if tensor_parallel else "weak",
        "vs_baseline": None, "dtype": "nvfp4xnvfp4->f32", "data": "synthetic",
        "config": {"workload": workload_name(context, args.kv_encoding, args.model, args.streams),
                   "layers": cfg["layers"],
                   "parallelism": f"tp{world}: one stream, model sharded over {world} GPUs" if tensor_parallel
                   else f"dp{world} replicas", "streams_per_gpu": args.streams,
                   "l2_policy": f"inputs larger than L2 ({step_bytes / 1e9:.1f} GB streamed per step)",
                   "prompt_cache": f"first {synthetic} positions seeded synthetic records, last {REAL_PREFILL} real prefill",
                   "gemv_impl": "tcgen05" if args.gemv_impl == 1 else "dp4a",
                   "attention_impl": {0: "scalar", 1: "mma.sync", 2: "tcgen05"}[args.attention_impl],
                   "split_tokens": cfg["split_tokens"],
                   "launch": "per kernel" if args.no_graph else "CUDA graph per step"},
        "accepted_len_per_step": tokens_a / (args.steps * args.streams * jobs),
        "tok_s_if_all_drafts_accepted": 5.0 * args.steps * args.streams * jobs / (ms_value * 1e-3),
        "step_algorithmic_gb": step_bytes / 1e9, "step_gbs": step_gbs, "step_frac_of_hbm": step_gbs / hbm_peak,
        # the stated target is on the verify pass: its algorithmic bytes / its measured time
        "verify_step": {"ms": ms_verify, "algorithmic_gb": verify_bytes / 1e9,
                        "achieved": verify_bytes / (ms_verify * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                        "frac": verify_bytes / (ms_verify * 1e-3) / 1e9 / hbm_peak, "target_frac": VERIFY_TARGET_FRAC,
                        "target_met": verify_bytes / (ms_verify * 1e-3) / 1e9 / hbm_peak >= VERIFY_TARGET_FRAC,
                        "how": "CUDA events around 8 back-to-back verify passes (graph replay), max over ranks"},
        "verify_frac_of_hbm": verify_bytes / (ms_verify * 1e-3) / 1e9 / hbm_peak,
        "roofline": {"bound": "hbm", "kernel": f"nvfp4_gemv {kernel_name} {kernel_shape.rows}x{kernel_shape.cols} M=5",
                     "achieved": achieved,
                     "peak": hbm_peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": captured_dram_bytes(kernel_shape.rows, kernel_shape.cols, 5) if args.gemv_impl == 1 else None,
                     "algorithmic_bytes": kernel_bytes, "kernel_ms": kernel_ms},
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 56,
                "ms_per_step": ms_e2e / (args.steps * args.streams)},
        "sampled_t0.7_top_p0.95_top_k20": {"value": tokens_c / (ms_sampled * 1e-3), "unit": "tok/s",
                                           "ms_per_step": ms_sampled / (sampled_steps * args.streams),
                                           "steps": sampled_steps},
        "echo_model_leg": echo_leg,
        "gpu_launches": int(launches_per_step * args.steps * args.streams),
        "clocks": clocks.summary(),
    }
    if tensor_parallel:
        line["step_bytes_scope"] = "per GPU: this rank's shard of the blocks and of the KV, plus the replicated heads"
    # the CPU leg runs at N = 1 only: at N > 1 the other ranks would sit in the closing barrier meanwhile
    if not args.no_cpu_baseline and not routed and world == 1:
        sample = OracleSteps(DENSE_27B, context, REFERENCE_LAYERS)
        sample.step()
        seconds, tokens, steps = 0.0, 0, 0
        while seconds < 12.0 or steps < 2:
            s, n = sample.step()
            seconds, tokens, steps = seconds + s, tokens + n, steps + 1
        line["cpu_baseline"] = {"value": tokens / seconds, "unit": "tok/s", "cores": sample.threads, "kind": "port",
                                "sample": f"{sample.description}; {steps} steps in {seconds:.1f} s"}
        # what a whole 64-layer step would take, from two MEASURED slices (1 and 2 layers): the time one
        # more layer adds, times the layers left out -- reported beside the measured value, not in its place
        per_step = seconds / steps
        del sample
        shallow = OracleSteps(DENSE_27B, context, 1)
        shallow.step()
        shallow_seconds = sum(shallow.step()[0] for _ in range(3)) / 3.0
        per_layer = max(per_step - shallow_seconds, 0.0) / (REFERENCE_LAYERS - 1)
        whole = per_step + (DENSE_27B["layers"] - REFERENCE_LAYERS) * per_layer
        del shallow
        line["cpu_baseline"]["whole_model_estimate"] = {
            "value": (tokens / steps) / whole, "unit": "tok/s", "seconds_per_step": whole,
            "how": f"measured {per_step:.3f} s per step with {REFERENCE_LAYERS} layers and {shallow_seconds:.3f} s with 1: "
                   f"{per_layer:.3f} s per layer x {DENSE_27B['layers']} layers + the rest"}
        line["cpu_baseline"]["reference_ffn"] = reference_cpu_ffn(DENSE_27B, line["cpu_baseline"]["cores"])
        line["cpu_baseline"]["reference_acceptance"] = reference_cpu_acceptance()
        # ... and one whole step measured, all 64 layers (about as long as the estimate says)
        if not args.no_cpu_full_step:
            whole_model = OracleSteps(DENSE_27B, context, DENSE_27B["layers"], share_layer_bytes=True)
            step_seconds, step_tokens = whole_model.step()
            line["cpu_baseline"]["whole_model_step"] = {
                "value": step_tokens / step_seconds, "unit": "tok/s", "seconds_per_step": step_seconds,
                "cores": whole_model.threads, "kind": "port", "sample": whole_model.description}
            del whole_model
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def microbench(args):
    """Kernel microbenchmark of the NVFP4 GEMV / skinny GEMM on the verify-step shapes: the 27B
    projections (N x K: qkv 7168x5120, o 5120x5120, gate/up 34816x5120, down 5120x17408, lm-head
    151936x5120) at M = 5, 40, 128, 160, 640 activation rows.  Random NVFP4 weights, N(0,1)
    activations; enough distinct matrices per shape to stream at least 1 GB (far beyond L2) per
    timed pass; the tensor-core kernel alone, CUDA events on the launching stream.  One JSON line
    per (shape, M): time, algorithmic GB/s (weights 0.5625 B/element + BF16 rows in and out) against
    the measured HBM peak, and FP4 TFLOP/s (2 M N K) against the nominal dense 9 PFLOP/s."""
    import torch
    from quantum_llm_b200 import build as qbuild
    qbuild.build()
    from quantum_llm_b200 import lib as ql
    from quantum_llm_b200 import synthetic
    L = ql.load()
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    try:
        hbm_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6650.0))
    except OSError:
        hbm_peak = 6650.0
    shapes = [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408),
              ("lm_head", 151936, 5120)]
    stream = torch.cuda.Stream(device=dev)
    sp = C.c_void_p(stream.cuda_stream)
    for name, n, k in shapes:
        weight_bytes = n * k * 9 // 16
        copies = max(1, -(-(1 << 30) // weight_bytes))
        mats, handles = [], []
        for i in range(copies):
            m = synthetic.quantize(synthetic._random_rows(n, k, 7000 + i, dev))
            h, cm = C.c_void_p(), m.c()
            ql.check(L.qllm_k_matrix_prepare(C.byref(cm), sp, C.byref(h)))
            mats.append(m)
            handles.append(h)
        stream.synchronize()
        for rows in (5, 40, 128, 160, 640):
            x = torch.randn((rows, k), device=dev, dtype=torch.float32)
            y = torch.empty((rows, n), device=dev, dtype=torch.float32)
            ws_bytes = L.qllm_k_nvfp4_gemv_workspace_bytes(rows, n, k)
            ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
            best = None
            with torch.cuda.stream(stream):
                # one full call quantises the activations into the workspace
                ql.check(L.qllm_k_nvfp4_gemv_prepared(handles[0], x.data_ptr(), y.data_ptr(), rows, ws.data_ptr(),
                                                     ws_bytes, 1, sp))
                for rep in range(4):
                    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    start.record(stream)
                    for h in handles:
                        ql.check(L.qllm_k_nvfp4_gemv_prepared_core(h, rows, ws.data_ptr(), ws_bytes, sp))
                    stop.record(stream)
                    stop.synchronize()
                    ms = start.elapsed_time(stop) / len(handles)
                    if rep > 0:
                        best = ms if best is None else min(best, ms)
            algorithmic = weight_bytes + rows * k * 2 + rows * n * 2
            gbs = algorithmic / (best * 1e-3) / 1e9
            tflops = 2.0 * rows * n * k / (best * 1e-3) / 1e12
            print(json.dumps({"microbench": "nvfp4_gemv_mma", "shape": name, "n": n, "k": k, "m": rows,
                              "us": best * 1e3, "algorithmic_bytes": algorithmic, "gbs": gbs,
                              "frac_of_hbm": gbs / hbm_peak, "fp4_tflops": tflops,
                              "frac_of_nominal_fp4": tflops / 9000.0, "matrices": copies}), flush=True)
            del x, y, ws
        for h in handles:
            L.qllm_k_matrix_release(h)
        del mats, handles
        torch.cuda.empty_cache()


def prefill_bench(args):
    """Prompt path on one GPU: target chunks of --chunk-rows rows (8 is the reference's microbatch
    limit, 128 the widest chunk here), each followed by its draft-priming batch, from an empty
    cache; host tokens in, first token out.  Every chunk streams the whole model once."""
    import numpy as np
    import torch
    assert torch.cuda.is_available(), "bench.py needs a CUDA device; there is no CPU path"
    from quantum_llm_b200 import build as qbuild
    qbuild.build()
    from quantum_llm_b200.provider import RequestParameters
    from quantum_llm_b200.synthetic import DENSE_27B, MOE_35B, DeviceModel
    cfg = dict(MOE_35B if args.model == "moe35b" else DENSE_27B)
    if args.small:
        cfg["layers"] = 4
    tokens = args.prefill_bench
    cfg["max_context"] = tokens + 1024
    model = DeviceModel(cfg, seed=0, device="cuda:0")
    provider = model.provider()
    provider.set_gemv_impl(args.gemv_impl)
    request = RequestParameters(sampling_seed=1, sampling_temperature_ppm=0, reserved_context_tokens=cfg["max_context"])
    prompt = np.random.default_rng(1).integers(0, cfg["vocab"], tokens, dtype=np.uint32)
    times = []
    for trial in range(3):          # the first pass warms the code paths up
        state = provider.create_request_state()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = provider.prefill(state, request, prompt, first_position=0, chunk_rows=args.chunk_rows)   # synchronous per chunk
        times.append(time.perf_counter() - t0)
        state.close()
    best = min(times[1:])
    print(json.dumps({"prefill_bench": args.model, "prompt_tokens": tokens, "chunk_rows": args.chunk_rows,
                      "time_to_first_token_ms": round(best * 1e3, 2), "prompt_tokens_per_s": round(tokens / best, 1),
                      "first_token": int(first), "layers": cfg["layers"]}))


if __name__ == "__main__":
    a = parse()
    if a.prefill_bench:
        prefill_bench(a)
    elif a.microbench:
        microbench(a)
    elif a.impl == "reference":
        reference_arm(a)
    else:
        ours(a)
