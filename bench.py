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
# dram__bytes_read.sum + dram__bytes_write.sum of one gate/up GEMV launch (tcgen05 kernel,
# 34816x5120, 5 rows), from the ncu capture summarised in
# profiles/nvfp4_gemv_and_attention_kernels_4layer_case.md (100.39 MB read + 3.62 MB written)
GATE_UP_DRAM_BYTES_NCU = 104.0e6


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--gemv-impl", type=int, default=int(os.environ.get("QLLM_GEMV_IMPL", "1")))
    ap.add_argument("--small", action="store_true", help="4-layer model for profiler captures")
    ap.add_argument("--model", default="dense27b", choices=["dense27b", "moe35b"],
                    help="dense27b: the headline workload; moe35b: the routed 35B-A3B-class target")
    ap.add_argument("--parallelism", default="dp", choices=["dp", "tp"],
                    help="N > 1: dp = N independent replicas (weak scaling, the default); tp = ONE stream whose "
                         "model is sharded over the N GPUs (tensor parallel, strong scaling; dense27b, N = 2 or 4)")
    ap.add_argument("--streams", type=int, default=1, help="independent requests per GPU, stepped in turn")
    ap.add_argument("--context", type=int, default=0, help="cached tokens (0: 32768 dense, 8192 routed)")
    ap.add_argument("--kv-encoding", default="q4h", choices=["q4h", "f16"],
                    help="target KV cache: Q4H (the headline metric) or exact F16 (metric ..._f16kv_32k)")
    ap.add_argument("--split-tokens", type=int, default=0,
                    help="cached tokens per attention CTA (multiple of 64; 0 = the model configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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


class CpuSample:
    """A bounded sample of the workload for the CPU oracle (a port of the reference's
    arithmetic): the four NVFP4 GEMVs of ONE 27B-geometry layer at 5 rows plus the Q4H
    attention of one layer over 2048 cached tokens (186 MB of weights, 2.2 MB of KV records).
    Built once; `time(seconds)` repeats passes over it and returns the mean seconds per pass,
    which the caller scales by algorithmic bytes to a full step."""

    def __init__(self, threads=None):
        import numpy as np
        from oracle import binding as ob
        self.ob, self.O = ob, ob.lib()
        # explicit: launchers such as torchrun export OMP_NUM_THREADS=1
        self.O.qo_set_threads(threads or len(os.sched_getaffinity(0)) or 1)
        self.threads = int(self.O.qo_max_threads())
        rng = np.random.default_rng(0)
        H, F, QH, KV, HD = 5120, 17408, 40, 8, 128
        self.geometry = (QH, KV, HD)
        shapes = [((QH + 2 * KV) * HD, H), (H, QH * HD), (2 * F, H), (H, F)]
        self.mats, self.bytes = [], 0
        for rows, cols in shapes:
            codes = rng.integers(0, 256, (rows, cols // 2), dtype=np.uint8)
            scales = rng.integers(0x20, 0x48, (rows, cols // 16), dtype=np.uint8)
            self.mats.append((ob.matrix(codes, scales, 1e-3, 336.0), codes, scales,
                              rng.normal(0, 1, (5, cols)).astype(np.float32)))
            self.bytes += codes.size + scales.size
        self.ctx, self.pt = 2048, 256
        layer_bytes = self.O.qo_kv_layer_bytes(ob.KV_Q4H, self.pt, KV, HD)
        self.pages = [rng.integers(0, 256, layer_bytes, dtype=np.uint8)
                      for _ in range((self.ctx + 4 + self.pt - 1) // self.pt)]
        self.table = (C.c_void_p * len(self.pages))(*[p.ctypes.data for p in self.pages])
        k = rng.normal(0, 1, (self.ctx + 4, KV * HD)).astype(np.float32)
        self.O.qo_kv_store(ob.KV_Q4H, self.table, 0, self.pt, KV, HD, ob._ptr(k), ob._ptr(k), self.ctx + 4, KV * HD, 0)
        self.q = rng.normal(0, 1, (5, QH * HD)).astype(np.float32)
        self.out = np.empty_like(self.q)
        self.bytes += (self.ctx + 4) * KV * (HD // 2 + 2) * 2
        self.description = ("one 27B-geometry layer (4 NVFP4 GEMVs at 5 rows, 186 MB of weights) + Q4H attention "
                            "over 2048 cached tokens, scaled by algorithmic bytes to a full step")

    def one_pass(self):
        QH, KV, HD = self.geometry
        for m, _, _, x in self.mats:
            self.ob.gemv(m, x)
        self.O.qo_attention(self.ob.KV_Q4H, self.table, 0, self.pt, self.ob._ptr(self.q), QH * HD, 5, self.ctx,
                            QH, KV, HD, 512, 1, self.ob._ptr(self.out))

    def time(self, seconds):
        passes, t0 = 0, time.perf_counter()
        while True:
            self.one_pass()
            passes += 1
            elapsed = time.perf_counter() - t0
            if elapsed >= seconds:
                return elapsed / passes, passes, elapsed


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


def reference_arm(args):
    """Reference arm: the reference's arithmetic for this path on the host cores.  The
    reference's provider itself needs a CUDA device and a compiled model artifact, so its CPU
    implementation of the path is the oracle port (kind "port").  One step = repeated passes
    over the bounded sample for about 3 s, scaled by algorithmic bytes to a full step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    assert args.model == "dense27b" and args.streams == 1, "the reference arm times the headline workload only"
    from quantum_llm_b200.synthetic import DENSE_27B
    step_bytes = algorithmic_step_bytes(DENSE_27B, args.context)
    sample = CpuSample()
    per_pass, passes = [], 0
    for i in range(args.warmup + args.steps):
        seconds, n, _ = sample.time(3.0 if i >= args.warmup else 1.0)
        if i >= args.warmup:
            per_pass.append(seconds)
            passes += n
    step_s = (sum(per_pass) / len(per_pass)) * step_bytes / sample.bytes
    value = 1.0 / step_s   # accepted length 1.0 on random-init weights: one token per step
    text = f"{sample.description}; {passes} timed passes on {sample.threads} threads"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4xnvfp4->f32", "data": "synthetic",
            "config": {"workload": workload_name(args.context), "layers": DENSE_27B["layers"],
                       "parallelism": "host cores of rank 0", "implementation": "CPU port of the reference arithmetic"},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": sample.threads, "kind": "port", "sample": text},
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

    (ms_value, ms_e2e, ms_sampled), (tokens_a, tokens_b, accepted_a, tokens_c) = reduce_over_ranks(
        [ms_value, ms_e2e, ms_sampled], [tokens_a, tokens_b, accepted_a, tokens_c], f"cuda:{local}")
    if tensor_parallel:   # every rank emitted the same tokens: count them once
        tokens_a, tokens_b, accepted_a, tokens_c = (x / world for x in (tokens_a, tokens_b, accepted_a, tokens_c))
    jobs = 1 if tensor_parallel else world
    if rank != 0:
        if world > 1:
            dist.barrier()   # tensor parallel: no rank unmaps its exchange area while a peer may still run
            dist.destroy_process_group()
        return

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
                   "launch": "per kernel" if args.no_graph else "CUDA graph per step"},
        "accepted_len_per_step": tokens_a / (args.steps * args.streams * jobs),
        "tok_s_if_all_drafts_accepted": 5.0 * args.steps * args.streams * jobs / (ms_value * 1e-3),
        "step_algorithmic_gb": step_bytes / 1e9, "step_gbs": step_gbs, "step_frac_of_hbm": step_gbs / hbm_peak,
        "roofline": {"bound": "hbm", "kernel": f"nvfp4_gemv {kernel_name} {kernel_shape.rows}x{kernel_shape.cols} M=5",
                     "achieved": achieved,
                     "peak": hbm_peak, "peak_source": peak_kind, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "traffic": GATE_UP_DRAM_BYTES_NCU if args.gemv_impl == 1 and not routed else None,
                     "algorithmic_bytes": kernel_bytes, "kernel_ms": kernel_ms},
        "e2e": {"value": e2e, "unit": "tok/s", "h2d_bytes_per_step": 12, "d2h_bytes_per_step": 56,
                "ms_per_step": ms_e2e / (args.steps * args.streams)},
        "sampled_t0.7_top_p0.95_top_k20": {"value": tokens_c / (ms_sampled * 1e-3), "unit": "tok/s",
                                           "ms_per_step": ms_sampled / (sampled_steps * args.streams),
                                           "steps": sampled_steps},
        "gpu_launches": int(launches_per_step * args.steps * args.streams),
        "clocks": clocks.summary(),
    }
    if tensor_parallel:
        line["step_bytes_scope"] = "per GPU: this rank's shard of the blocks and of the KV, plus the replicated heads"
    if not args.no_cpu_baseline:
        sample = CpuSample()
        per_pass, passes, elapsed = sample.time(12.0)
        cpu_step = per_pass * step_bytes / sample.bytes
        line["cpu_baseline"] = {"value": 1.0 / cpu_step, "unit": "tok/s", "cores": sample.threads, "kind": "port",
                                "sample": f"{sample.description}; {passes} passes in {elapsed:.1f} s"}
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
