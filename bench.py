"""Benchmark of the speculative-decoding verify step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload (one session per GPU; weights replicated, no collective - sessions are independent):
Qwen3-8B-shaped AWQ model (36 layers, hidden 4096, 32 Q / 8 KV heads, head_dim 128, FFN 12288, vocab 151936,
int4 group-128 linears, BF16 embeddings / norms / lm_head), context capacity 4096, seeded 2048-token prompt,
k = 8 drafts = the model's own greedy continuation with p = 0.2 random substitution (the same seed on every rank).
Random-init synthetic weights stand in for a checkpoint. A step is one verify step: one forward of
[pending, 8 drafts] over the session's KV cache, greedy acceptance and KV commit.

Prints ONE JSON line:
  value        accepted tokens/s, device-resident loop (drafts, pending token and context length on the device,
               steps enqueued back to back, one drain at the end), whole job over all GPUs. The timed region of
               exactly K steps is repeated until it covers a second; the median region is reported, with the
               minimum and maximum beside it
  e2e          the same metric through ei_session_verify with host token buffers: per step an H2D copy of the
               tokens, the graph, a D2H copy of the result and one host synchronisation
  roofline     the dominant kernel (fused gate/up int4 projection, 53 MB of weights per launch) timed alone with
               CUDA events over the 36 layers' distinct weights (1.9 GB > L2), algorithmic bytes / time / measured
               HBM peak
  step_roofline  the whole step: (prepared weight bytes + live KV bytes) / step time / measured HBM peak
  cpu_baseline the CPU oracle port of the reference's FP32 executor, timed on the host cores (N = 1 only)
  reference_cuda  the UNMODIFIED reference's own CUDA path (oracle/_ref: Qwen3Session<bf16>::prefill_eager +
               op::cuda::sample, its kernels recompiled for sm_100) on the same model, GPU and step shape, outside
               the timed region (N = 1 only; absent where oracle/_ref is not built)
  sessions_leg the sharded-sessions configuration: Qwen2.5-7B-shaped AWQ model, 64 sessions with seeded prompt
               lengths in [256, 8192] split evenly over the GPUs, k = 4, p = 0.3, three sessions stacked per
               forward (ei_batch_verify)
`--impl reference` times the CPU implementation alone (rank 0 only), whole 36-layer-deep steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

METRIC = "accepted_tokens_per_s_per_session_qwen3_8b_awq_k8"
UNIT = "tokens/s"
K_DRAFTS = 8
PROMPT = 2048
CAPACITY = 4096
P_SUBSTITUTE = 0.2
SEED = 0  # prompt and draft substitutions: the same on every rank, so every rank times the same steps


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: in-process NVML reads every few
    milliseconds (the region can be shorter than one nvidia-smi start-up), nvidia-smi in a loop if NVML cannot
    be loaded. Only reads: no setting of the GPU is touched."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.lines, self.samples = [], []
        self.process = None
        self.thread = None
        self.stop_event = threading.Event()
        self.max_clock = None
        self.source = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            masks = {"hw_slowdown": pynvml.nvmlClocksEventReasonHwSlowdown,
                     "hw_thermal_slowdown": pynvml.nvmlClocksEventReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": pynvml.nvmlClocksEventReasonSwThermalSlowdown,
                     "sw_power_cap": pynvml.nvmlClocksEventReasonSwPowerCap}

            def loop():
                while not self.stop_event.is_set():
                    try:
                        clock = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        bits = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                        self.samples.append((clock, [name for name, mask in masks.items() if bits & mask]))
                    except pynvml.NVMLError:
                        pass
                    self.stop_event.wait(0.005)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            self.thread = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            self.source = "nvidia-smi"
        except OSError:
            self.process = None

    def _read(self):
        for line in self.process.stdout:
            self.lines.append(line.strip())

    def stop(self):
        clocks, max_clocks, reasons = [], [], set()
        if self.thread:
            self.stop_event.set()
            self.thread.join(timeout=2)
            for clock, active in self.samples:
                clocks.append(clock)
                reasons.update(active)
            max_clocks = [self.max_clock] if self.max_clock else []
        if self.process:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
            for line in self.lines:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    max_clocks.append(float(parts[2]))
                except ValueError:
                    continue
                for name, value in zip(self.NAMES, parts[5:9]):
                    if value.lower().startswith("active"):
                        reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(max_clocks) if max_clocks else None,
                "reasons": sorted(reasons), "samples": len(clocks), "source": self.source}


def continuation_length(steps_total: int) -> int:
    """Tokens of greedy continuation both arms walk over (first generated token included)."""
    rows = K_DRAFTS + 1
    return min(CAPACITY - PROMPT - rows - 1, steps_total * rows + rows) + 1


def simulated_tokens_per_step(package, steps: int, warmup: int) -> float:
    """Mean accept length of the timed steps: with exact greedy drafts it depends on the seeded substitution mask
    alone, so the CPU arm (which cannot afford to generate the continuation) and the GPU arm agree on it."""
    rows = K_DRAFTS + 1
    length = continuation_length(steps + warmup)
    mask = package.synthetic.substitution_mask(SEED, length, P_SUBSTITUTE)
    budget = (length - rows) // rows
    emitted = package.sharding.simulate_accepts(mask, rows, steps, budget)
    return float(sum(emitted)) / len(emitted)


class CpuStep:
    """Whole verify steps of the 8B shape on the host cores with the CPU oracle in FP32 mode (the arithmetic of the
    reference's CPU executor; its AWQ weights dequantised to FP32). The 36 layers have identical shapes, so ONE
    layer's FP32 weights (1.6 GB instead of 58 GB) are run 36 times per step, each pass over 9 rows at context
    2048, followed by the full 151936-row lm_head. Every pass does the work of its layer; only the values repeat."""

    def __init__(self, oracle, package, threads: int):
        self.oracle, self.package, self.threads = oracle, package, threads
        shape = package.synthetic.qwen3_8b_awq()
        self.shape = shape
        oracle.oracle_library().vo_set_threads(threads)
        rng = np.random.default_rng(0)
        layer_shape = package.Shape(vocab_size=8, n_layers=1, n_heads=shape.n_heads, n_kv_heads=shape.n_kv_heads,
                                    hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size,
                                    max_position_embeddings=CAPACITY, qk_norm=True)
        H, F = shape.hidden_size, shape.intermediate_size
        qw, kvw = shape.n_heads * 128, shape.n_kv_heads * 128
        f2b = package.synthetic.float_to_bf16

        def dense(out, inp):
            return [(0, f2b(rng.standard_normal((out, inp), dtype=np.float32) * np.float32(0.02)))]

        ones = lambda n: [(0, f2b(np.ones(n, dtype=np.float32)))]  # noqa: E731
        tensors = {"token_embeddings.weight": dense(8, H), "rms_out_w": ones(H), "lm_head": dense(8, H),
                   "rms_att_w0": ones(H), "rms_ffn_w0": ones(H), "q_norm0": ones(128), "k_norm0": ones(128),
                   "wq0": dense(qw, H), "wk0": dense(kvw, H), "wv0": dense(kvw, H), "wo0": dense(H, qw),
                   "w_gate0": dense(F, H), "w_up0": dense(F, H), "w_down0": dense(H, F)}
        self.layer = oracle.OracleModel(layer_shape, tensors, capacity=CAPACITY)
        self.tokens = np.arange(K_DRAFTS + 1, dtype=np.uint32) % 8
        self.x = rng.standard_normal((K_DRAFTS + 1, H), dtype=np.float32)
        self.head = rng.standard_normal((shape.vocab_size, H), dtype=np.float32)
        self.sample = (f"CPU oracle port of the reference FP32 executor, {threads} threads: whole steps = 36 passes of "
                       f"one decoder layer of the 8B shape (9 rows at context {PROMPT}; the layers' shapes are "
                       "identical, one layer's FP32 weights are reused) + the full 151936-row lm_head")

    def step(self) -> float:
        start = time.perf_counter()
        for _ in range(self.shape.n_layers):
            self.layer.resize(PROMPT)                          # cached keys/values present (their values are irrelevant)
            self.layer.forward(self.tokens, 0)
        self.oracle.op_linear(self.x, self.head, None)
        return time.perf_counter() - start

    def one_layer_single_thread(self) -> float:
        """One layer pass on ONE thread: what one executor of the reference (single-threaded) would take."""
        lib = self.oracle.oracle_library()
        lib.vo_set_threads(1)
        self.layer.resize(PROMPT)
        start = time.perf_counter()
        self.layer.forward(self.tokens, 0)
        elapsed = time.perf_counter() - start
        lib.vo_set_threads(self.threads)
        return elapsed


WORKLOAD = ("qwen3-8b-shape AWQ verify step: 36 layers, hidden 4096, 32Q/8KV, FFN 12288, vocab 151936, k=8 (9 rows), "
            "prompt 2048, capacity 4096, p=0.2 draft substitution, one session per GPU")


def workload_config(package, steps: int, warmup: int) -> dict:
    """The `config` object of both arms, key for key."""
    return {"workload": WORKLOAD, "sessions_per_gpu": 1,
            "tokens_per_step": simulated_tokens_per_step(package, steps, warmup)}


def run_reference(args, rank: int):
    if rank != 0:
        return
    package, oracle = entry.load_package(), entry.load_oracle()
    threads = os.cpu_count() or 1
    cpu = CpuStep(oracle, package, threads)
    for _ in range(min(args.warmup, 1)):
        cpu.step()
    # Whole steps, each about five seconds of all host cores: as many of the requested steps as fit in three minutes
    # (at least three), so that the arm ends within a few minutes whatever --steps asks for.
    times, budget = [], 180.0
    while len(times) < max(1, args.steps) and (len(times) < 3 or sum(times) < budget):
        times.append(cpu.step())
    step_seconds = sum(times) / len(times)
    config = workload_config(package, args.steps, args.warmup)
    value = config["tokens_per_step"] / step_seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "executor": "CPU, FP32, AWQ weights dequantised; tokens per step = accept lengths of the seeded drafts",
        "steps_timed": len(times),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": cpu.sample + "; %d whole steps timed" % len(times),
                         "ms_per_step_min": min(times) * 1e3, "ms_per_step_max": max(times) * 1e3},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def time_dominant_kernel(package, torch, shape, layers: int, rows: int, repeats: int):
    """Fused gate/up int4 projection alone, cycling over `layers` distinct weight sets (> L2). One pass over the
    sets is captured in a CUDA graph (as the step itself runs from one) and replayed; CUDA events on the stream
    the kernels run on. Issued call by call from Python the host, not the kernel, would set the pace."""
    ops, syn = package.operators, package.synthetic
    stream = torch.cuda.Stream()
    ctx = ops.prepare_execution_context(stream.cuda_stream)
    H, F = shape.hidden_size, shape.intermediate_size
    groups = H // 128
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    weights, keep = [], []
    for _ in range(layers):
        q = torch.randint(-2**31, 2**31 - 1, (2 * F, H // 8), dtype=torch.int32, device="cuda", generator=gen)
        z = torch.randint(-2**31, 2**31 - 1, (2 * F, (groups + 7) // 8), dtype=torch.int32, device="cuda", generator=gen)
        s = (torch.rand((2 * F, groups), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
        keep.append((q, z, s))
        weights.append(ops.prepare_awq(q, s, z, 128, H))
    x = torch.randn((rows, H), device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.empty((rows, F), dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()

    def one_pass():
        for w in weights:
            ops.awq_gate_up_silu(ctx, x, w, out)

    with torch.cuda.stream(stream):
        one_pass()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            one_pass()
        for _ in range(3):
            graph.replay()
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(repeats):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    seconds = start.elapsed_time(end) * 1e-3 / (repeats * layers)
    n, k = 2 * F, H
    algorithmic = n * k // 2 + n * groups * 2 + n * ((groups + 7) // 8) * 4 + rows * k * 2 + rows * F * 2
    del keep
    return seconds, algorithmic


def time_reference_cuda(package, oracle, torch, shape, tensors, drafts, first, steps: int):
    """Verify steps of the same shape through the unmodified reference's CUDA path (oracle/_ref) on this GPU:
    cache.resize(+9), Qwen3Session<bf16>::prefill_eager of [pending, 8 drafts], op::cuda::sample per row, the
    greedy tokens copied to the host, acceptance on the host, cache.resize back (what its SpeculativeDecoder does
    per round, runtime/src/speculative_decoder.cpp:190-224). Wall clock around whole steps, each ending in the
    reference's own stream synchronisation."""
    rows = K_DRAFTS + 1
    host = {}
    for name, kinds in tensors.items():
        items = []
        for kind, t in kinds:
            if t.dtype == torch.bfloat16:
                items.append((kind, t.view(torch.int16).cpu().numpy().view(np.uint16)))
            else:
                items.append((kind, t.cpu().numpy()))
        host[name] = items
    reference = oracle.ReferenceCuda(shape, host, CAPACITY)
    del host
    prompt = package.synthetic.make_prompt(SEED, PROMPT, shape.vocab_size)
    reference.forward(prompt, want_logits=False)
    reference.resize(0)
    begin = time.perf_counter()
    reference.forward(prompt, want_logits=False)   # the reference's own prompt prefill, warm
    prompt_seconds = time.perf_counter() - begin

    def run(count: int):
        emitted_total, offset, pending = 0, 0, first
        start = time.perf_counter()
        for _ in range(count):
            if offset + rows + 1 >= len(drafts):
                reference.resize(PROMPT)
                offset, pending = 0, first
            inputs = np.concatenate([[pending], drafts[offset + 1:offset + rows]]).astype(np.uint32)
            length = reference.size()
            _, greedy = reference.forward(inputs, want_logits=False)
            emitted = oracle.accept(inputs, greedy)
            reference.resize(length + emitted)
            pending = int(greedy[emitted - 1])
            offset += emitted
            emitted_total += emitted
        return time.perf_counter() - start, emitted_total

    run(3)
    reference.resize(PROMPT)
    seconds, emitted = run(steps)
    del reference
    torch.cuda.empty_cache()
    return seconds / steps, emitted / steps, prompt_seconds


def run_speculative_leg(package, torch, target_model, rounds: int) -> dict:
    """Whole speculative rounds (the reference's SpeculativeDecoder loop, runtime/src/speculative_decoder.cpp:227-306)
    with the 8B-shape AWQ target and a 0.6B-shape BF16 draft, k = 8: nine draft decode steps chained on the device,
    one verify forward, the hand-over between the two sessions; the host synchronises once for all rounds. Both models
    are random-init, so nearly every draft is rejected: the figure is the time of a round and its parts, not the
    acceptance."""
    syn = package.synthetic
    draft_shape = syn.qwen3_0_6b(max_position_embeddings=CAPACITY)
    draft_model = package.Model(draft_shape, syn.make_device_model(draft_shape, seed=1))
    target, draft = target_model.new_session(CAPACITY, graph=True), draft_model.new_session(CAPACITY, graph=True)
    decoder = package.runtime.SpeculativeDecoder(target, draft, K_DRAFTS)
    prompt = syn.make_prompt(SEED, PROMPT, target_model.shape.vocab_size)
    decoder.prefill(prompt)
    decoder.enqueue(3)
    decoder.drain()
    decoder.truncate(1)
    torch.cuda.synchronize()
    begin = time.perf_counter()
    decoder.enqueue(rounds)
    produced = decoder.drain()
    round_ms = (time.perf_counter() - begin) * 1e3 / rounds
    # One draft decode step alone, chained the same way (no host synchronisation between steps).
    decoder.close()
    draft.prefill(prompt)
    token = 1
    draft.decode(token)
    torch.cuda.synchronize()
    begin = time.perf_counter()
    for _ in range(32):
        draft.decode(token)
    torch.cuda.synchronize()
    draft_ms = (time.perf_counter() - begin) * 1e3 / 32
    del target, draft, draft_model
    torch.cuda.empty_cache()
    return {"workload": "qwen3-8b-shape AWQ target + qwen3-0.6b-shape BF16 draft, k=8, prompt 2048, rounds chained on "
                        "the device, one host synchronisation for all rounds",
            "rounds": rounds, "ms_per_round": round_ms, "tokens_per_round": (len(produced) - 1) / rounds,
            "draft_decode_ms_per_token_host_driven": draft_ms,
            "note": "random-init draft: nearly every draft is rejected, so tokens_per_round is about 1"}


def prompt_leg(shape, ms: float) -> dict:
    """Prefill of the benchmark's 2048-token prompt through the public call. The arithmetic counted is the four
    projections of every layer over all rows (2 * rows * N * K each) and causal attention (QK and PV over half the
    square); the denominator is the measured sustained BF16 GEMM rate."""
    rows, hidden, ffn = PROMPT, shape.hidden_size, shape.intermediate_size
    qkv = (shape.n_heads + 2 * shape.n_kv_heads) * shape.head_dim
    per_layer = 2.0 * rows * hidden * (qkv + shape.n_heads * shape.head_dim + 3 * ffn)
    attention = 2.0 * 2.0 * shape.n_heads * shape.head_dim * rows * rows / 2.0
    flops = shape.n_layers * (per_layer + attention)
    peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text()) if (ROOT / "MEASURED_PEAKS.json").exists() else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    achieved = flops / (ms * 1e-3) / 1e12
    return {"rows": rows, "ms": ms, "value": rows / (ms * 1e-3), "unit": "prompt tokens/s",
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak,
                         "peak_source": "measured (sustained)" if peaks else "fallback"},
            "what": "session prefill of the 2048-token prompt, host tokens in, median of 3 calls; projections on "
                    "tcgen05 (int4 dequantised in shared memory), one attention launch over all rows"}


def run_sessions_leg(package, torch, dist, rank: int, world: int, rounds: int, profile: bool = False):
    """The sharded-sessions configuration: 64 sessions of the Qwen2.5-7B-shaped AWQ model with seeded prompt lengths
    in [256, 8192], split evenly over the ranks, k = 4 drafts with p = 0.3 substitution. Every forward verifies ALL
    sessions of the rank at once (ei_batch_verify in its wide form: the stacked rows go through the projections as
    one tcgen05 GEMM, one attention launch serves all sessions); the same rounds with three sessions per forward
    (the <= 16-row kernels) are timed beside it. The histories are SYNTHETIC: every session's K/V rows are seeded
    with random BF16 values and adopted (no prefill of 270 000 prompt tokens); the drafts are each session's own
    greedy continuation from there."""
    syn, sharding = package.synthetic, package.sharding
    total_sessions, stack, k_drafts, p_sub = 64, 3, 4, 0.3
    rows = k_drafts + 1
    shape = syn.qwen25_7b_awq()
    capacity = shape.max_position_embeddings
    ids, lengths, batches = sharding.plan_sessions(total_sessions, world, rank, stack, 5, 256, 8192)
    model = package.Model(shape, syn.make_device_model(shape, seed=1))
    torch.cuda.empty_cache()
    sessions = [model.new_session(capacity, graph=True) for _ in ids]
    kv_width = shape.n_kv_heads * shape.head_dim
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    k_rows = torch.randn((8192, kv_width), device="cuda", generator=gen).to(torch.bfloat16)
    v_rows = torch.randn((8192, kv_width), device="cuda", generator=gen).to(torch.bfloat16)
    firsts = [int(t) for t in syn.make_prompt(11, len(ids), shape.vocab_size)]
    for session, length, first in zip(sessions, lengths, firsts):
        for layer in range(shape.n_layers):
            session.write_kv(layer, 0, k_rows[:length], v_rows[:length])
        session.adopt_history(length, first)
    del k_rows, v_rows
    everyone = package.runtime.SessionBatch(sessions)
    # Greedy continuation of every session, found with forwards of the very shape that is timed below (all
    # sessions, `rows` rows each, fillers as drafts): a row's bits do not depend on its place in the stack, but
    # they do depend on the kernels a row count selects, and with random-init weights a last-bit difference is
    # enough to change a greedy token.
    need = rounds * rows + rows
    continuation = [[first] for first in firsts]
    filler = [int(t) for t in syn.make_prompt(13, rows - 1, shape.vocab_size)]
    while min(len(c) for c in continuation) <= need:
        outs = everyone.verify([[c[-1]] + filler for c in continuation])
        for c, out in zip(continuation, outs):
            c.extend(out.tokens)
    drafts = [syn.corrupt_drafts(1000 + session_id, np.array(c, dtype=np.uint32), p_sub, shape.vocab_size)
              for session_id, c in zip(ids, continuation)]
    groups = [package.runtime.SessionBatch([sessions[i] for i in batch]) for batch in batches]
    pending = list(firsts)

    def rewind():
        for i, (session, length, first) in enumerate(zip(sessions, lengths, firsts)):
            session.truncate(length)
            session.set_pending(first)
            pending[i] = first

    def run(count: int, plan, handles):
        emitted_total = 0
        for _ in range(count):
            for batch, group in zip(plan, handles):
                inputs = []
                for i in batch:
                    offset = sessions[i].context_size() - lengths[i]
                    inputs.append([pending[i]] + [int(t) for t in drafts[i][offset + 1:offset + rows]])
                for i, out in zip(batch, group.verify(inputs)):
                    pending[i] = out.tokens[-1]
                    emitted_total += out.emitted
        return emitted_total

    def timed(count: int, plan, handles):
        rewind()
        run(2, plan, handles)                                  # warms (and, for the narrow form, captures the graphs)
        rewind()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        start = time.perf_counter()
        emitted = run(count, plan, handles)
        torch.cuda.synchronize()
        elapsed_ms = (time.perf_counter() - start) * 1e3
        if dist:
            dist.barrier()
        return emitted, elapsed_ms

    if profile:                                                # for `ncu --profile-from-start off`: one forward of all sessions
        rewind()
        run(1, [list(range(len(sessions)))], [everyone])
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        run(1, [list(range(len(sessions)))], [everyone])
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        return {"profiled": "one forward of all %d sessions" % len(sessions)}
    kv_per_token = 2 * shape.n_layers * kv_width * 2
    narrow_rounds = max(2, rounds // 6)
    narrow_emitted, narrow_ms = timed(narrow_rounds, batches, groups)
    emitted, elapsed_ms = timed(rounds, [list(range(len(sessions)))], [everyone])
    session_steps = rounds * len(sessions)
    bytes_moved = rounds * model.weight_bytes() + rounds * sum(lengths) * kv_per_token
    totals, times = sharding.aggregate(dist, torch, [emitted, session_steps, rounds, bytes_moved, narrow_emitted,
                                                     narrow_rounds * len(sessions), narrow_rounds * len(batches)],
                                       [elapsed_ms, narrow_ms], "cuda")
    del groups, everyone, sessions, model
    torch.cuda.empty_cache()
    peak, peak_kind = measured_peaks()
    achieved = totals[3] / (times[0] * 1e-3) / 1e9 / world
    return {
        "workload": ("qwen2.5-7b-shape AWQ (28 layers, hidden 3584, 28Q/4KV, q/k/v bias, FFN 18944, vocab 152064), "
                     "64 sessions, seeded prompt lengths in [256, 8192], k=4 (5 rows), p=0.3, all sessions of a GPU "
                     "per forward"),
        "history": "synthetic: K/V rows seeded with random BF16 values and adopted (no prompt prefill)",
        "sessions_total": total_sessions, "sessions_per_gpu": [len(sharding.session_shard(total_sessions, world, r))
                                                                 for r in range(world)],
        "rounds": rounds, "accepted_tokens_per_s": sharding.throughput(totals[0], times[0]),
        "session_steps_per_s": sharding.throughput(totals[1], times[0]),
        "tokens_per_session_step": totals[0] / totals[1], "ms_per_forward": times[0] * world / totals[2],
        "stacked_rows_per_forward": rows * len(ids),
        "timing": "host clock around the rounds (one host synchronisation per forward), maximum over ranks",
        "step_roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                          "peak_source": peak_kind, "note": "per GPU: weights once per forward + the live KV of its sessions"},
        "three_sessions_per_forward": {"rounds": narrow_rounds,
                                       "accepted_tokens_per_s": sharding.throughput(totals[4], times[1]),
                                       "session_steps_per_s": sharding.throughput(totals[5], times[1]),
                                       "ms_per_forward": times[1] * world / totals[6]},
    }


def run_native(args, rank: int, world: int, local_rank: int):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the verify step has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_module
        dist = dist_module
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    package = entry.load_package()
    package.abi.load_library()
    syn = package.synthetic
    if args.profile_sessions:
        leg = run_sessions_leg(package, torch, dist, rank, world, rounds=2, profile=True)
        if rank == 0:
            print(json.dumps(leg))
        if dist:
            dist.destroy_process_group()
        return
    shape = syn.qwen3_8b_awq(max_position_embeddings=CAPACITY)
    rows = K_DRAFTS + 1

    tensors = syn.make_device_model(shape, seed=0)
    model = package.Model(shape, tensors)
    keep_tensors = tensors if (rank == 0 and world == 1 and not args.no_reference_cuda) else None
    del tensors
    torch.cuda.empty_cache()
    session = model.new_session(CAPACITY, graph=True)
    prompt = syn.make_prompt(SEED, PROMPT, shape.vocab_size)
    session.prefill(prompt)
    # The prompt leg: the same prefill again, timed on the host around the public call (host tokens in, one
    # synchronisation at its end).
    prompt_ms = []
    for _ in range(3):
        torch.cuda.synchronize()
        begin = time.perf_counter()
        session.prefill(prompt)
        prompt_ms.append((time.perf_counter() - begin) * 1e3)
    if args.profile_prompt:
        torch.cuda.profiler.start()                    # for `ncu --profile-from-start off`: one prompt prefill only
        session.prefill(prompt)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        if rank == 0:
            print(json.dumps({"profiled": "one prefill of the %d-token prompt" % PROMPT, "ms": sorted(prompt_ms)[1]}))
        return
    first = package.runtime.greedy_token(session.read_logits(1)[0])

    # The model's own greedy continuation (ordinary decoding), then corrupted drafts.
    need = continuation_length(args.steps + args.warmup) - 1
    continuation, token = [first], first
    for _ in range(need):
        session.decode(token)
        token = package.runtime.greedy_token(session.read_logits(1)[0])
        continuation.append(token)
    continuation = np.array(continuation, dtype=np.uint32)
    drafts = syn.corrupt_drafts(SEED, continuation, P_SUBSTITUTE, shape.vocab_size)
    device_drafts = torch.from_numpy(drafts.view(np.int32)).cuda()
    stream = torch.cuda.ExternalStream(session.stream())

    def rewind():
        session.truncate(PROMPT)
        session.set_pending(first)

    def device_loop(steps: int):
        """Enqueues `steps` verify steps without host synchronisation; rewinds when the continuation runs out."""
        emitted, done, elapsed_ms, context_steps = 0, 0, 0.0, 0.0
        budget = (len(drafts) - rows) // rows          # steps that certainly fit before the drafts run out
        while done < steps:
            chunk = min(steps - done, budget)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(chunk):
                session.verify_enqueue(device_drafts, PROMPT, rows)
            end.record(stream)
            _, total = session.drain()
            elapsed_ms += start.elapsed_time(end)
            emitted += total
            done += chunk
            context_steps += chunk * (PROMPT + total / 2.0)   # the context grows linearly within a chunk
            rewind()
        return emitted, elapsed_ms, context_steps / max(1, steps)

    def host_loop(steps: int):
        """The same steps through ei_session_verify with host token buffers and one sync per step."""
        emitted, elapsed_ms, done = 0, 0.0, 0
        pending = first
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        while done < steps:
            i = session.context_size() - PROMPT
            if i + rows + 1 >= len(drafts):
                end.record(stream)
                torch.cuda.synchronize()
                elapsed_ms += start.elapsed_time(end)
                rewind()
                pending, i = first, 0
                start.record(stream)
            out = session.verify([pending] + [int(t) for t in drafts[i + 1:i + rows]])
            emitted += out.emitted
            pending = out.tokens[-1]
            done += 1
        end.record(stream)
        torch.cuda.synchronize()
        elapsed_ms += start.elapsed_time(end)
        return emitted, elapsed_ms

    rewind()
    device_loop(max(3, args.warmup))                   # captures the graph and warms the caches
    rewind()
    _, warm_ms, _ = device_loop(max(3, args.warmup))   # the same steps again: their time sizes the timed regions
    # The timed region is exactly `steps` steps; it is repeated until the regions cover about a second, so that
    # the reported (median) region is not a 50 ms sample.
    regions = int(min(64, max(1, np.ceil(1000.0 / max(1e-3, warm_ms / max(3, args.warmup) * args.steps)))))
    if args.profile_region:
        regions = 1
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    if args.profile_region:
        torch.cuda.profiler.start()                    # for `ncu --profile-from-start off`: the timed steps only
    region_emitted, region_ms, region_context = [], [], []
    for _ in range(regions):
        if dist:
            dist.barrier()
        torch.cuda.synchronize()
        emitted, elapsed_ms, mean_context = device_loop(args.steps)
        torch.cuda.synchronize()
        region_emitted.append(emitted)
        region_ms.append(elapsed_ms)
        region_context.append(mean_context)
    if args.profile_region:
        torch.cuda.profiler.stop()
    if dist:
        dist.barrier()
    clocks = sampler.stop()

    host_loop(max(3, args.warmup))
    rewind()
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    e2e_emitted, e2e_ms = host_loop(args.steps)
    if dist:
        dist.barrier()

    # Per region: tokens summed and times maximised over the ranks; the median region is the reported one.
    totals, times = package.sharding.aggregate(dist, torch, region_emitted + [e2e_emitted], region_ms + [e2e_ms], "cuda")
    order = sorted(range(regions), key=lambda r: times[r])
    median = order[len(order) // 2]
    value = package.sharding.throughput(totals[median], times[median])
    e2e_value = package.sharding.throughput(totals[regions], times[regions])
    ms_per_step = times[median] / args.steps
    mean_context = region_context[median]
    launches = session.launches_per_step(rows)

    line = None
    if rank == 0:
        peak, peak_kind = measured_peaks()
        weight_bytes = model.weight_bytes()
        kv_per_token = 2 * shape.n_layers * shape.n_kv_heads * shape.head_dim * 2
        step_bytes = weight_bytes + kv_per_token * mean_context + rows * shape.hidden_size * 2
        step_achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 activations, int4 group-128 weights, fp32 accumulation", "data": "synthetic",
            "config": workload_config(package, args.steps, args.warmup),
            "l2_policy": "inputs larger than L2 (4.85 GB of weights per step)",
            "timed_regions": {"count": regions, "steps_each": args.steps, "reported": "median region",
                              "ms_per_step_min": times[order[0]] / args.steps,
                              "ms_per_step_median": ms_per_step,
                              "ms_per_step_max": times[order[-1]] / args.steps},
            "tokens_per_step_measured": totals[median] / (args.steps * world),
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": 96,
                    "ms_per_step": times[regions] / args.steps},
            "gpu_launches": int(launches * args.steps),
            "prompt_leg": prompt_leg(shape, sorted(prompt_ms)[1]),
            "step_roofline": {"bound": "hbm", "achieved": step_achieved, "peak": peak, "unit": "GB/s",
                              "frac": step_achieved / peak, "peak_source": peak_kind, "bytes_per_step": step_bytes,
                              "launches_per_step": int(launches)},
        }
    del session
    if rank == 0:
        kernel_seconds, kernel_bytes = time_dominant_kernel(package, torch, shape, layers=36, rows=rows, repeats=5)
        achieved = kernel_bytes / kernel_seconds / 1e9
        traffic_path = ROOT / "profiles" / "awq_tma_kernel_gate_up_24576x4096_m9.traffic.json"
        traffic = json.loads(traffic_path.read_text()) if traffic_path.exists() else None
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                            "traffic": traffic["dram_bytes_per_launch"] if traffic else None,
                            "traffic_source": str(traffic_path.relative_to(ROOT)) if traffic else None,
                            "kernel": "awq_tma_kernel (int4 gate|up projection + SwiGLU) N=24576 K=4096 M=9",
                            "us_per_launch": kernel_seconds * 1e6, "algorithmic_bytes": kernel_bytes,
                            "peak_source": peak_kind}
        if keep_tensors is not None:
            oracle = entry.load_oracle()
            if oracle.reference_available():
                try:
                    step_seconds, tokens, reference_prompt_seconds = time_reference_cuda(package, oracle, torch, shape, keep_tensors, drafts, first,
                                                               max(10, min(args.steps, 40)))
                    same_drafts = line["config"]["tokens_per_step"]
                    line["reference_cuda"] = {
                        "ms_per_step": step_seconds * 1e3, "value": same_drafts / step_seconds, "unit": UNIT,
                        "speedup_e2e_ms_per_step": step_seconds * 1e3 / line["e2e"]["ms_per_step"],
                        "tokens_per_step_observed": tokens,
                        "prompt_ms": reference_prompt_seconds * 1e3,
                        "prompt_speedup": reference_prompt_seconds * 1e3 / line["prompt_leg"]["ms"],
                        "what": "unmodified reference (oracle/_ref, its kernels recompiled for sm_100): "
                                "prefill_eager of 9 rows + op::cuda::sample + host acceptance, same model, GPU and "
                                "step shape; `value` uses this bench's accept lengths (the step time does not depend "
                                "on acceptance; the reference's own greedy path leaves this library's continuation "
                                "within a few tokens on a random-init model, so it accepts next to nothing of "
                                "these drafts)"}
                except Exception as error:  # the reference arm must not take the bench line down with it
                    line["reference_cuda"] = {"unavailable": str(error)[:200]}
            else:
                line["reference_cuda"] = {"unavailable": "oracle/_ref is not built"}
    keep_tensors = None
    if rank == 0 and not args.no_sessions_leg:
        line["speculative_leg"] = run_speculative_leg(package, torch, model, rounds=24)
    del model
    torch.cuda.empty_cache()
    if not args.no_sessions_leg:
        leg = run_sessions_leg(package, torch, dist, rank, world, rounds=max(4, min(args.steps, 24)))
        if rank == 0:
            line["sessions_leg"] = leg
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            oracle = entry.load_oracle()
            threads = os.cpu_count() or 1
            cpu = CpuStep(oracle, package, threads)
            cpu.step()
            cpu_times = [cpu.step() for _ in range(2)]
            step_seconds = sum(cpu_times) / len(cpu_times)
            one_thread_layer = cpu.one_layer_single_thread()
            line["cpu_baseline"] = {"value": line["config"]["tokens_per_step"] / step_seconds, "unit": UNIT,
                                    "cores": threads, "kind": "port", "sample": cpu.sample + "; 2 timed steps",
                                    "ms_per_step": step_seconds * 1e3,
                                    "one_thread_ms_per_layer_pass": one_thread_layer * 1e3}
        print(json.dumps(line))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=None, help="default 60 (native), 5 (--impl reference)")
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-reference-cuda", action="store_true")
    parser.add_argument("--no-sessions-leg", action="store_true")
    parser.add_argument("--profile-region", action="store_true",
                        help="bracket the timed steps with cudaProfilerStart/Stop (for a profiler started with "
                             "profiling off); the numbers of such a run are not bench values")
    parser.add_argument("--profile-sessions", action="store_true",
                        help="run only the 64-session leg and bracket one forward of all sessions the same way")
    parser.add_argument("--profile-prompt", action="store_true",
                        help="bracket one prefill of the prompt the same way and stop after it")
    args = parser.parse_args()
    if args.steps is None:
        args.steps = 5 if args.impl == "reference" else 60
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_native(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
