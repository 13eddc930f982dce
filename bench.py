"""Benchmark of the speculative-decoding verify step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one session per GPU; weights replicated, no collective - sessions are independent):
Qwen3-8B-shaped AWQ model (36 layers, hidden 4096, 32 Q / 8 KV heads, head_dim 128, FFN 12288, vocab 151936,
int4 group-128 linears, BF16 embeddings / norms / lm_head), context capacity 4096, seeded 2048-token prompt,
k = 8 drafts = the model's own greedy continuation with p = 0.2 random substitution. Random-init synthetic
weights stand in for a checkpoint. A step is one verify step: one forward of [pending, 8 drafts] over the
session's KV cache, greedy acceptance and KV commit.

Prints ONE JSON line:
  value        accepted tokens/s, device-resident loop (drafts, pending token and context length on the device,
               steps enqueued back to back, one drain at the end), whole job over all GPUs
  e2e          the same metric through ei_session_verify with host token buffers: per step an H2D copy of the
               tokens, the graph, a D2H copy of the result and one host synchronisation
  roofline     the dominant kernel (fused gate/up int4 projection, 53 MB of weights per launch) timed alone with
               CUDA events over the 36 layers' distinct weights (1.9 GB > L2), algorithmic bytes / time / measured
               HBM peak
  step_roofline  the whole step: (prepared weight bytes + live KV bytes) / step time / measured HBM peak
  cpu_baseline the CPU oracle port of the reference's FP32 executor, timed on the host cores on a bounded sample
`--impl reference` times that CPU implementation alone (rank 0 only).
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
EXPECTED_EMITTED = 1 + sum((1 - P_SUBSTITUTE) ** i for i in range(1, K_DRAFTS + 1))  # 4.33 tokens per step


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


def cpu_verify_sample(oracle, package, threads: int, repeats: int):
    """Times the CPU oracle (FP32 mode: the reference executor's arithmetic) on one decoder layer of the 8B shape,
    9 rows at context 2048, and once on the lm_head; returns (seconds per full 36-layer step, description)."""
    shape = package.synthetic.qwen3_8b_awq()
    lib = oracle.oracle_library()
    lib.vo_set_threads(threads)
    rng = np.random.default_rng(0)
    layer_shape = package.Shape(vocab_size=8, n_layers=1, n_heads=shape.n_heads, n_kv_heads=shape.n_kv_heads,
                                hidden_size=shape.hidden_size, intermediate_size=shape.intermediate_size,
                                max_position_embeddings=CAPACITY, qk_norm=True)
    H, F = shape.hidden_size, shape.intermediate_size
    qw, kvw = shape.n_heads * 128, shape.n_kv_heads * 128

    def dense(out, inp):
        return [(0, package.synthetic.float_to_bf16(rng.standard_normal((out, inp), dtype=np.float32) * np.float32(0.02)))]

    ones = lambda n: [(0, package.synthetic.float_to_bf16(np.ones(n, dtype=np.float32)))]  # noqa: E731
    tensors = {"token_embeddings.weight": dense(8, H), "rms_out_w": ones(H), "lm_head": dense(8, H),
               "rms_att_w0": ones(H), "rms_ffn_w0": ones(H), "q_norm0": ones(128), "k_norm0": ones(128),
               "wq0": dense(qw, H), "wk0": dense(kvw, H), "wv0": dense(kvw, H), "wo0": dense(H, qw),
               "w_gate0": dense(F, H), "w_up0": dense(F, H), "w_down0": dense(H, F)}
    layer = oracle.OracleModel(layer_shape, tensors, capacity=CAPACITY)
    tokens = np.arange(K_DRAFTS + 1, dtype=np.uint32) % 8
    layer_times = []
    for _ in range(repeats):
        layer.resize(PROMPT)                                   # cached keys/values present (their values are irrelevant)
        start = time.perf_counter()
        layer.forward(tokens, 0)
        layer_times.append(time.perf_counter() - start)
    x = rng.standard_normal((K_DRAFTS + 1, H), dtype=np.float32)
    head_rows = 8192                                           # a slice of the 151936-row lm_head, scaled up
    w = rng.standard_normal((head_rows, H), dtype=np.float32)
    start = time.perf_counter()
    oracle.op_linear(x, w, None)
    head = (time.perf_counter() - start) * shape.vocab_size / head_rows
    per_layer = statistics.median(layer_times)
    step = shape.n_layers * per_layer + head
    sample = (f"CPU oracle port of the reference FP32 executor: {repeats} x one decoder layer of the 8B shape "
              f"(9 rows at context {PROMPT}) + a {head_rows}-row slice of the lm_head, extrapolated to 36 layers + "
              f"151936 rows; {per_layer:.3f} s/layer, {head:.3f} s head")
    return step, sample, layer_times


WORKLOAD = ("qwen3-8b-shape AWQ verify step: 36 layers, hidden 4096, 32Q/8KV, FFN 12288, vocab 151936, k=8 (9 rows), "
            "prompt 2048, capacity 4096, p=0.2 draft substitution, one session per GPU")


def run_reference(args, rank: int):
    if rank != 0:
        return
    package, oracle = entry.load_package(), entry.load_oracle()
    threads = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        cpu_verify_sample(oracle, package, threads, 1)
    step_seconds, sample, times = cpu_verify_sample(oracle, package, threads, max(1, args.steps))
    value = EXPECTED_EMITTED / step_seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_seconds * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sessions_per_gpu": 1, "executor": "CPU, FP32, AWQ weights dequantised",
                   "tokens_per_step": EXPECTED_EMITTED},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
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
    shape = syn.qwen3_8b_awq(max_position_embeddings=CAPACITY)
    rows = K_DRAFTS + 1

    tensors = syn.make_device_model(shape, seed=0)
    model = package.Model(shape, tensors)
    del tensors
    torch.cuda.empty_cache()
    session = model.new_session(CAPACITY, graph=True)
    prompt = syn.make_prompt(rank, PROMPT, shape.vocab_size)
    session.prefill(prompt)
    first = package.runtime.greedy_token(session.read_logits(1)[0])

    # The model's own greedy continuation (ordinary decoding), then corrupted drafts.
    total_steps = args.steps + args.warmup
    need = min(CAPACITY - PROMPT - rows - 1, total_steps * rows + rows)
    continuation, token = [first], first
    for _ in range(need):
        session.decode(token)
        token = package.runtime.greedy_token(session.read_logits(1)[0])
        continuation.append(token)
    continuation = np.array(continuation, dtype=np.uint32)
    drafts = syn.corrupt_drafts(rank, continuation, P_SUBSTITUTE, shape.vocab_size)
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
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    if args.profile_region:
        torch.cuda.profiler.start()                    # for `ncu --profile-from-start off`: the timed steps only
    emitted, elapsed_ms, mean_context = device_loop(args.steps)
    torch.cuda.synchronize()
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

    totals, times = package.sharding.aggregate(dist, torch, [emitted, e2e_emitted], [elapsed_ms, e2e_ms], "cuda")
    value = package.sharding.throughput(totals[0], times[0])
    e2e_value = package.sharding.throughput(totals[1], times[1])
    ms_per_step = times[0] / args.steps

    if rank == 0:
        peak, peak_kind = measured_peaks()
        weight_bytes = model.weight_bytes()
        kv_per_token = 2 * shape.n_layers * shape.n_kv_heads * shape.head_dim * 2
        step_bytes = weight_bytes + kv_per_token * mean_context + rows * shape.hidden_size * 2
        step_achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        launches = session.launches_per_step(rows)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 activations, int4 group-128 weights, fp32 accumulation", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "sessions_per_gpu": 1, "l2_policy": "inputs larger than L2 (4.85 GB of weights per step)",
                       "tokens_per_step": totals[0] / (args.steps * world)},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": rows * 4, "d2h_bytes_per_step": 96,
                    "ms_per_step": times[1] / args.steps},
            "gpu_launches": int(launches * args.steps),
            "step_roofline": {"bound": "hbm", "achieved": step_achieved, "peak": peak, "unit": "GB/s",
                              "frac": step_achieved / peak, "peak_source": peak_kind, "bytes_per_step": step_bytes,
                              "launches_per_step": int(launches)},
        }
        del session
        kernel_seconds, kernel_bytes = time_dominant_kernel(package, torch, shape, layers=36, rows=rows, repeats=5)
        achieved = kernel_bytes / kernel_seconds / 1e9
        line["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                            "traffic": 52_524_000,  # ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch
                            "traffic_source": "profiles/awq_tma_kernel_gate_up_24576x4096_m9.md", "kernel": "awq_tma_kernel (int4 gate|up projection + SwiGLU) N=24576 K=4096 M=9",
                            "us_per_launch": kernel_seconds * 1e6, "algorithmic_bytes": kernel_bytes,
                            "peak_source": peak_kind}
        if world == 1 and not args.no_cpu_baseline:
            oracle = entry.load_oracle()
            threads = os.cpu_count() or 1
            step_seconds, sample, _ = cpu_verify_sample(oracle, package, threads, 3)
            line["cpu_baseline"] = {"value": (totals[0] / args.steps) / step_seconds, "unit": UNIT, "cores": threads,
                                    "kind": "port", "sample": sample, "ms_per_step": step_seconds * 1e3}
        print(json.dumps(line))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=60)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="native", choices=["native", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--profile-region", action="store_true",
                        help="bracket the timed steps with cudaProfilerStart/Stop (for a profiler started with "
                             "profiling off); the numbers of such a run are not bench values")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_native(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
