"""Operator sweep of the verify path on one GPU (the benchmark suite's operator configuration):

  AWQ int4 linear   M in {1,2,4,8,9,16} x (N,K) in {(4096,4096),(1024,4096),(24576,4096),(4096,12288)}
  verify attention  q_len in {1,5,9}, 32 Q / 8 KV heads, head_dim 128, KV length in {512,2048,8192,32768}
  dense BF16 head   (151936, 4096)
  prompt GEMM       the same AWQ shapes at T in {128, 512, 2048} rows (the tcgen05 kernel the linear operators
                    take above 32 rows), reported in TFLOP/s against the measured BF16 GEMM rate

Every case cycles over enough distinct operand sets to exceed L2 (126 MB), is replayed from a CUDA graph so
that host launch cost is excluded, and is timed with CUDA events. Prints one line per case:
time per launch, algorithmic bytes, achieved GB/s and the fraction of the measured HBM peak.

    python opbench.py                       # full sweep
    python opbench.py --op awq --n 24576 --k 4096 --rows 9 --fused   # one case (for ncu)
    python opbench.py --op prompt --n 4096 --k 4096 --rows 512 --copies 2 --iters 1
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402


def hbm_peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    return float(json.loads(path.read_text())["hbm_gbs"]) if path.exists() else 6650.0


def tensor_peak() -> float:
    path = ROOT / "MEASURED_PEAKS.json"
    return float(json.loads(path.read_text())["bf16_tflops"]) if path.exists() else 1590.0


def graph_time(torch, stream, body, iters: int) -> float:
    """Microseconds per call of `body` (a whole pass over the operand sets), replayed from a CUDA graph."""
    with torch.cuda.stream(stream):
        body()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            body()
        graph.replay()
        stream.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(iters):
            graph.replay()
        end.record(stream)
        stream.synchronize()
    return start.elapsed_time(end) * 1e3 / iters


def awq_bytes(n: int, k: int, rows: int, out_columns: int) -> int:
    groups = k // 128
    return n * k // 2 + n * groups * 2 + n * ((groups + 7) // 8) * 4 + rows * k * 2 + rows * out_columns * 2


def bench_awq(torch, package, stream, ctx, n, k, rows, fused, iters, copies=None):
    ops = package.operators
    gen = torch.Generator(device="cuda")
    gen.manual_seed(n + k)
    groups = k // 128
    copies = copies or max(2, int(300e6 / (n * k / 2)) + 1)
    keep, weights = [], []
    for _ in range(copies):
        q = torch.randint(-2**31, 2**31 - 1, (n, k // 8), dtype=torch.int32, device="cuda", generator=gen)
        z = torch.randint(-2**31, 2**31 - 1, (n, (groups + 7) // 8), dtype=torch.int32, device="cuda", generator=gen)
        s = (torch.rand((n, groups), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
        keep.append((q, z, s))
        weights.append(ops.prepare_awq(q, s, z, 128, k))
    x = torch.randn((rows, k), device="cuda", generator=gen).to(torch.bfloat16)
    columns = n // 2 if fused else n
    out = torch.empty((rows, columns), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(max(16, ops.linear_scratch_bytes(rows, k, n)), dtype=torch.uint8, device="cuda")

    def body():
        for w in weights:
            if fused:
                ops.awq_gate_up_silu(ctx, x, w, out)
            else:
                ops.awq_linear(ctx, x, w, out, scratch)

    us = graph_time(torch, stream, body, iters) / copies
    return us, awq_bytes(n, k, rows, columns)


def bench_dense(torch, package, stream, ctx, n, k, rows, iters):
    ops = package.operators
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1)
    copies = max(2, int(300e6 / (n * k * 2)) + 1)
    mats = [torch.randn((n, k), device="cuda", generator=gen).to(torch.bfloat16) for _ in range(copies)]
    weights = [ops.prepare_dense(m.t()) for m in mats]
    x = torch.randn((rows, k), device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(max(16, ops.linear_scratch_bytes(rows, k, n)), dtype=torch.uint8, device="cuda")

    def body():
        for w in weights:
            ops.linear(ctx, x, w, out, scratch)

    us = graph_time(torch, stream, body, iters) / copies
    return us, n * k * 2 + rows * k * 2 + rows * n * 2


def bench_attention(torch, package, stream, ctx, rows, length, iters, heads=32, kv_heads=8):
    ops = package.operators
    gen = torch.Generator(device="cuda")
    gen.manual_seed(length)
    kv_bytes = 2 * length * kv_heads * 128 * 2
    copies = max(2, int(300e6 / kv_bytes) + 1)
    ks = [torch.randn((length, kv_heads, 128), device="cuda", generator=gen).to(torch.bfloat16) for _ in range(copies)]
    vs = [torch.randn((length, kv_heads, 128), device="cuda", generator=gen).to(torch.bfloat16) for _ in range(copies)]
    q = torch.randn((rows, heads, 128), device="cuda", generator=gen).to(torch.bfloat16)
    out = torch.empty_like(q)
    scratch = torch.empty(ops.attention_scratch_bytes(rows, heads, 128, length), dtype=torch.uint8, device="cuda")

    def body():
        for k, v in zip(ks, vs):
            ops.attention_prefill(ctx, q, k, v, out, length - rows, scratch)

    us = graph_time(torch, stream, body, iters) / copies
    return us, kv_bytes + 2 * rows * heads * 128 * 2


def main():
    import torch

    parser = argparse.ArgumentParser()
    parser.add_argument("--op", default="all", choices=["all", "awq", "dense", "attention", "prompt"])
    parser.add_argument("--n", type=int, default=24576)
    parser.add_argument("--k", type=int, default=4096)
    parser.add_argument("--rows", type=int, default=9)
    parser.add_argument("--length", type=int, default=2048)
    parser.add_argument("--fused", action="store_true", help="fused gate/up SwiGLU projection instead of a plain linear")
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--copies", type=int, default=0)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("opbench needs a CUDA device")
    package = entry.load_package()
    package.abi.load_library()
    stream = torch.cuda.Stream()
    ctx = package.operators.prepare_execution_context(stream.cuda_stream)
    peak = hbm_peak()

    def report(name, us, nbytes):
        gbs = nbytes / us / 1e3
        print(f"{name:44s} {us:9.2f} us  {nbytes / 1e6:9.2f} MB  {gbs:8.1f} GB/s  {gbs / peak:6.3f} of measured HBM peak",
              flush=True)

    def report_prompt(n, k, rows, us):
        tflops = 2.0 * rows * n * k / us / 1e6
        print(f"{f'prompt awq N={n} K={k} T={rows}':44s} {us:9.2f} us  {2.0 * rows * n * k / 1e9:9.2f} GFLOP  "
              f"{tflops:8.1f} TFLOP/s  {tflops / tensor_peak():6.3f} of measured BF16 GEMM peak (burst)", flush=True)

    if args.op == "prompt":
        us, _ = bench_awq(torch, package, stream, ctx, args.n, args.k, args.rows, False, args.iters, args.copies or None)
        report_prompt(args.n, args.k, args.rows, us)
        return
    if args.op == "awq":
        us, nbytes = bench_awq(torch, package, stream, ctx, args.n, args.k, args.rows, args.fused, args.iters,
                               args.copies or None)
        report(f"awq{'_gate_up_silu' if args.fused else ''} N={args.n} K={args.k} M={args.rows}", us, nbytes)
        return
    if args.op == "dense":
        us, nbytes = bench_dense(torch, package, stream, ctx, args.n, args.k, args.rows, args.iters)
        report(f"dense N={args.n} K={args.k} M={args.rows}", us, nbytes)
        return
    if args.op == "attention":
        us, nbytes = bench_attention(torch, package, stream, ctx, args.rows, args.length, args.iters)
        report(f"attention q_len={args.rows} L={args.length} 32Q/8KV", us, nbytes)
        return
    for n, k in [(4096, 4096), (1024, 4096), (24576, 4096), (4096, 12288)]:
        for rows in [1, 2, 4, 8, 9, 16]:
            us, nbytes = bench_awq(torch, package, stream, ctx, n, k, rows, False, args.iters)
            report(f"awq N={n} K={k} M={rows}", us, nbytes)
    for rows in [1, 9, 16]:
        us, nbytes = bench_awq(torch, package, stream, ctx, 24576, 4096, rows, True, args.iters)
        report(f"awq_gate_up_silu N=24576 K=4096 M={rows}", us, nbytes)
    for rows in [1, 9, 16]:
        us, nbytes = bench_dense(torch, package, stream, ctx, 151936, 4096, rows, args.iters)
        report(f"dense N=151936 K=4096 M={rows}", us, nbytes)
    for n, k in [(6144, 4096), (4096, 4096), (24576, 4096), (4096, 12288)]:
        for rows in [128, 512, 2048]:
            us, _ = bench_awq(torch, package, stream, ctx, n, k, rows, False, args.iters)
            report_prompt(n, k, rows, us)
    for length in [512, 2048, 8192, 32768]:
        for rows in [1, 5, 9]:
            us, nbytes = bench_attention(torch, package, stream, ctx, rows, length, args.iters)
            report(f"attention q_len={rows} L={length} 32Q/8KV", us, nbytes)


if __name__ == "__main__":
    main()
