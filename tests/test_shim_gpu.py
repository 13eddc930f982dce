"""The drop-in C++ header (include/operators/cuda/execution.hpp: namespace op::cuda, the reference's signatures)
driven by a C++ caller on the GPU: the operators a decoder layer calls run through it on seeded inputs and must
give, bit for bit, what the same library gives through the ctypes binding; the sampling contract of the reference
(operators/src/cuda/execution.cu:455-475, operators/tests/operators_cuda_sampling_test.cu:230-259: an invalid or
non-greedy policy is rejected before any write) is checked inside the C++ program."""
import shutil
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu

PROGRAM = r"""
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "operators/cuda/execution.hpp"

using B = unsigned short;  // BF16 payload: the library only sees pointers
static void ok(cudaError_t e) { if (e != cudaSuccess) { std::printf("cuda: %s\n", cudaGetErrorString(e)); std::exit(2); } }
template <typename T> T* device(const std::vector<T>& h) {
  T* d = nullptr; ok(cudaMalloc(&d, h.size() * sizeof(T)));
  ok(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice)); return d;
}
template <typename T> std::vector<T> read(FILE* f, size_t n) {
  std::vector<T> v(n); if (std::fread(v.data(), sizeof(T), n, f) != n) { std::printf("short input\n"); std::exit(3); } return v;
}
template <typename T> void write(FILE* f, const T* d, size_t n) {
  std::vector<T> h(n); ok(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost)); std::fwrite(h.data(), sizeof(T), n, f);
}
template <typename F> bool rejected(F&& f) { try { f(); } catch (const std::invalid_argument&) { return true; } catch (...) {} return false; }

int main(int argc, char** argv) {
  const size_t rows = 9, K = 1024, N = 512, groups = K / 128, heads = 8, kv_heads = 2, d = 128, L = 300, V = 4096;
  FILE* in = std::fopen(argv[1], "rb"); FILE* out = std::fopen(argv[2], "wb");
  auto x = read<B>(in, rows * K); auto norm_w = read<B>(in, K);
  auto qweight = read<int>(in, N * K / 8); auto scales = read<B>(in, N * groups); auto zeros = read<int>(in, N * 1);
  auto bias = read<B>(in, N);
  auto q = read<B>(in, rows * heads * d); auto k = read<B>(in, L * kv_heads * d); auto v = read<B>(in, L * kv_heads * d);
  auto table = read<float>(in, 512 * d); auto logits = read<B>(in, rows * V);
  cudaStream_t stream; ok(cudaStreamCreate(&stream));
  const auto ctx = op::cuda::prepare_execution_context(nullptr, stream);
  op::cuda::bind_execution_context(ctx);

  B *dx = device(x), *dw = device(norm_w), *dnormed = nullptr; ok(cudaMalloc(&dnormed, rows * K * 2));
  op::cuda::rms_norm<B>(ctx, {dx, rows * K}, {dw, K}, {dnormed, rows * K}, rows, K, 1e-6f);

  int *dq = device(qweight), *dz = device(zeros); B *ds = device(scales), *db = device(bias), *dy = nullptr;
  ok(cudaMalloc(&dy, rows * N * 2));
  const auto weight = op::cuda::prepare_awq<B>(TensorView<const int, 2>::contiguous(dq, {N, K / 8}),
                                               TensorView<const B, 2>::contiguous(ds, {N, groups}),
                                               TensorView<const int, 2>::contiguous(dz, {N, 1}), 128, K,
                                               TensorView<const B, 1>::contiguous(db, {N}));
  op::cuda::awq_linear<B>(ctx, TensorView<const B, 2>::contiguous(dnormed, {rows, K}), weight,
                          TensorView<B, 2>::contiguous(dy, {rows, N}));

  B* dact = nullptr; ok(cudaMalloc(&dact, rows * (N / 2) * 2));
  // gate = columns [0, N/2), up = columns [N/2, N) of row 0..: here simply the two halves of the flat buffer
  op::cuda::silu_multiply<B>({dy, rows * N / 2}, {dy + rows * N / 2, rows * N / 2}, {dact, rows * N / 2}, stream);

  B *dqh = device(q), *dk = device(k), *dv = device(v), *dattn = nullptr; ok(cudaMalloc(&dattn, rows * heads * d * 2));
  float* dtable = device(table);
  op::cuda::rope_precomputed<B>(ctx, TensorView<B, 3>::contiguous(dqh, {rows, heads, d}),
                                TensorView<const float, 2>::contiguous(dtable, {512, d}), L - rows);
  op::cuda::attention_prefill<B>(ctx, TensorView<const B, 3>::contiguous(dqh, {rows, heads, d}),
                                 TensorView<const B, 3>::contiguous(dk, {L, kv_heads, d}),
                                 TensorView<const B, 3>::contiguous(dv, {L, kv_heads, d}),
                                 TensorView<B, 3>::contiguous(dattn, {rows, heads, d}), L - rows);

  B* dlogits = device(logits); unsigned* dtokens = nullptr; ok(cudaMalloc(&dtokens, rows * 4));
  ok(cudaMemset(dtokens, 0xee, rows * 4));
  const auto plan = op::cuda::prepare_sampling(ctx, V);
  unsigned char* dwork = nullptr; ok(cudaMalloc(&dwork, plan.total_bytes));
  const auto lv = TensorView<const B, 2>::contiguous(dlogits, {rows, V});
  const auto tv = TensorView<unsigned, 1>::contiguous(dtokens, {rows});
  const auto wv = TensorView<unsigned char, 1>::contiguous(dwork, {plan.total_bytes});
  int contract = 0;
  contract += rejected([&] { op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 0.7f, 0.9f, 0, nullptr); });       // top_k = 0
  contract += rejected([&] { op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 0.7f, 1.5f, 1, nullptr); });       // top_p > 1
  contract += rejected([&] { op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 0.7f, 0.9f, 2048, nullptr); });    // > 1024 candidates
  contract += rejected([&] { op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 0.7f, 0.9f, 5, nullptr); });       // stochastic, no RNG
  contract += rejected([&] { op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 0.7f, 0.9f, 5, reinterpret_cast<curandState*>(dwork)); });
  ok(cudaStreamSynchronize(stream));
  std::vector<unsigned> untouched(rows); ok(cudaMemcpy(untouched.data(), dtokens, rows * 4, cudaMemcpyDeviceToHost));
  for (unsigned t : untouched) contract += t == 0xeeeeeeeeu ? 0 : -100;                                          // rejected before any write
  op::cuda::sample<B>(ctx, lv, tv, {}, wv, plan, 1.0f, 1.0f, 1, nullptr);                                        // greedy
  // attention beyond the built-in split buffer is refused with the same exception class
  contract += rejected([&] {
    op::cuda::attention_prefill<B>(ctx, TensorView<const B, 3>::contiguous(dqh, {16, 32, d}),
                                   TensorView<const B, 3>::contiguous(dk, {8192, 8, d}),
                                   TensorView<const B, 3>::contiguous(dv, {8192, 8, d}),
                                   TensorView<B, 3>::contiguous(dattn, {16, 32, d}), 8192 - 16); });
  ok(cudaStreamSynchronize(stream));
  write(out, dnormed, rows * K); write(out, dy, rows * N); write(out, dact, rows * N / 2);
  write(out, dqh, rows * heads * d); write(out, dattn, rows * heads * d); write(out, dtokens, rows);
  std::fclose(out);
  std::printf("contract %d\n", contract);
  return contract == 6 ? 0 : 1;
}
"""


def test_cpp_caller_through_the_drop_in_header_matches_ctypes(cuda, package, tmp_path):
    torch, ops, syn = cuda, package.operators, package.synthetic
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    rows, K, N, heads, kv_heads, d, L, V = 9, 1024, 512, 8, 2, 128, 300, 4096
    rng = np.random.default_rng(3)
    f2b = syn.float_to_bf16
    x = f2b(rng.standard_normal((rows, K), dtype=np.float32))
    norm_w = f2b(1.0 + 0.1 * rng.standard_normal(K, dtype=np.float32))
    qweight, scales, zeros = syn.awq_triple(3, "shim", N, K)
    bias = f2b(rng.standard_normal(N, dtype=np.float32) * 0.1)
    q = f2b(rng.standard_normal((rows, heads, d), dtype=np.float32))
    k = f2b(rng.standard_normal((L, kv_heads, d), dtype=np.float32))
    v = f2b(rng.standard_normal((L, kv_heads, d), dtype=np.float32))
    table = ops.build_rope_table(512, d, 1e6)
    logits = f2b(rng.standard_normal((rows, V), dtype=np.float32))
    blob = tmp_path / "inputs.bin"
    with open(blob, "wb") as handle:
        for array in (x, norm_w, qweight, scales, zeros, bias, q, k, v, table, logits):
            handle.write(np.ascontiguousarray(array).tobytes())
    source, binary, result_path = tmp_path / "caller.cpp", tmp_path / "caller", tmp_path / "outputs.bin"
    source.write_text(PROGRAM)
    library = Path(package.abi.LIB_PATH)
    cuda_home = Path("/usr/local/cuda")
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", str(ROOT / "include"), "-I", str(cuda_home / "include"),
                    str(source), "-o", str(binary), f"-L{library.parent}", "-ledge_infer_b200",
                    f"-L{cuda_home / 'lib64'}", "-lcudart", f"-Wl,-rpath,{library.parent}",
                    f"-Wl,-rpath,{cuda_home / 'lib64'}"], check=True)
    run = subprocess.run([str(binary), str(blob), str(result_path)], capture_output=True, text=True)
    assert run.returncode == 0, run.stdout + run.stderr
    raw = np.fromfile(result_path, dtype=np.uint8)

    # The same calls through ctypes.
    def dev(bits):
        return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)

    ctx = ops.prepare_execution_context(0)
    dx, dnormed = dev(x), torch.empty((rows, K), dtype=torch.bfloat16, device="cuda")
    ops.rms_norm(ctx, dx, dev(norm_w), dnormed, rows, K, 1e-6)
    weight = ops.prepare_awq(torch.from_numpy(qweight).cuda(), dev(scales), torch.from_numpy(zeros).cuda(), 128, K,
                             dev(bias))
    dy = torch.empty((rows, N), dtype=torch.bfloat16, device="cuda")
    ops.awq_linear(ctx, dnormed, weight, dy, None)
    flat = dy.view(-1)
    dact = torch.empty(rows * N // 2, dtype=torch.bfloat16, device="cuda")
    ops.silu_multiply(ctx, flat[:rows * N // 2], flat[rows * N // 2:], dact)
    dq, dattn = dev(q), torch.empty((rows, heads, d), dtype=torch.bfloat16, device="cuda")
    ops.rope_precomputed(ctx, dq, torch.from_numpy(table).cuda(), L - rows)
    ops.attention_prefill_static(ctx, dq, dev(k), dev(v), dattn, L - rows)
    tokens = torch.empty(rows, dtype=torch.int32, device="cuda")
    scratch = torch.empty(ops.sample_scratch_bytes(rows, V), dtype=torch.uint8, device="cuda")
    ops.sample_greedy(ctx, dev(logits), tokens, scratch)
    torch.cuda.synchronize()
    expected = b"".join(t.contiguous().view(torch.uint8).cpu().numpy().tobytes()
                        for t in (dnormed, dy, dact, dq, dattn, tokens))
    assert raw.tobytes() == expected
