"""Single operators of this library against the SAME operators of the unmodified reference (op::cuda::*, compiled
into oracle/_ref by oracle/Makefile), on identical device inputs on the same GPU.

Bounds, fixed:
  rms_norm, add, silu_multiply, rope_precomputed, store_kv   bit-equal BF16 - what the reference's own contract
      test pins for its kernels (operators/tests/operators_cuda_bf16_contract_test.cu:66-139, 235-416). The norm
      kernels here take the sum of squares in the reference kernel's order, so the inverse RMS has the same bits.
  awq_linear (M > 1), linear                                   |a - r| <= 0.015625 + 0.01 max(|a|, |r|), the
      reference's BF16 tolerance (operators/tests/operators_cuda_awq_test.cu:175-177); the two differ only in
      the order of the FP32 accumulation.
  attention_prefill                                            the same element bound, and a relative RMS distance
      of at most 4e-3 (about one BF16 unit in the last place of the output): both kernels round the softmax
      numerators to BF16 and accumulate in FP32, in different tile orders.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(cuda, oracle):
    if not oracle.reference_available():
        pytest.skip("oracle/_ref is not built")
    try:
        return oracle.ReferenceOps()
    except RuntimeError as error:
        pytest.skip(str(error))


@pytest.fixture(scope="module")
def ctx(cuda, package):
    return package.operators.prepare_execution_context(0)


def bf16_normal(torch, shape, seed, scale=1.0):
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=gen) * scale).to(torch.bfloat16)


def bits(t):
    import torch
    return t.contiguous().view(torch.int16)


def reference_bound(a, r):
    return 0.015625 + 0.01 * np.maximum(np.abs(a), np.abs(r))


@pytest.mark.parametrize("width", [128, 896, 1024, 2048, 3584, 4096, 10240])
def test_rms_norm_equals_reference_kernel(cuda, package, ref, ctx, width):
    torch, ops = cuda, package.operators
    rows = 9
    x = bf16_normal(torch, (rows, width), width, 3.0)
    w = bf16_normal(torch, (width,), width + 1, 0.3) + 1.0
    mine, theirs = torch.empty_like(x), torch.empty_like(x)
    ops.rms_norm(ctx, x, w, mine, rows, width, 1e-6)
    ref.rms_norm(x, w, theirs, rows, width, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))


def test_qk_norm_rows_equal_reference_kernel(cuda, package, ref, ctx):
    """The per-head norm the reference runs over [rows * heads, 128] (decoder.hpp:125-128)."""
    torch, ops = cuda, package.operators
    rows, width = 9 * 40, 128
    x = bf16_normal(torch, (rows, width), 5, 2.0)
    w = bf16_normal(torch, (width,), 6, 0.3) + 1.0
    mine, theirs = torch.empty_like(x), torch.empty_like(x)
    ops.rms_norm(ctx, x, w, mine, rows, width, 1e-6)
    ref.rms_norm(x, w, theirs, rows, width, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))


@pytest.mark.parametrize("count", [18, 4099, 9 * 12288])
def test_add_and_silu_multiply_equal_reference_kernels(cuda, package, ref, ctx, count):
    torch, ops = cuda, package.operators
    a = bf16_normal(torch, (count,), count, 4.0)
    b = bf16_normal(torch, (count,), count + 1, 4.0)
    a[:6] = torch.tensor([-100.0, -90.0, -81.0, 1e-38, 30.0, 0.0], device="cuda").to(torch.bfloat16)  # the tails
    mine, theirs = torch.empty_like(a), torch.empty_like(a)
    ops.add(ctx, a, b, mine)
    ref.add(a, b, theirs, count)
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))
    ops.silu_multiply(ctx, a, b, mine)
    ref.silu_multiply(a, b, theirs, count)
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))


def test_rope_and_store_kv_equal_reference_kernels(cuda, package, ref, ctx):
    torch, ops = cuda, package.operators
    rows, heads, d, offset, positions, theta = 9, 40, 128, 2039, 2304, 1e6
    table = torch.from_numpy(ops.build_rope_table(positions, d, theta)).cuda()
    x = bf16_normal(torch, (rows, heads, d), 11)
    mine, theirs = x.clone(), x.clone()
    ops.rope_precomputed(ctx, mine, table, offset)
    ref.rope_precomputed(theirs, rows, heads, d, table, positions, offset)
    torch.cuda.synchronize()
    assert torch.equal(bits(mine), bits(theirs))
    width, capacity = 1024, 64
    source = bf16_normal(torch, (rows, width), 12)
    cache_a = torch.full((capacity, width), 7.0, dtype=torch.bfloat16, device="cuda")
    cache_b = cache_a.clone()
    ops.store_kv(ctx, source, cache_a, 31)
    ref.store_kv(source, cache_b, rows, width, capacity, 31)
    torch.cuda.synchronize()
    assert torch.equal(bits(cache_a), bits(cache_b))


@pytest.mark.parametrize("rows", [2, 5, 9, 16, 300])       # 300: the tcgen05 prompt kernel against the reference's GEMM
@pytest.mark.parametrize("nk_bias", [((4096, 4096), False), ((1024, 4096), False), ((4096, 12288), False),
                                     ((512, 3584), True), ((3584, 18944), False)])
def test_awq_linear_against_reference_kernel(cuda, package, ref, ctx, rows, nk_bias):
    torch, ops, syn = cuda, package.operators, package.synthetic
    (n, k), with_bias = nk_bias
    q, s, z = syn.awq_triple(31, f"ref{n}x{k}", n, k)
    dq, dz = torch.from_numpy(q).cuda(), torch.from_numpy(z).cuda()
    ds = torch.from_numpy(s.view(np.int16)).cuda().view(torch.bfloat16)
    bias = bf16_normal(torch, (n,), n) if with_bias else None
    x = bf16_normal(torch, (rows, k), rows + n)
    weight = ops.prepare_awq(dq, ds, dz, 128, k, bias)
    mine = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    theirs = torch.empty_like(mine)
    scratch = torch.empty(max(16, ops.linear_scratch_bytes(rows, k, n)), dtype=torch.uint8, device="cuda")
    ops.awq_linear(ctx, x, weight, mine, scratch)
    ref.awq_linear(x, rows, k, n, dq, ds, s.shape[1], dz, 128, bias, theirs)
    torch.cuda.synchronize()
    a, r = mine.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.all(np.abs(a - r) <= reference_bound(a, r))
    # Same dequantised weights, same FP32 accumulation: most outputs agree to the last BF16 bit.
    assert np.mean(a == r) > 0.9


@pytest.mark.parametrize("rows", [1, 9, 16, 300])
@pytest.mark.parametrize("nk", [(8192, 4096), (2048, 2048), (1024, 6144)])
def test_dense_linear_against_reference_cublas(cuda, package, ref, ctx, rows, nk):
    torch, ops = cuda, package.operators
    n, k = nk
    w = bf16_normal(torch, (n, k), n + k, 0.02)
    bias = bf16_normal(torch, (n,), n)
    x = bf16_normal(torch, (rows, k), rows)
    weight = ops.prepare_dense(w.t(), bias)
    mine = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    theirs = torch.empty_like(mine)
    scratch = torch.empty(max(16, ops.linear_scratch_bytes(rows, k, n)), dtype=torch.uint8, device="cuda")
    ops.linear(ctx, x, weight, mine, scratch)
    ref.linear(x, rows, k, n, w, bias, theirs)
    torch.cuda.synchronize()
    a, r = mine.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.all(np.abs(a - r) <= reference_bound(a, r))


@pytest.mark.parametrize("rows", [1, 5, 9])
@pytest.mark.parametrize("length", [512, 2048, 4099])
@pytest.mark.parametrize("heads_kv", [(32, 8), (28, 4)])
def test_attention_against_reference_kernel(cuda, package, ref, ctx, rows, length, heads_kv):
    torch, ops = cuda, package.operators
    heads, kv_heads = heads_kv
    d = 128
    q = bf16_normal(torch, (rows, heads, d), rows + length)
    k = bf16_normal(torch, (length, kv_heads, d), length)
    v = bf16_normal(torch, (length, kv_heads, d), length + 1)
    mine, theirs = torch.empty_like(q), torch.empty_like(q)
    scratch = torch.empty(ops.attention_scratch_bytes(rows, heads, d, length), dtype=torch.uint8, device="cuda")
    ops.attention_prefill(ctx, q, k, v, mine, length - rows, scratch)
    ref.attention_prefill(q, k, v, theirs, rows, heads, kv_heads, d, length, length - rows)
    torch.cuda.synchronize()
    a, r = mine.float().cpu().numpy(), theirs.float().cpu().numpy()
    assert np.all(np.abs(a - r) <= reference_bound(a, r))
    assert float(np.sqrt(((a - r) ** 2).mean())) <= 4e-3 * float(np.sqrt((r ** 2).mean()))
