"""GPU parity of the direct operators, called through the C ABI, against the CPU oracle's staged arithmetic
and against the reference tests' own known answers. Tolerances are the reference's:
BF16 linear  |a - r| <= 0.015625 + 0.01 |r|      (operators/tests/operators_cuda_awq_test.cu:175-177)
attention    |a - e| <= 2.5e-4 + 0.008 max(|a|,|e|) against the reference CPU executor's FP32 attention; twice the
             bound the reference gives its FP32-numerator decode kernels
             (operators/tests/operators_cuda_attention_precision_test.cu:108), because the verify kernel, like the
             reference's prefill kernel, rounds the softmax numerators to BF16
rope / add / gather / store_kv / greedy / accept: bit-exact BF16 against the oracle's host formulas.
norm / silu*up: compared here with HOST formulas, whose 1/sqrt and exp differ from the device's rsqrt / ex2 in the
             last FP32 bit, so a BF16 rounding flips in well under 1 % of the outputs (rate asserted below); bit
             equality of these two is pinned against the reference's own CUDA kernels on the same GPU in
             tests/test_reference_ops_gpu.py (operators/tests/operators_cuda_bf16_contract_test.cu:66-139, 235-268)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def to_dev(torch, bits: np.ndarray):
    return torch.from_numpy(bits.view(np.int16)).cuda().view(torch.bfloat16)


def to_host(t) -> np.ndarray:
    import torch
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.fixture(scope="module")
def ctx(cuda, package):
    return package.operators.prepare_execution_context(0)


def linear_tolerance(ref):
    return 0.015625 + 0.01 * np.abs(ref)


@pytest.mark.parametrize("rows", [1, 2, 4, 8, 9, 16])
@pytest.mark.parametrize("nk", [(4096, 4096), (1024, 4096), (24576, 4096), (4096, 12288)])
def test_awq_linear_sweep(cuda, package, oracle, ctx, rows, nk):
    """Operator sweep of the benchmark configuration: packed uint4 uniform, zeros uniform, group 128, BF16
    scales uniform [0.002, 0.02], BF16 activations N(0, 1)."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    n, k = nk
    q, s, z = syn.awq_triple(13, f"sweep{n}x{k}", n, k)
    x = syn.float_to_bf16(np.random.default_rng(rows).standard_normal((rows, k), dtype=np.float32))
    dq, ds, dz, dx = torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda(), to_dev(torch, x)
    weight = ops.prepare_awq(dq, ds, dz, 128, k)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(ops.linear_scratch_bytes(rows, k, n), dtype=torch.uint8, device="cuda")
    ops.awq_linear(ctx, dx, weight, out, scratch)
    again = torch.empty_like(out)
    ops.awq_linear(ctx, dx, weight, again, scratch)               # same bits on every call
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    # Oracle on a column subset (the CPU follows 256 columns in well under a second).
    cols = np.random.default_rng(n + k).choice(n, size=256, replace=False)
    dense = syn.awq_dequantize(q[cols], s[cols], z[cols], k)
    ref = oracle.op_linear(syn.bf16_to_float(x), dense, None)
    got = syn.bf16_to_float(to_host(out))[:, cols]
    assert np.all(np.abs(got - ref) <= linear_tolerance(ref))
    # FP32 accumulation order is the only freedom: almost every output must agree to the last BF16 bit.
    assert np.mean(got == ref) > 0.97


@pytest.mark.parametrize("shape", [(24, 16, 4), (24, 16, 8), (24, 16, 12), (256, 16, 128), (32, 17, 4), (1024, 17, 128)])
@pytest.mark.parametrize("rows", [1, 3])
def test_awq_linear_reference_fixture_shapes(cuda, package, oracle, ctx, shape, rows):
    """The shapes of the reference's own AWQ test ({K, N, group}; padded scale columns poisoned with -73),
    including odd widths that take the any-shape kernel."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    k, n, group = shape
    groups = k // group
    q, s, z = syn.awq_triple(5, f"fix{k}x{n}x{group}", n, k, group, padded_groups=groups + 3)
    bias = syn.float_to_bf16(np.linspace(-0.1, 0.1, n, dtype=np.float32))
    x = syn.float_to_bf16(np.random.default_rng(3).standard_normal((rows, k), dtype=np.float32) * 0.25)
    dq, ds, dz, db = torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda(), to_dev(torch, bias)
    weight = ops.prepare_awq(dq, ds, dz, group, k, db)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    ops.awq_linear(ctx, to_dev(torch, x), weight, out, None)
    torch.cuda.synchronize()
    dense = syn.awq_dequantize(q, s, z, k, group)
    ref = oracle.op_linear(syn.bf16_to_float(x), dense, syn.bf16_to_float(bias))
    got = syn.bf16_to_float(to_host(out))
    assert np.all(np.abs(got - ref) <= linear_tolerance(ref))


@pytest.mark.parametrize("rows", [1, 3])
@pytest.mark.parametrize("kn", [(256, 16), (512, 24)])
def test_awq_bias_cancellation_known_answer(cuda, package, ctx, rows, kn):
    """Known answer of the reference test (operators_cuda_awq_test.cu:242-300): dot = +-(1 + 1/256), bias = -+1.
    The exact result +-1/256 survives only if the bias joins the FP32 sum before the single rounding."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    k, n = kn
    groups = k // 128
    x = np.zeros((rows, k), dtype=np.float32)
    x[:, 0], x[:, 1] = 1.0, 1.0 / 256.0
    q = np.full((n, k // 8), 0x88888888, dtype=np.uint32)
    z = np.full((n, (groups + 7) // 8), 0x88888888, dtype=np.uint32)
    signs = np.where(np.arange(n) % 2 == 0, 1.0, -1.0).astype(np.float32)
    quantized = np.where(signs > 0, 9, 7).astype(np.uint32)
    q[:, 0] = (0x88888888 & ~0xFF) | quantized | (quantized << 4)
    scales = syn.float_to_bf16(np.ones((n, groups), dtype=np.float32))
    bias = syn.float_to_bf16(-signs)
    # The prepared weight borrows these buffers: keep them alive for as long as it is used.
    dq, ds, dz, db = (torch.from_numpy(q.view(np.int32)).cuda(), to_dev(torch, scales),
                      torch.from_numpy(z.view(np.int32)).cuda(), to_dev(torch, bias))
    weight = ops.prepare_awq(dq, ds, dz, 128, k, db)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    ops.awq_linear(ctx, to_dev(torch, syn.float_to_bf16(x)), weight, out, None)
    torch.cuda.synchronize()
    got = syn.bf16_to_float(to_host(out))
    assert np.array_equal(got, np.tile(signs / 256.0, (rows, 1)))
    weight.bias = None
    ops.awq_linear(ctx, to_dev(torch, syn.float_to_bf16(x)), weight, out, None)
    torch.cuda.synchronize()
    assert np.array_equal(syn.bf16_to_float(to_host(out)), np.tile(signs, (rows, 1)))


@pytest.mark.parametrize("rows", [5, 16])
@pytest.mark.parametrize("nk", [(4608, 3584), (3584, 18944), (512, 3584), (3584, 2048)])
def test_awq_linear_qwen25_7b_shapes(cuda, package, oracle, ctx, rows, nk):
    """Projections of the 28-head / 4-KV-head model with bias: 28 or 148 scale groups per row (row pitches TMA
    cannot address), 14 and 74 units of 256 inputs (a short last slice), N not a multiple of the block count."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    n, k = nk
    q, s, z = syn.awq_triple(29, f"c5_{n}x{k}", n, k)
    bias = syn.float_to_bf16(np.random.default_rng(n).standard_normal(n, dtype=np.float32) * 0.1)
    x = syn.float_to_bf16(np.random.default_rng(rows + k).standard_normal((rows, k), dtype=np.float32))
    dq, ds, dz, db, dx = (torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda(), to_dev(torch, bias),
                          to_dev(torch, x))
    weight = ops.prepare_awq(dq, ds, dz, 128, k, db)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(ops.linear_scratch_bytes(rows, k, n), dtype=torch.uint8, device="cuda")
    ops.awq_linear(ctx, dx, weight, out, scratch)
    torch.cuda.synchronize()
    cols = np.random.default_rng(n + k).choice(n, size=256, replace=False)
    dense = syn.awq_dequantize(q[cols], s[cols], z[cols], k)
    ref = oracle.op_linear(syn.bf16_to_float(x), dense, syn.bf16_to_float(bias[cols]))
    got = syn.bf16_to_float(to_host(out))[:, cols]
    assert np.all(np.abs(got - ref) <= linear_tolerance(ref))
    assert np.mean(got == ref) > 0.97


@pytest.mark.parametrize("rows", [1, 9, 16])
@pytest.mark.parametrize("fk", [(12288, 4096), (18944, 3584), (128, 512), (64, 4096)])
def test_awq_gate_up_silu_matches_unfused_sequence(cuda, package, oracle, ctx, rows, fk):
    """The fused SwiGLU projection against the reference's sequence (two projections, then silu_multiply:
    runtime/include/execution/decoder.hpp:162-165): every rounding point is kept, so the bits agree with this
    library's unfused operators up to the FP32 summation order, and with the oracle within the linear bound."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    f, k = fk
    q, s, z = syn.awq_triple(17, f"gateup{f}x{k}", 2 * f, k)
    bias = syn.float_to_bf16(np.random.default_rng(3).standard_normal(2 * f, dtype=np.float32) * 0.05)
    x = syn.float_to_bf16(np.random.default_rng(rows).standard_normal((rows, k), dtype=np.float32))
    dq, ds, dz, db, dx = (torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda(), to_dev(torch, bias),
                          to_dev(torch, x))
    weight = ops.prepare_awq(dq, ds, dz, 128, k, db)
    scratch = torch.empty(ops.linear_scratch_bytes(rows, k, 2 * f), dtype=torch.uint8, device="cuda")
    fused = torch.empty((rows, f), dtype=torch.bfloat16, device="cuda")
    ops.awq_gate_up_silu(ctx, dx, weight, fused)
    both = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device="cuda")
    ops.awq_linear(ctx, dx, weight, both, scratch)
    unfused = torch.empty_like(fused)
    gate, up = both[:, :f].contiguous(), both[:, f:].contiguous()
    ops.silu_multiply(ctx, gate.view(-1), up.view(-1), unfused.view(-1))
    torch.cuda.synchronize()
    a, b = syn.bf16_to_float(to_host(fused)), syn.bf16_to_float(to_host(unfused))
    assert np.array_equal(a, b)                                   # same kernel, same summation order
    cols = np.random.default_rng(f).choice(f, size=min(f, 128), replace=False)
    pick = np.concatenate([cols, cols + f])
    dense = syn.awq_dequantize(q[pick], s[pick], z[pick], k)
    ref = oracle.op_linear(syn.bf16_to_float(x), dense, syn.bf16_to_float(bias[pick]))
    n = len(cols)
    want = oracle.op_silu_multiply(ref[:, :n].reshape(-1), ref[:, n:].reshape(-1)).reshape(rows, n)
    # A gate or up value that differs from the oracle's by one BF16 rounding moves the product by up to 2^-7
    # of itself (times the slope of silu, < 1.1): allow that on top of the linear bound of each factor.
    bound = 0.015625 + 0.03 * np.abs(want) + 0.02 * np.abs(ref[:, n:])
    assert np.all(np.abs(a[:, cols] - want) <= bound)


@pytest.mark.parametrize("rows", [1, 5, 16, 21])
# K = 6144 and 12288 take two and three K slices (FP32 partials + the fixed-order merge), K = 768 leaves most
# warps of the TMA-fed kernel without inputs, K = 320 takes the register-prefetching kernel.
@pytest.mark.parametrize("nk", [(4096, 2048), (151936, 1024), (1000, 320), (6144, 4096), (2048, 6144), (1024, 12288),
                                (512, 768)])
def test_dense_linear(cuda, package, oracle, ctx, rows, nk):
    torch, ops, syn = cuda, package.operators, package.synthetic
    n, k = nk
    w = syn.dense_matrix(2, f"dense{n}x{k}", n, k)
    bias = syn.float_to_bf16(np.random.default_rng(1).standard_normal(n, dtype=np.float32) * 0.05)
    x = syn.float_to_bf16(np.random.default_rng(rows).standard_normal((rows, k), dtype=np.float32))
    dw, db = to_dev(torch, w), to_dev(torch, bias)
    weight = ops.prepare_dense(dw.t(), db)                       # logical [in, out] view of the [out, in] matrix
    assert weight.operation == 1
    out = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
    scratch = torch.empty(ops.linear_scratch_bytes(rows, k, n), dtype=torch.uint8, device="cuda")
    ops.linear(ctx, to_dev(torch, x), weight, out, scratch)
    torch.cuda.synchronize()
    cols = np.random.default_rng(n).choice(n, size=min(n, 256), replace=False)
    ref = oracle.op_linear(syn.bf16_to_float(x), syn.bf16_to_float(w[cols]), syn.bf16_to_float(bias[cols]))
    got = syn.bf16_to_float(to_host(out))[:, cols]
    assert np.all(np.abs(got - ref) <= linear_tolerance(ref))
    # Row-major [in, out] storage takes the any-shape kernel and must agree too.
    if n <= 6144:
        dw_rm = dw.t().contiguous()
        weight_rm = ops.prepare_dense(dw_rm, db)
        assert weight_rm.operation == 0
        out2 = torch.empty_like(out)
        ops.linear(ctx, to_dev(torch, x), weight_rm, out2, None)
        torch.cuda.synchronize()
        got2 = syn.bf16_to_float(to_host(out2))[:, cols]
        assert np.all(np.abs(got2 - ref) <= linear_tolerance(ref))


def test_dense_bias_before_rounding_known_answer(cuda, package, ctx):
    """operators_cuda_bf16_contract_test.cu:286-326: dot = 1 + 1/256 is a BF16 tie; adding the bias -1 after a
    rounding would lose the 1/256."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    features, outputs, rows = 64, 8, 2
    x = np.zeros((rows, features), dtype=np.float32)
    x[0, 0], x[0, 1], x[1, 0], x[1, 1] = 1.0, 1 / 256, -1.0, -1 / 256
    w = np.zeros((outputs, features), dtype=np.float32)
    w[0::2, 0] = w[0::2, 1] = 1.0
    w[1::2, 0] = w[1::2, 1] = -1.0
    bias = np.where(np.arange(outputs) % 2 == 0, -1.0, 1.0).astype(np.float32)
    dw, db = to_dev(torch, syn.float_to_bf16(w)), to_dev(torch, syn.float_to_bf16(bias))
    weight = ops.prepare_dense(dw.t(), db)
    out = torch.empty((rows, outputs), dtype=torch.bfloat16, device="cuda")
    ops.linear(ctx, to_dev(torch, syn.float_to_bf16(x)), weight, out, None)
    torch.cuda.synchronize()
    got = syn.bf16_to_float(to_host(out))
    assert np.array_equal(got[0], np.where(np.arange(outputs) % 2 == 0, 1 / 256, -1 / 256))
    assert np.array_equal(got[1], np.where(np.arange(outputs) % 2 == 0, -2.0, 2.0))


@pytest.mark.parametrize("width", [7, 128, 1024, 4096, 10240])
def test_rms_norm_against_host_formula(cuda, package, oracle, ctx, width):
    torch, ops, syn = cuda, package.operators, package.synthetic
    rows = 5
    rng = np.random.default_rng(width)
    x = syn.float_to_bf16(rng.standard_normal((rows, width), dtype=np.float32) * 3)
    w = syn.float_to_bf16(0.63 + (np.arange(width) % 5) * 0.17)
    dx, dw = to_dev(torch, x), to_dev(torch, w)
    out = torch.empty_like(dx)
    ops.rms_norm(ctx, dx, dw, out, rows, width, 1e-6)
    torch.cuda.synchronize()
    ref = oracle.op_rms_norm(syn.bf16_to_float(x), syn.bf16_to_float(w), 1e-6)
    got = syn.bf16_to_float(to_host(out))
    # The inverse RMS may differ in its last FP32 bit (reduction order, rsqrt); a BF16 rounding flips rarely.
    assert np.mean(got == ref) > 0.995
    assert np.all(np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-30)
    ops.rms_norm(ctx, dx, dw, dx, rows, width, 1e-6)              # in place
    torch.cuda.synchronize()
    assert np.array_equal(to_host(dx), to_host(out))
    with pytest.raises(RuntimeError):
        ops.rms_norm(ctx, torch.empty(10241, dtype=torch.bfloat16, device="cuda"),
                     torch.empty(10241, dtype=torch.bfloat16, device="cuda"),
                     torch.empty(10241, dtype=torch.bfloat16, device="cuda"), 1, 10241, 1e-6)


def test_rms_norm_reference_fixture_against_host_formula(cuda, package, ctx):
    """The reference's own fixture (operators_cuda_bf16_contract_test.cu:235-268) with its scalar expectation."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    width = 128
    i = np.arange(width)
    x = syn.bf16_to_float(syn.float_to_bf16((-0.8 + (i % 7) * 0.25).astype(np.float32)))
    w = syn.bf16_to_float(syn.float_to_bf16((0.63 + (i % 5) * 0.17).astype(np.float32)))
    total = np.float32(0)
    for v in x:
        total = np.float32(total + v * v)
    inv = np.float32(1.0) / np.sqrt(np.float32(total / np.float32(width) + np.float32(1e-6)))
    rounded = syn.bf16_to_float(syn.float_to_bf16(x * inv))
    expected = syn.float_to_bf16(rounded * w)
    out = torch.empty(width, dtype=torch.bfloat16, device="cuda")
    ops.rms_norm(ctx, to_dev(torch, syn.float_to_bf16(x)), to_dev(torch, syn.float_to_bf16(w)), out, 1, width, 1e-6)
    torch.cuda.synchronize()
    assert np.mean(to_host(out) == expected) > 0.98


def test_rope_precomputed_bit_exact(cuda, package, oracle, ctx):
    torch, ops, syn = cuda, package.operators, package.synthetic
    rows, heads, d, offset, max_pos, theta = 5, 3, 128, 37, 64, 1e6
    x = syn.float_to_bf16(np.random.default_rng(0).standard_normal((rows, heads, d), dtype=np.float32))
    table = torch.from_numpy(ops.build_rope_table(max_pos, d, theta)).cuda()
    dx = to_dev(torch, x)
    ops.rope_precomputed(ctx, dx, table, offset)
    torch.cuda.synchronize()
    ref = oracle.op_rope(syn.bf16_to_float(x), offset, theta, max_pos)
    assert np.array_equal(syn.bf16_to_float(to_host(dx)), ref)
    # device-side offsets (graph mode of the reference)
    dx2 = to_dev(torch, x)
    offsets = torch.tensor([offset], dtype=torch.int64, device="cuda")
    ops.rope_precomputed(ctx, dx2, table, 0, offsets)
    torch.cuda.synchronize()
    assert np.array_equal(to_host(dx2), to_host(dx))
    with pytest.raises(IndexError):
        ops.rope_precomputed(ctx, dx2, table, max_pos - 2)


def test_rope_small_angle_basis(cuda, package, ctx):
    """operators_cuda_bf16_contract_test.cu:372-416: a unit basis rotated at positions 0..20 (theta 1e6) must give
    the BF16-rounded FP64 cosine / sine."""
    torch, ops, syn = cuda, package.operators, package.synthetic
    d, positions, theta = 128, 21, 1e6
    table = torch.from_numpy(ops.build_rope_table(positions, d, theta)).cuda()
    basis = np.zeros((1, 1, d), dtype=np.float32)
    basis[..., : d // 2] = 1.0
    for p in range(positions):
        dx = to_dev(torch, syn.float_to_bf16(basis))
        ops.rope_precomputed(ctx, dx, table, p)
        torch.cuda.synchronize()
        got = syn.bf16_to_float(to_host(dx))[0, 0]
        i = np.arange(d // 2)
        angle = p / np.power(float(theta), 2.0 * i / d)
        assert np.array_equal(got[: d // 2], syn.bf16_to_float(syn.float_to_bf16(np.cos(angle).astype(np.float32))))
        assert np.array_equal(got[d // 2:], syn.bf16_to_float(syn.float_to_bf16(np.sin(angle).astype(np.float32))))


@pytest.mark.parametrize("count", [17, 18, 4098, 4099])
def test_add_exact_and_silu_multiply_against_host_formula(cuda, package, oracle, ctx, count):
    torch, ops, syn = cuda, package.operators, package.synthetic
    rng = np.random.default_rng(count)
    a = syn.float_to_bf16(rng.standard_normal(count, dtype=np.float32) * 4)
    b = syn.float_to_bf16(rng.standard_normal(count, dtype=np.float32) * 4)
    a[:4] = syn.float_to_bf16(np.array([-100.0, -90.0, 1e-38, 30.0], dtype=np.float32))   # tails
    da, db = to_dev(torch, a), to_dev(torch, b)
    out = torch.empty_like(da)
    ops.add(ctx, da, db, out)
    torch.cuda.synchronize()
    assert np.array_equal(syn.bf16_to_float(to_host(out)), oracle.op_add(syn.bf16_to_float(a), syn.bf16_to_float(b)))
    ops.silu_multiply(ctx, da, db, out)
    torch.cuda.synchronize()
    ref = oracle.op_silu_multiply(syn.bf16_to_float(a), syn.bf16_to_float(b))
    got = syn.bf16_to_float(to_host(out))
    # expf differs from the host exp in the last FP32 bits; BF16 results agree except for rare rounding ties.
    assert np.mean(got == ref) > 0.995 and np.all(np.abs(got - ref) <= 2.0 ** -7 * np.abs(ref) + 1e-37)
    ops.silu_multiply(ctx, da, db, da)                            # output = gate aliasing
    torch.cuda.synchronize()
    assert np.array_equal(to_host(da), to_host(out))
    with pytest.raises(RuntimeError):
        ops.add(ctx, da, db, torch.empty(count + 1, dtype=torch.bfloat16, device="cuda"))


def test_gather_and_store_kv(cuda, package, ctx):
    torch, ops, syn = cuda, package.operators, package.synthetic
    table = syn.dense_matrix(0, "table", 50, 64)
    ids = np.array([3, 49, 50, 0, 4000000000], dtype=np.uint32)    # two out-of-vocabulary ids -> zeros
    out = torch.empty((5, 64), dtype=torch.bfloat16, device="cuda")
    ops.gather(ctx, torch.from_numpy(ids.view(np.int32)).cuda(), to_dev(torch, table), out)
    torch.cuda.synchronize()
    got = to_host(out)
    assert np.array_equal(got[0], table[3]) and np.array_equal(got[1], table[49]) and np.array_equal(got[3], table[0])
    assert not got[2].any() and not got[4].any()
    cache = torch.full((16, 64), 0.375, dtype=torch.bfloat16, device="cuda")
    ops.store_kv(ctx, out[:3].contiguous(), cache, 5)
    torch.cuda.synchronize()
    host = to_host(cache)
    assert np.array_equal(host[5:8], got[:3])
    poison = syn.float_to_bf16(np.float32(0.375))
    assert (host[:5] == poison).all() and (host[8:] == poison).all()      # guard band untouched
    with pytest.raises(ValueError):
        ops.store_kv(ctx, out, cache, 12)                          # 12 + 5 > 16: rejected before any write
    torch.cuda.synchronize()
    assert np.array_equal(to_host(cache), host)


def attention_case(torch, package, oracle, ctx, rows, heads, kv_heads, length, device_offset, seed=0, capacity=None):
    ops, syn = package.operators, package.synthetic
    d = 128
    rng = np.random.default_rng(seed)
    offset = length - rows
    capacity = capacity or length
    q = syn.float_to_bf16(rng.standard_normal((rows, heads, d), dtype=np.float32))
    # Separate streams, so that the first `length` rows do not depend on the capacity.
    k = syn.float_to_bf16(np.random.default_rng(seed + 1000).standard_normal((capacity, kv_heads, d), dtype=np.float32))
    v = syn.float_to_bf16(np.random.default_rng(seed + 2000).standard_normal((capacity, kv_heads, d), dtype=np.float32))
    dq, dk, dv = to_dev(torch, q), to_dev(torch, k), to_dev(torch, v)
    out = torch.empty_like(dq)
    scratch = torch.empty(ops.attention_scratch_bytes(rows, heads, d, capacity), dtype=torch.uint8, device="cuda")
    if device_offset:
        off = torch.tensor([offset], dtype=torch.int32, device="cuda")
        ops.attention_verify(ctx, dq, dk, dv, out, off, scratch)
    else:
        ops.attention_prefill(ctx, dq, dk[:length], dv[:length], out, offset, scratch)
    torch.cuda.synchronize()
    fq, fk, fv = syn.bf16_to_float(q), syn.bf16_to_float(k[:length]), syn.bf16_to_float(v[:length])
    exact = oracle.op_attention(fq, fk, fv, offset, 0)            # runtime/src/qwen.cpp:382-403 arithmetic
    staged = oracle.op_attention(fq, fk, fv, offset, 1)           # BF16 numerators, exact accumulation
    got = syn.bf16_to_float(to_host(out))
    # Element-wise against the staged value: both round the numerators to BF16, though relative to different
    # running maxima, and both round the output once. An output element is sum_i p_i v_i with independent
    # relative errors of up to 2^-9 on every p_i, so its error scales with sqrt(sum p_i^2) |v|, which is the
    # spread of the whole (row, head) output vector and not the size of the one element (elements that are
    # small through cancellation carry the same error): the last term allows six standard deviations of the
    # difference of two such sums, 6 sqrt(2) 2^-9 / sqrt(3) < 2^-6 of the vector's root mean square.
    spread = np.sqrt((staged ** 2).mean(axis=-1, keepdims=True))
    bound = 2.5e-4 + 0.008 * np.maximum(np.abs(got), np.abs(staged)) + 2.0 ** -6 * spread
    assert np.all(np.abs(got - staged) <= bound), float(np.abs(got - staged).max())
    # In the mean the kernel must be as close to the reference executor's FP32 attention as the staged ideal is.
    rms = lambda a: float(np.sqrt((a ** 2).mean()))               # noqa: E731
    assert rms(got - exact) <= 1.25 * rms(staged - exact) + 1e-6, (rms(got - exact), rms(staged - exact))
    return got


@pytest.mark.parametrize("rows", [1, 5, 9])
@pytest.mark.parametrize("length", [512, 2048, 8192, 32768])
def test_verify_attention_sweep(cuda, package, oracle, ctx, rows, length):
    """Benchmark sweep: 32 Q / 8 KV heads, head_dim 128, BF16 K/V N(0,1)."""
    attention_case(cuda, package, oracle, ctx, rows, 32, 8, length, device_offset=False, seed=length + rows)


@pytest.mark.parametrize("length", [1, 2, 8, 9, 16, 17, 24, 25, 32, 33, 41, 63, 64, 65, 129])
def test_verify_attention_ragged_lengths(cuda, package, oracle, ctx, length):
    """The reference precision test's lengths (4 Q / 2 KV heads) plus tile boundaries, q_len 1."""
    attention_case(cuda, package, oracle, ctx, 1, 4, 2, length, device_offset=False, seed=length)


@pytest.mark.parametrize("rows,heads,kv_heads", [(16, 28, 4), (5, 16, 8), (16, 4, 4), (3, 14, 2)])
def test_verify_attention_group_shapes_and_device_offset(cuda, package, oracle, ctx, rows, heads, kv_heads):
    length = 300
    a = attention_case(cuda, package, oracle, ctx, rows, heads, kv_heads, length, device_offset=False, seed=9)
    b = attention_case(cuda, package, oracle, ctx, rows, heads, kv_heads, length, device_offset=True, seed=9, capacity=1000)
    assert np.array_equal(a, b) or np.abs(a - b).max() < 1e-2     # chunking differs with the capacity


def test_verify_attention_rejects_bad_shapes(cuda, package, ctx):
    torch, ops = cuda, package.operators
    q = torch.zeros((9, 32, 128), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((64, 8, 128), dtype=torch.bfloat16, device="cuda")
    out = torch.full_like(q, 0.5)
    scratch = torch.empty(ops.attention_scratch_bytes(9, 32, 128, 64), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        ops.attention_prefill(ctx, q, kv, kv, out, 60, scratch)              # 60 + 9 > 64
    with pytest.raises(ValueError):
        ops.attention_prefill(ctx, q, kv, kv, out, 0, scratch[:16])          # scratch too small
    with pytest.raises(ValueError):
        ops.attention_prefill(ctx, q, kv[:, :5].contiguous(), kv[:, :5].contiguous(), out, 0, scratch)  # 32 % 5
    torch.cuda.synchronize()
    assert (out == 0.5).all()                                                # rejected before any write


@pytest.mark.parametrize("rows,vocab", [(1, 151936), (9, 151936), (16, 1000), (20, 77)])
def test_greedy_sampling_rules(cuda, package, oracle, ctx, rows, vocab):
    torch, ops, syn = cuda, package.operators, package.synthetic
    rng = np.random.default_rng(vocab)
    logits = rng.standard_normal((rows, vocab), dtype=np.float32) * 3
    logits[0, 5] = np.nan
    if vocab > 100:
        logits[:, 100] = 40.0
        logits[:, 60] = 40.0                                       # tie: lowest index wins
        logits[rows - 1, :] = np.nan                               # all-NaN row -> index 0
    bits = syn.float_to_bf16(logits)
    tokens = torch.zeros(rows, dtype=torch.int32, device="cuda")
    scratch = torch.empty(ops.sample_scratch_bytes(rows, vocab), dtype=torch.uint8, device="cuda")
    ops.sample_greedy(ctx, to_dev(torch, bits), tokens, scratch)
    torch.cuda.synchronize()
    assert np.array_equal(tokens.cpu().numpy().view(np.uint32), oracle.argmax(syn.bf16_to_float(bits)))


def test_verify_accept_kernel(cuda, package, oracle, ctx):
    torch, ops, abi = cuda, package.operators, package.abi
    cases = [([9, 1, 2, 3], [1, 2, 3, 4]), ([9, 1, 2, 3], [1, 7, 3, 4]), ([9, 1, 2, 3], [5, 2, 3, 4]), ([9], [5]),
             (list(range(16)), list(range(1, 17)))]
    for inputs, targets in cases:
        di = torch.tensor(inputs, dtype=torch.int32, device="cuda")
        dt = torch.tensor(targets, dtype=torch.int32, device="cuda")
        context = torch.tensor([100], dtype=torch.int32, device="cuda")
        pending = torch.zeros(1, dtype=torch.int32, device="cuda")
        result = torch.zeros(18, dtype=torch.int32, device="cuda")
        ops.verify_accept(ctx, di, dt, len(inputs), context, pending, result)
        torch.cuda.synchronize()
        emitted = oracle.accept(inputs, targets)
        host = result.cpu().numpy()
        assert host[0] == emitted and host[1] == 100 + emitted and int(context.item()) == 100 + emitted
        assert int(pending.item()) == targets[emitted - 1]
        assert list(host[2:2 + len(targets)]) == targets
