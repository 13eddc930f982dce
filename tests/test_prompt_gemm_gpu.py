"""GPU parity of the prompt (prefill) GEMM - the tcgen05 kernel the linear operators take above 32 rows - called
through the C ABI, against the CPU oracle's staged arithmetic and against the small-M streaming kernels of the same
library (the <= 16-row path, itself pinned against the reference's CUDA kernels in tests/test_reference_ops_gpu.py).

Tolerance: the reference's BF16 linear bound |a - r| <= 0.015625 + 0.01 |r|
(operators/tests/operators_cuda_awq_test.cu:175-177). FP32 accumulation order is the only freedom between the two
kernels, so nearly all outputs must also agree to the last BF16 bit."""
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


def tolerance(ref):
    return 0.015625 + 0.01 * np.abs(ref)


def narrow_rows(torch, call, x, n):
    """The same operator fed 16 rows at a time: the streaming kernels."""
    out = torch.empty((x.shape[0], n), dtype=torch.bfloat16, device="cuda")
    for first in range(0, x.shape[0], 16):
        call(x[first:first + 16], out[first:first + 16])
    return out


# (N, K): one feature tile / several; a feature tail (272 = 256 + 16); K of 2 and 56 groups; a qkv projection of
# the 28-head model (18 tiles, 28 groups, with bias).
AWQ_SHAPES = [(256, 256), (1536, 1024), (272, 512), (4608, 3584)]


@pytest.mark.parametrize("rows", [33, 128, 129, 300, 600])
@pytest.mark.parametrize("nk", AWQ_SHAPES)
def test_awq_prompt_gemm(cuda, package, oracle, ctx, rows, nk):
    torch, ops, syn = cuda, package.operators, package.synthetic
    n, k = nk
    q, s, z = syn.awq_triple(17, f"prompt{n}x{k}", n, k)
    bias = syn.float_to_bf16(np.random.default_rng(n).standard_normal(n, dtype=np.float32) * 0.1) if n == 4608 else None
    x = syn.float_to_bf16(np.random.default_rng(rows + k).standard_normal((rows, k), dtype=np.float32))
    dq, ds, dz, dx = torch.from_numpy(q).cuda(), to_dev(torch, s), torch.from_numpy(z).cuda(), to_dev(torch, x)
    db = to_dev(torch, bias) if bias is not None else None
    weight = ops.prepare_awq(dq, ds, dz, 128, k, db)
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    guard = torch.full((rows + 1, n), 7.0, dtype=torch.bfloat16, device="cuda")   # the row after the last stays
    ops.awq_linear(ctx, dx, weight, out, None)
    ops.awq_linear(ctx, dx, weight, guard[:rows], None)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), guard[:rows].view(torch.int16))     # same bits on every call
    assert (guard[rows] == 7.0).all()
    scratch = torch.empty(ops.linear_scratch_bytes(16, k, n), dtype=torch.uint8, device="cuda")
    narrow = narrow_rows(torch, lambda a, b: ops.awq_linear(ctx, a, weight, b, scratch), dx, n)
    torch.cuda.synchronize()
    got, other = syn.bf16_to_float(to_host(out)), syn.bf16_to_float(to_host(narrow))
    assert np.all(np.abs(got - other) <= tolerance(other))
    assert np.mean(got == other) > 0.97
    # With caller scratch the kernel may split K over blocks (FP32 slices added by a second kernel).
    wide_scratch = torch.empty(ops.linear_scratch_bytes(rows, k, n), dtype=torch.uint8, device="cuda")
    split = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.awq_linear(ctx, dx, weight, split, wide_scratch)
    torch.cuda.synchronize()
    with_split = syn.bf16_to_float(to_host(split))
    assert np.all(np.abs(with_split - other) <= tolerance(other))
    assert np.mean(with_split == other) > 0.97
    cols = np.random.default_rng(n + k).choice(n, size=min(n, 128), replace=False)
    pick = np.random.default_rng(rows).choice(rows, size=min(rows, 64), replace=False)
    dense = syn.awq_dequantize(q[cols], s[cols], z[cols], k)
    ref = oracle.op_linear(syn.bf16_to_float(x[pick]), dense, syn.bf16_to_float(bias[cols]) if bias is not None else None)
    assert np.all(np.abs(got[np.ix_(pick, cols)] - ref) <= tolerance(ref))
    assert np.mean(got[np.ix_(pick, cols)] == ref) > 0.97


@pytest.mark.parametrize("rows", [33, 128, 257, 600])
@pytest.mark.parametrize("nk", [(512, 512), (272, 192), (4096, 2048)])
def test_dense_prompt_gemm(cuda, package, oracle, ctx, rows, nk):
    torch, ops, syn = cuda, package.operators, package.synthetic
    n, k = nk
    rng = np.random.default_rng(n * 7 + k)
    w = syn.float_to_bf16(rng.standard_normal((n, k), dtype=np.float32) * 0.05)
    bias = syn.float_to_bf16(rng.standard_normal(n, dtype=np.float32) * 0.1) if n == 512 else None
    x = syn.float_to_bf16(rng.standard_normal((rows, k), dtype=np.float32))
    dw, dx = to_dev(torch, w), to_dev(torch, x)
    db = to_dev(torch, bias) if bias is not None else None
    weight = ops.prepare_dense(dw.t(), db)                       # logical [in, out] view of the [out, in] matrix
    out = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.linear(ctx, dx, weight, out, None)
    scratch = torch.empty(ops.linear_scratch_bytes(16, k, n), dtype=torch.uint8, device="cuda")
    narrow = narrow_rows(torch, lambda a, b: ops.linear(ctx, a, weight, b, scratch), dx, n)
    torch.cuda.synchronize()
    got, other = syn.bf16_to_float(to_host(out)), syn.bf16_to_float(to_host(narrow))
    assert np.all(np.abs(got - other) <= tolerance(other))
    assert np.mean(got == other) > 0.97
    cols = rng.choice(n, size=min(n, 128), replace=False)
    pick = rng.choice(rows, size=min(rows, 64), replace=False)
    ref = oracle.op_linear(syn.bf16_to_float(x[pick]), syn.bf16_to_float(w[cols]),
                           syn.bf16_to_float(bias[cols]) if bias is not None else None)
    assert np.all(np.abs(got[np.ix_(pick, cols)] - ref) <= tolerance(ref))
    assert np.mean(got[np.ix_(pick, cols)] == ref) > 0.97
