"""The attention entry point that takes no scratch (split partials in an array built into the library) gives
the same bits as the caller-scratch entry point, on two calls in a row, and rejects shapes beyond its array.
Collected last so that it also runs after every other GPU test has used the library."""
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

pytestmark = pytest.mark.gpu


def test_static_scratch_attention_matches_caller_scratch():
    import torch

    package = entry.load_package()
    package.abi.load_library()
    ops, syn = package.operators, package.synthetic
    ctx = ops.prepare_execution_context(0)
    rows, heads, kv_heads, d = 9, 32, 8, 128
    for call, length in enumerate((2048 + rows, 300)):               # two calls in a row, different split counts
        rng = np.random.default_rng(100 + call)
        q = torch.from_numpy(syn.float_to_bf16(rng.standard_normal((rows, heads, d), dtype=np.float32)).view(np.int16))
        k = torch.from_numpy(syn.float_to_bf16(rng.standard_normal((length, kv_heads, d), dtype=np.float32)).view(np.int16))
        v = torch.from_numpy(syn.float_to_bf16(rng.standard_normal((length, kv_heads, d), dtype=np.float32)).view(np.int16))
        dq, dk, dv = (t.cuda().view(torch.bfloat16) for t in (q, k, v))
        expected = torch.empty_like(dq)
        scratch = torch.empty(ops.attention_scratch_bytes(rows, heads, d, length), dtype=torch.uint8, device="cuda")
        ops.attention_prefill(ctx, dq, dk, dv, expected, length - rows, scratch)
        got = torch.full_like(dq, 7.0)
        torch.cuda.synchronize()
        # Free device memory as the DRIVER sees it (cudaMemGetInfo): an allocation made inside the library would
        # not show in torch's own allocator statistics. The first call may load the kernel's module, so the
        # comparison brackets the second call.
        free_before = torch.cuda.mem_get_info()[0] if call else None
        ops.attention_prefill_static(ctx, dq, dk, dv, got, length - rows)
        torch.cuda.synchronize()
        if call:
            assert torch.cuda.mem_get_info()[0] >= free_before
        assert torch.equal(got.view(torch.int16), expected.view(torch.int16)), call


def test_static_scratch_attention_rejects_oversized_shapes():
    import torch

    package = entry.load_package()
    package.abi.load_library()
    ops = package.operators
    ctx = ops.prepare_execution_context(0)
    rows, heads, kv_heads, d, length = 16, 32, 8, 128, 8192            # 64 splits x 512 row-heads x 528 B > 10 MiB
    assert ops.attention_scratch_bytes(rows, heads, d, length) > ops.STATIC_ATTENTION_SCRATCH_BYTES
    q = torch.zeros((rows, heads, d), dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros((length, kv_heads, d), dtype=torch.bfloat16, device="cuda")
    out = torch.full_like(q, 0.5)
    with pytest.raises(ValueError, match="built into the library"):
        ops.attention_prefill_static(ctx, q, kv, kv, out, length - rows)
    torch.cuda.synchronize()
    assert (out == 0.5).all()                                            # rejected before any write
