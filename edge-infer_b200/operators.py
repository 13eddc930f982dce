"""Host-side mirror of edge-infer's direct-operator API (namespace op::cuda) over the C ABI.

Same names, argument meaning and error behaviour as
operators/include/operators/cuda/execution.hpp:28-157 and direct.hpp:23-47 of the reference,
for BF16 tensors. Tensors are torch CUDA tensors used purely as device buffers; every call
launches on the context's stream and allocates nothing (scratch is passed in).
"""
from __future__ import annotations

import ctypes as C

from . import abi


def _lib():
    return abi.load_library()


def prepare_execution_context(stream_ptr: int = 0) -> abi.Context:
    ctx = abi.Context()
    abi.check(_lib().ei_prepare_execution_context(C.c_void_p(stream_ptr), C.byref(ctx)))
    return ctx


def prepare_dense(weight, bias=None) -> abi.DenseWeight:
    """weight: logical [in, out] view (either row-major or the transpose of an [out, in] matrix)."""
    out = abi.DenseWeight()
    abi.check(_lib().ei_prepare_dense_bf16(abi.view2(weight), abi.view1(bias), C.byref(out)))
    return out


def prepare_awq(qweight, scales, zeros, group_size: int, input_features: int, bias=None) -> abi.AwqWeight:
    out = abi.AwqWeight()
    abi.check(_lib().ei_prepare_awq_bf16(abi.view2(qweight), abi.view2(scales), abi.view2(zeros), group_size,
                                         input_features, abi.view1(bias), C.byref(out)))
    return out


def linear_scratch_bytes(rows: int, input_features: int, output_features: int) -> int:
    return _lib().ei_linear_scratch_bytes(rows, input_features, output_features)


def _scratch(scratch):
    if scratch is None:
        return None, 0
    return C.c_void_p(scratch.data_ptr()), scratch.numel() * scratch.element_size()


def linear(ctx, input, weight: abi.DenseWeight, output, scratch=None) -> None:
    ptr, size = _scratch(scratch)
    abi.check(_lib().ei_linear_bf16(C.byref(ctx), abi.view2(input), C.byref(weight), abi.view2(output), ptr, size))


def awq_linear(ctx, input, weight: abi.AwqWeight, output, scratch=None) -> None:
    ptr, size = _scratch(scratch)
    abi.check(_lib().ei_awq_linear_bf16(C.byref(ctx), abi.view2(input), C.byref(weight), abi.view2(output), ptr, size))


def awq_gate_up_silu(ctx, input, weight: abi.AwqWeight, output) -> None:
    """Fused SwiGLU projection over a weight whose rows are [gate; up]: output = silu(gate) * up, staged as BF16."""
    abi.check(_lib().ei_awq_gate_up_silu_bf16(C.byref(ctx), abi.view2(input), C.byref(weight), abi.view2(output)))


def add(ctx, a, b, output) -> None:
    abi.check(_lib().ei_add_bf16(C.byref(ctx), abi.array(a), abi.array(b), abi.array(output)))


def silu_multiply(ctx, gate, up, output) -> None:
    abi.check(_lib().ei_silu_multiply_bf16(C.byref(ctx), abi.array(gate), abi.array(up), abi.array(output)))


def rms_norm(ctx, input, weight, output, rows: int, features: int, epsilon: float) -> None:
    abi.check(_lib().ei_rms_norm_bf16(C.byref(ctx), abi.array(input), abi.array(weight), abi.array(output), rows,
                                      features, epsilon))


def gather(ctx, ids, table, output) -> None:
    abi.check(_lib().ei_gather_bf16(C.byref(ctx), abi.view1(ids), abi.view2(table), abi.view2(output)))


def rope_precomputed(ctx, input, cache, offset: int = 0, offsets=None, pingpong=None) -> None:
    abi.check(_lib().ei_rope_precomputed_bf16(
        C.byref(ctx), abi.view3(input), abi.view2(cache), offset,
        C.c_void_p(offsets.data_ptr()) if offsets is not None else None,
        C.c_void_p(pingpong.data_ptr()) if pingpong is not None else None))


def build_rope_table(max_positions: int, head_dim: int, theta: float):
    import numpy as np
    table = np.empty((max_positions, head_dim), dtype=np.float32)
    abi.check(_lib().ei_build_rope_table(table.ctypes.data_as(C.c_void_p), max_positions, head_dim, theta))
    return table


def store_kv(ctx, source, capacity, offset: int, device_offset=None) -> None:
    abi.check(_lib().ei_store_kv_bf16(C.byref(ctx), abi.view2(source), abi.view2(capacity), offset,
                                      C.c_void_p(device_offset.data_ptr()) if device_offset is not None else None))


def attention_scratch_bytes(q_rows: int, query_heads: int, head_dim: int, kv_length: int) -> int:
    return _lib().ei_attention_scratch_bytes(q_rows, query_heads, head_dim, kv_length)


def attention_prefill(ctx, q, k, v, output, offset: int, scratch) -> None:
    ptr, size = _scratch(scratch)
    abi.check(_lib().ei_attention_prefill_bf16(C.byref(ctx), abi.view3(q), abi.view3(k), abi.view3(v),
                                               abi.view3(output), offset, ptr, size))


STATIC_ATTENTION_SCRATCH_BYTES = 10 * 1024 * 1024


def attention_prefill_static(ctx, q, k, v, output, offset: int) -> None:
    """attention_prefill with the split partials in the library's built-in array: allocates nothing, takes no
    scratch; shapes needing more than STATIC_ATTENTION_SCRATCH_BYTES raise ValueError. Calls on one device
    share the array and must not overlap."""
    abi.check(_lib().ei_attention_prefill_static_bf16(C.byref(ctx), abi.view3(q), abi.view3(k), abi.view3(v),
                                                      abi.view3(output), offset))


def attention_verify(ctx, q, k_capacity, v_capacity, output, device_offset, scratch) -> None:
    ptr, size = _scratch(scratch)
    abi.check(_lib().ei_attention_verify_bf16(C.byref(ctx), abi.view3(q), abi.view3(k_capacity),
                                              abi.view3(v_capacity), abi.view3(output),
                                              C.c_void_p(device_offset.data_ptr()), ptr, size))


def sample_scratch_bytes(rows: int, vocabulary: int) -> int:
    return _lib().ei_sample_scratch_bytes(rows, vocabulary)


def sample_greedy(ctx, logits, tokens, scratch) -> None:
    """op::cuda::sample with top_k == 1: tokens[row] = argmax of logits[row] (NaN as -inf, lowest index on ties)."""
    ptr, size = _scratch(scratch)
    abi.check(_lib().ei_sample_greedy_bf16(C.byref(ctx), abi.view2(logits), abi.view1(tokens), ptr, size))


def verify_accept(ctx, inputs, targets, rows: int, context_length, pending, result) -> None:
    abi.check(_lib().ei_verify_accept(C.byref(ctx), C.c_void_p(inputs.data_ptr()), C.c_void_p(targets.data_ptr()),
                                      rows, C.c_void_p(context_length.data_ptr()), C.c_void_p(pending.data_ptr()),
                                      C.c_void_p(result.data_ptr())))
