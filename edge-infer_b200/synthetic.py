"""Seeded synthetic models, prompts and drafts with the shapes and value distributions of the
benchmark configurations. They stand in for real checkpoints, which are not available offline.

Weights (per tensor, an independent PCG64 stream keyed by (seed, crc32(name))):
  dense linear / embedding / lm_head : N(0, 0.02), stored BF16 as the physical [out, in] matrix
  norm weights                        : 1.0 (or 1 + N(0, 0.1) with vary_norms, to exercise the weights)
  AWQ int4 linear                     : nibbles uniform 0..15 packed N-major (nibble k%8 at bit 4*(k%8)),
                                        zeros uniform 0..15 packed 8 per int32, BF16 scales uniform [0.002, 0.02]
Names follow the reference's weight schema (runtime/include/models/qwen3_model.hpp:363-408).
"""
from __future__ import annotations

import zlib
from typing import Dict, List, Tuple

import numpy as np

from .runtime import DENSE, QWEIGHT, SCALES, ZEROS, Shape

Tensors = Dict[str, List[Tuple[int, np.ndarray]]]


def float_to_bf16(values: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even FP32 -> BF16 payload (uint16)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = bits + 0x7FFF + ((bits >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def bf16_to_float(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64([seed, zlib.crc32(name.encode())]))


def dense_matrix(seed: int, name: str, out: int, inp: int, std: float = 0.02) -> np.ndarray:
    return float_to_bf16(_rng(seed, name).standard_normal((out, inp), dtype=np.float32) * np.float32(std))


def awq_triple(seed: int, name: str, out: int, inp: int, group: int = 128, padded_groups: int = 0):
    """(qweight int32 [out, in/8], scales BF16 [out, padded], zeros int32 [out, ceil(groups/8)])."""
    rng = _rng(seed, name)
    groups = inp // group
    padded = max(padded_groups, groups)
    nibbles = rng.integers(0, 16, size=(out, inp), dtype=np.uint32)
    shifts = (np.arange(inp, dtype=np.uint32) % 8) * 4
    qweight = np.bitwise_or.reduce((nibbles << shifts).reshape(out, inp // 8, 8), axis=2).astype(np.uint32)
    zero_values = rng.integers(0, 16, size=(out, groups), dtype=np.uint32)
    zero_stride = (groups + 7) // 8
    padded_zero = np.zeros((out, zero_stride * 8), dtype=np.uint32)
    padded_zero[:, :groups] = zero_values
    zshifts = (np.arange(zero_stride * 8, dtype=np.uint32) % 8) * 4
    zeros = np.bitwise_or.reduce((padded_zero << zshifts).reshape(out, zero_stride, 8), axis=2).astype(np.uint32)
    scales = np.full((out, padded), float_to_bf16(np.float32(-73.0)), dtype=np.uint16)  # poison in the padding
    scales[:, :groups] = float_to_bf16(rng.uniform(0.002, 0.02, size=(out, groups)).astype(np.float32))
    return qweight.view(np.int32), scales, zeros.view(np.int32)


def awq_dequantize(qweight: np.ndarray, scales: np.ndarray, zeros: np.ndarray, inp: int, group: int = 128,
                   round_bf16: bool = True) -> np.ndarray:
    """Dense FP32 [out, in] weights: (w - z) * scale, optionally rounded to BF16 (the rows > 1 rule)."""
    out = qweight.shape[0]
    k = np.arange(inp)
    w = (qweight.view(np.uint32)[:, k // 8] >> ((k % 8) * 4).astype(np.uint32)) & 15
    g = k // group
    z = (zeros.view(np.uint32)[:, g // 8] >> ((g % 8) * 4).astype(np.uint32)) & 15
    s = bf16_to_float(scales)[:, g]
    dense = (w.astype(np.float32) - z.astype(np.float32)) * s
    assert dense.shape == (out, inp)
    return bf16_to_float(float_to_bf16(dense)) if round_bf16 else dense


def make_model(shape: Shape, seed: int = 0, vary_norms: bool = False, padded_groups: int = 0) -> Tensors:
    """All tensors of a model on the host (numpy). Intended for shapes the CPU oracle can follow."""
    H, F, V = shape.hidden_size, shape.intermediate_size, shape.vocab_size
    qw, kvw = shape.n_heads * shape.head_dim, shape.n_kv_heads * shape.head_dim
    tensors: Tensors = {}

    def norm(name: str, width: int) -> None:
        values = np.ones(width, dtype=np.float32)
        if vary_norms:
            values = values + _rng(seed, name).standard_normal(width, dtype=np.float32) * np.float32(0.1)
        tensors[name] = [(DENSE, float_to_bf16(values))]

    def linear(name: str, out: int, inp: int) -> None:
        if shape.quant_type == 1:
            q, s, z = awq_triple(seed, name, out, inp, shape.group_size, padded_groups)
            tensors[name] = [(QWEIGHT, q), (SCALES, s), (ZEROS, z)]
        else:
            tensors[name] = [(DENSE, dense_matrix(seed, name, out, inp))]

    tensors["token_embeddings.weight"] = [(DENSE, dense_matrix(seed, "token_embeddings.weight", V, H))]
    norm("rms_out_w", H)
    if not shape.tied_embeddings:
        tensors["lm_head"] = [(DENSE, dense_matrix(seed, "lm_head", V, H))]
    for i in range(shape.n_layers):
        norm(f"rms_att_w{i}", H)
        norm(f"rms_ffn_w{i}", H)
        if shape.qk_norm:
            norm(f"q_norm{i}", shape.head_dim)
            norm(f"k_norm{i}", shape.head_dim)
        linear(f"wq{i}", qw, H)
        linear(f"wk{i}", kvw, H)
        linear(f"wv{i}", kvw, H)
        linear(f"wo{i}", H, qw)
        linear(f"w_gate{i}", F, H)
        linear(f"w_up{i}", F, H)
        linear(f"w_down{i}", H, F)
        if shape.qkv_bias:
            for proj, width in (("q", qw), ("k", kvw), ("v", kvw)):
                name = f"layers.{i}.self_attn.{proj}_proj.bias"
                tensors[name] = [(DENSE, float_to_bf16(_rng(seed, name).standard_normal(width, dtype=np.float32)
                                                       * np.float32(0.02)))]
    return tensors


def make_device_model(shape: Shape, seed: int = 0) -> Dict[str, List[Tuple[int, object]]]:
    """The same distributions generated directly in device memory with torch (for the multi-GB shapes
    no CPU oracle follows). Not bit-identical to make_model: a different generator."""
    import torch
    H, F, V = shape.hidden_size, shape.intermediate_size, shape.vocab_size
    qw, kvw = shape.n_heads * shape.head_dim, shape.n_kv_heads * shape.head_dim
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    tensors: Dict[str, List[Tuple[int, object]]] = {}

    def dense(out: int, inp: int):
        t = torch.empty((out, inp), dtype=torch.bfloat16, device="cuda")
        t.normal_(0.0, 0.02, generator=gen)
        return t

    def linear(name: str, out: int, inp: int) -> None:
        if shape.quant_type == 1:
            groups = inp // shape.group_size
            q = torch.randint(-2**31, 2**31 - 1, (out, inp // 8), dtype=torch.int32, device="cuda", generator=gen)
            z = torch.randint(-2**31, 2**31 - 1, (out, (groups + 7) // 8), dtype=torch.int32, device="cuda", generator=gen)
            s = (torch.rand((out, groups), device="cuda", generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
            tensors[name] = [(QWEIGHT, q), (SCALES, s), (ZEROS, z)]
        else:
            tensors[name] = [(DENSE, dense(out, inp))]

    def ones(name: str, width: int) -> None:
        tensors[name] = [(DENSE, torch.ones(width, dtype=torch.bfloat16, device="cuda"))]

    tensors["token_embeddings.weight"] = [(DENSE, dense(V, H))]
    ones("rms_out_w", H)
    if not shape.tied_embeddings:
        tensors["lm_head"] = [(DENSE, dense(V, H))]
    for i in range(shape.n_layers):
        ones(f"rms_att_w{i}", H)
        ones(f"rms_ffn_w{i}", H)
        if shape.qk_norm:
            ones(f"q_norm{i}", shape.head_dim)
            ones(f"k_norm{i}", shape.head_dim)
        linear(f"wq{i}", qw, H)
        linear(f"wk{i}", kvw, H)
        linear(f"wv{i}", kvw, H)
        linear(f"wo{i}", H, qw)
        linear(f"w_gate{i}", F, H)
        linear(f"w_up{i}", F, H)
        linear(f"w_down{i}", H, F)
        if shape.qkv_bias:
            for proj, width in (("q", qw), ("k", kvw), ("v", kvw)):
                b = torch.empty(width, dtype=torch.bfloat16, device="cuda")
                b.normal_(0.0, 0.02, generator=gen)
                tensors[f"layers.{i}.self_attn.{proj}_proj.bias"] = [(DENSE, b)]
    return tensors


def make_prompt(seed: int, length: int, vocab: int) -> np.ndarray:
    return _rng(seed, "prompt").integers(0, vocab, size=length, dtype=np.uint32)


def corrupt_drafts(seed: int, continuation: np.ndarray, p: float, vocab: int) -> np.ndarray:
    """Drafts = the greedy continuation with each position independently replaced, with probability p,
    by a uniform random id."""
    rng = _rng(seed, "drafts")
    replace = rng.random(len(continuation)) < p
    random_ids = rng.integers(0, vocab, size=len(continuation), dtype=np.uint32)
    return np.where(replace, random_ids, continuation).astype(np.uint32)


def substitution_mask(seed: int, length: int, p: float) -> np.ndarray:
    """Which positions corrupt_drafts(seed, continuation of `length`, p, ...) replaces (the same generator)."""
    return _rng(seed, "drafts").random(length) < p


# The benchmark configurations' shapes.
def qwen3_0_6b(**kw) -> Shape:
    return Shape(vocab_size=151936, n_layers=28, n_heads=16, n_kv_heads=8, hidden_size=1024, intermediate_size=3072,
                 tied_embeddings=True, **kw)


def qwen3_1_7b(**kw) -> Shape:
    return Shape(vocab_size=151936, n_layers=28, n_heads=16, n_kv_heads=8, hidden_size=2048, intermediate_size=6144, **kw)


def qwen3_8b_awq(**kw) -> Shape:
    return Shape(vocab_size=151936, n_layers=36, n_heads=32, n_kv_heads=8, hidden_size=4096, intermediate_size=12288,
                 quant_type=1, **kw)


def qwen25_7b_awq(**kw) -> Shape:
    return Shape(vocab_size=152064, n_layers=28, n_heads=28, n_kv_heads=4, hidden_size=3584, intermediate_size=18944,
                 quant_type=1, qk_norm=False, qkv_bias=True, max_position_embeddings=8448, **kw)
