"""Checkpoint admission for the verify path: HF-style decoder checkpoints (dense BF16 or AutoAWQ "GEMV" int4) to the
prepared-tensor names and layouts ei_model_create takes.

Mirrors what the reference does between a checkpoint and its prepared model:
  * AWQ metadata admission - only the 4-bit asymmetric GEMV packing, one agreed group size
    (bindings/python/include/decoder_weight_mapper.hpp:47-79, frontend/checkpoint.py:27-57);
  * tied / explicit output head (decoder_weight_mapper.hpp:81-102);
  * checkpoint key -> prepared name, kind and rank (decoder_weight_mapper.hpp:104-166, 219-253);
  * config.json -> decoder shape.
Linear weights stay in the checkpoint's own physical layout: [out, in] BF16, and for AWQ-GEMV
qweight int32 [out, in / 8], scales [out, groups (+ padding)], qzeros int32 [out, ceil(groups / 8)] - exactly what
the kernels stream, so nothing is repacked.

A minimal safetensors reader (the format is an 8-byte header length, a JSON header and raw little-endian data) is
included so that a local checkpoint directory can be read with numpy alone; nothing is ever fetched.
"""
from __future__ import annotations

import json
import re
import struct
from pathlib import Path
from typing import Dict, List, Mapping, Optional, Tuple

import numpy as np

from .runtime import Shape

DENSE, QWEIGHT, SCALES, ZEROS = 0, 1, 2, 3

MODEL_TYPES = ("qwen_bf16", "qwen_awq", "qwen3_bf16", "qwen3_awq")

_PROJECTIONS = {
    "self_attn.q_proj": "wq", "self_attn.k_proj": "wk", "self_attn.v_proj": "wv", "self_attn.o_proj": "wo",
    "mlp.gate_proj": "w_gate", "mlp.up_proj": "w_up", "mlp.down_proj": "w_down",
}
_FORMATS = {"weight": DENSE, "qweight": QWEIGHT, "scales": SCALES, "qzeros": ZEROS}
_LAYER = re.compile(r"^model\.layers\.(0|[1-9][0-9]*)\.(.+)$")


def awq_group_size(config: Mapping) -> int:
    """Admits the AWQ metadata of a config (top level and `quantization_config`): the method must be AWQ, the
    packing GEMV, 4 bits, asymmetric, and every declared group size the same. Returns the group size (128 when
    none is declared)."""
    quantization = config.get("quantization_config", {})
    if not isinstance(quantization, Mapping):
        raise ValueError("quantization_config must be a dictionary")
    group: Optional[int] = None
    for settings in (config, quantization):
        method = settings.get("quant_method", "awq")
        if not isinstance(method, str) or method.lower() != "awq":
            raise ValueError("Only AWQ quant_method is supported")
        version = settings.get("version", "gemv")
        if not isinstance(version, str) or version.lower() != "gemv":
            raise ValueError("Only AWQ GEMV packing is supported")
        for key in ("bits", "w_bit"):
            if key in settings and (type(settings[key]) is not int or settings[key] != 4):
                raise ValueError("Only 4-bit AWQ packing is supported")
        if "zero_point" in settings and settings["zero_point"] is not True:
            raise ValueError("AWQ zero_point must be true for asymmetric packing")
        for key in ("group_size", "q_group_size"):
            if key not in settings:
                continue
            declared = settings[key]
            if type(declared) is not int or not 0 < declared <= 2**31 - 1:
                raise ValueError(f"AWQ {key} must be a positive integer")
            if group is not None and declared != group:
                raise ValueError("Contradictory AWQ group sizes")
            group = declared
    return 128 if group is None else group


def parse_name(source: str, qk_norm: bool, n_layers: int = 0) -> Tuple[str, int, int]:
    """Checkpoint key -> (prepared name, kind, rank). Raises ValueError for a key the decoder does not know, a
    malformed layer index or a layer beyond the configuration."""
    if source == "model.embed_tokens.weight":
        return "token_embeddings.weight", DENSE, 2
    if source == "model.norm.weight":
        return "rms_out_w", DENSE, 1
    for prefix in ("lm_head.", "model.lm_head."):
        if source.startswith(prefix):
            return _projection(source, "lm_head", "lm_head.bias", source[len(prefix):])
    match = _LAYER.match(source)
    if not match:
        if source.startswith("model.layers."):
            raise ValueError("Malformed decoder layer index: " + source)
        raise ValueError("Unsupported decoder weight key: " + source)
    layer, suffix = int(match.group(1)), match.group(2)
    if layer > 2**31 - 1:
        raise ValueError("Decoder layer index exceeds the supported range: " + source)
    if n_layers and layer >= n_layers:
        raise ValueError("Decoder weight layer exceeds configuration: " + source)
    norms = {"input_layernorm.weight": "rms_att_w", "post_attention_layernorm.weight": "rms_ffn_w"}
    if qk_norm:
        norms.update({"self_attn.q_norm.weight": "q_norm", "self_attn.k_norm.weight": "k_norm"})
    if suffix in norms:
        return f"{norms[suffix]}{layer}", DENSE, 1
    base, _, fmt = suffix.rpartition(".")
    if base in _PROJECTIONS:
        return _projection(source, f"{_PROJECTIONS[base]}{layer}", f"layers.{layer}.{base}.bias", fmt)
    raise ValueError("Unsupported decoder weight key: " + source)


def _projection(source: str, name: str, bias_name: str, fmt: str) -> Tuple[str, int, int]:
    if fmt == "bias":
        return bias_name, DENSE, 1
    if fmt in _FORMATS:
        return name, _FORMATS[fmt], 2
    raise ValueError("Unsupported decoder weight key: " + source)


def shape_from_config(config: Mapping, model_type: str) -> Shape:
    """Decoder shape from an HF config.json dictionary."""
    if model_type not in MODEL_TYPES:
        raise ValueError(f"Unsupported model type: {model_type}")
    heads = int(config["num_attention_heads"])
    head_dim = int(config.get("head_dim", int(config["hidden_size"]) // heads))
    awq = model_type.endswith("_awq")
    return Shape(vocab_size=int(config["vocab_size"]), n_layers=int(config["num_hidden_layers"]), n_heads=heads,
                 n_kv_heads=int(config.get("num_key_value_heads", heads)), hidden_size=int(config["hidden_size"]),
                 intermediate_size=int(config["intermediate_size"]), head_dim=head_dim,
                 max_position_embeddings=int(config.get("max_position_embeddings", 4096)),
                 rms_norm_eps=float(config.get("rms_norm_eps", 1e-6)), rope_theta=float(config.get("rope_theta", 1e6)),
                 quant_type=1 if awq else 0, group_size=awq_group_size(config) if awq else 128,
                 qk_norm=model_type.startswith("qwen3"), qkv_bias=not model_type.startswith("qwen3"),
                 tied_embeddings=False, bos_token_id=int(config.get("bos_token_id", 0) or 0),
                 eos_token_id=_first_int(config.get("eos_token_id", 0xFFFFFFFF)))


def _first_int(value) -> int:
    if isinstance(value, (list, tuple)):
        value = value[0]
    return int(value)


def _bits(array, name: str, kind: int):
    """Payload in the element type the library takes: BF16 as uint16 for dense / scales, int32 for packed data.
    Accepts numpy arrays and torch tensors (host or device); floating-point inputs are rounded to BF16."""
    if hasattr(array, "detach"):                             # torch tensor: stays where it is
        import torch
        if kind in (QWEIGHT, ZEROS):
            if array.dtype != torch.int32:
                raise ValueError("AWQ packed weights and zeros must have int32 dtype: " + name)
            return array.contiguous()
        return array.to(torch.bfloat16).contiguous()
    array = np.asarray(array)
    if kind in (QWEIGHT, ZEROS):
        if array.dtype.kind != "i" or array.dtype.itemsize != 4:
            raise ValueError("AWQ packed weights and zeros must have int32 dtype: " + name)
        return np.ascontiguousarray(array)
    if array.dtype == np.uint16:                             # already a BF16 payload
        return np.ascontiguousarray(array)
    from .synthetic import float_to_bf16
    return float_to_bf16(np.ascontiguousarray(array, dtype=np.float32))


def admit(config: Mapping, weights: Mapping, model_type: str):
    """(Shape, tensors for runtime.Model) from a config dictionary and a checkpoint's name -> array mapping.
    Validates names, ranks, AWQ completeness (packed weight, scales and zero points come together and never beside a
    dense weight of the same projection) and resolves a declared embedding tie."""
    shape = shape_from_config(config, model_type)
    tied = config.get("tie_word_embeddings", False)
    if not isinstance(tied, bool):
        raise ValueError("tie_word_embeddings must be a boolean")
    if "model.embed_tokens.weight" not in weights:
        raise ValueError("Decoder checkpoint requires model.embed_tokens.weight")
    has_head = any(key.startswith(("lm_head.", "model.lm_head.")) for key in weights)
    if not has_head and not tied:
        raise ValueError("Untied decoder checkpoint requires an explicit lm_head weight")
    tensors: Dict[str, List[Tuple[int, object]]] = {}
    for source, array in weights.items():
        if not isinstance(source, str):
            raise ValueError("Decoder checkpoint weight names must be strings")
        name, kind, rank = parse_name(source, shape.qk_norm, shape.n_layers)
        if kind != DENSE and shape.quant_type != 1:
            raise ValueError("Packed decoder weights require an AWQ model: " + name)
        payload = _bits(array, source, kind)
        if len(payload.shape) != rank:
            raise ValueError("Decoder checkpoint weight rank mismatch: " + name)
        entries = tensors.setdefault(name, [])
        if any(existing == kind for existing, _ in entries):
            raise ValueError("Duplicate normalized decoder weight: " + name)
        entries.append((kind, payload))
    for name, entries in tensors.items():
        kinds = {kind for kind, _ in entries}
        if kinds & {QWEIGHT, SCALES, ZEROS}:
            if DENSE in kinds:
                raise ValueError("Dense and AWQ weights overlap: " + name)
            if kinds != {QWEIGHT, SCALES, ZEROS}:
                raise ValueError("Incomplete AWQ decoder weight: " + name)
    shape.tied_embeddings = not has_head
    return shape, tensors


# ---------------------------------------------------------------- safetensors (read-only, numpy)
_DTYPES = {"BF16": (np.uint16, 2), "F16": (np.float16, 2), "F32": (np.float32, 4), "I32": (np.int32, 4),
           "I64": (np.int64, 8), "U8": (np.uint8, 1)}


def read_safetensors(path) -> Dict[str, np.ndarray]:
    """name -> array of one .safetensors file, memory-mapped. BF16 tensors come back as uint16 payloads."""
    path = Path(path)
    with path.open("rb") as handle:
        (header_bytes,) = struct.unpack("<Q", handle.read(8))
        header = json.loads(handle.read(header_bytes))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + header_bytes)
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        if entry["dtype"] not in _DTYPES:
            raise ValueError(f"Unsupported safetensors dtype {entry['dtype']}: {name}")
        dtype, _ = _DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        tensors[name] = data[begin:end].view(dtype).reshape(entry["shape"])
    return tensors


def _checkpoint_file(root: Path, name) -> Path:
    if not isinstance(name, str) or not name or Path(name).is_absolute():
        raise ValueError("Checkpoint shard names must be relative paths")
    path = (root / name).resolve()
    if root not in path.parents:
        raise ValueError("Checkpoint shards must stay inside the model directory")
    if not path.is_file():
        raise FileNotFoundError(path)
    return path


def load_directory(model_path, model_type: str):
    """(config, weights) of a local checkpoint directory: config.json plus model.safetensors or the shards its index
    names. Never fetches anything."""
    if model_type not in MODEL_TYPES:
        raise ValueError(f"Unsupported model type: {model_type}")
    root = Path(model_path).resolve()
    config = json.loads((root / "config.json").read_text(encoding="utf-8"))
    if not isinstance(config, dict):
        raise ValueError("Model configuration must be a JSON object")
    index_path = root / "model.safetensors.index.json"
    if index_path.is_file():
        index = json.loads(index_path.read_text(encoding="utf-8"))
        weight_map = index.get("weight_map") if isinstance(index, dict) else None
        if not isinstance(weight_map, dict) or not weight_map:
            raise ValueError("The safetensors index must contain a nonempty weight_map")
        shards = sorted({_checkpoint_file(root, shard) for shard in weight_map.values()})
        wanted = set(weight_map)
    else:
        shards, wanted = [_checkpoint_file(root, "model.safetensors")], None
    weights: Dict[str, np.ndarray] = {}
    for shard in shards:
        for name, array in read_safetensors(shard).items():
            if wanted is None or name in wanted:
                weights[name] = array
    if not weights:
        raise ValueError("The checkpoint contains no tensors")
    return config, weights
