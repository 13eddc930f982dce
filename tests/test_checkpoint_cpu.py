"""Checkpoint admission on the CPU: AWQ metadata, checkpoint key mapping, tie resolution and the safetensors reader.
The cases follow what the reference's binding layer admits and rejects
(bindings/python/include/decoder_weight_mapper.hpp:47-166, 219-253; frontend/checkpoint.py:27-57)."""
import json
import struct

import numpy as np
import pytest


@pytest.fixture(scope="module")
def checkpoint(package):
    return package.checkpoint


def test_awq_metadata_admission(checkpoint):
    assert checkpoint.awq_group_size({}) == 128
    assert checkpoint.awq_group_size({"quantization_config": {"quant_method": "AWQ", "version": "GEMV", "bits": 4,
                                                              "zero_point": True, "group_size": 64}}) == 64
    assert checkpoint.awq_group_size({"q_group_size": 128, "quantization_config": {"group_size": 128}}) == 128
    for bad in ({"quantization_config": {"quant_method": "gptq"}},
                {"quantization_config": {"version": "GEMM"}},
                {"quantization_config": {"bits": 8}},
                {"w_bit": True},                                            # a boolean is not a bit count
                {"quantization_config": {"zero_point": False}},
                {"group_size": 128, "quantization_config": {"group_size": 64}},
                {"group_size": 0},
                {"quantization_config": [1, 2]}):
        with pytest.raises(ValueError):
            checkpoint.awq_group_size(bad)


def test_checkpoint_key_mapping(checkpoint):
    D, Q, S, Z = checkpoint.DENSE, checkpoint.QWEIGHT, checkpoint.SCALES, checkpoint.ZEROS
    parse = checkpoint.parse_name
    assert parse("model.embed_tokens.weight", True) == ("token_embeddings.weight", D, 2)
    assert parse("model.norm.weight", True) == ("rms_out_w", D, 1)
    assert parse("lm_head.weight", True) == ("lm_head", D, 2)
    assert parse("model.lm_head.qweight", True) == ("lm_head", Q, 2)
    assert parse("model.layers.7.input_layernorm.weight", True) == ("rms_att_w7", D, 1)
    assert parse("model.layers.7.post_attention_layernorm.weight", False) == ("rms_ffn_w7", D, 1)
    assert parse("model.layers.0.self_attn.q_norm.weight", True) == ("q_norm0", D, 1)
    assert parse("model.layers.3.self_attn.k_proj.bias", False) == ("layers.3.self_attn.k_proj.bias", D, 1)
    assert parse("model.layers.12.mlp.down_proj.qzeros", True) == ("w_down12", Z, 2)
    assert parse("model.layers.12.mlp.gate_proj.scales", True) == ("w_gate12", S, 2)
    assert parse("model.layers.12.self_attn.o_proj.weight", True, 13) == ("wo12", D, 2)
    for bad in ("model.layers.01.mlp.up_proj.weight",                       # leading zero
                "model.layers.x.mlp.up_proj.weight", "model.layers.2", "model.rotary.inv_freq",
                "model.layers.2.mlp.up_proj.g_idx", "model.layers.2.self_attn.rotary_emb.inv_freq"):
        with pytest.raises(ValueError):
            parse(bad, True)
    with pytest.raises(ValueError):
        parse("model.layers.0.self_attn.q_norm.weight", False)              # a model without QK-norm has no such weight
    with pytest.raises(ValueError):
        parse("model.layers.13.mlp.up_proj.weight", True, 13)              # beyond the configured depth


def tiny_config(**extra):
    config = {"vocab_size": 32, "num_hidden_layers": 1, "num_attention_heads": 2, "num_key_value_heads": 1,
              "hidden_size": 256, "head_dim": 128, "intermediate_size": 256, "max_position_embeddings": 64,
              "rms_norm_eps": 1e-6, "rope_theta": 1e6, "eos_token_id": [31, 30]}
    config.update(extra)
    return config


def tiny_awq_weights(package, tied=False):
    syn = package.synthetic
    H, F = 256, 256
    weights = {"model.embed_tokens.weight": np.zeros((32, H), dtype=np.float32), "model.norm.weight": np.ones(H, np.float32),
               "model.layers.0.input_layernorm.weight": np.ones(H, np.float32),
               "model.layers.0.post_attention_layernorm.weight": np.ones(H, np.float32),
               "model.layers.0.self_attn.q_norm.weight": np.ones(128, np.float32),
               "model.layers.0.self_attn.k_norm.weight": np.ones(128, np.float32)}
    if not tied:
        weights["lm_head.weight"] = np.zeros((32, H), dtype=np.float32)
    for base, (out, inp) in {"self_attn.q_proj": (256, H), "self_attn.k_proj": (128, H), "self_attn.v_proj": (128, H),
                             "self_attn.o_proj": (H, 256), "mlp.gate_proj": (F, H), "mlp.up_proj": (F, H),
                             "mlp.down_proj": (H, F)}.items():
        q, s, z = syn.awq_triple(1, base, out, inp)
        weights[f"model.layers.0.{base}.qweight"] = q
        weights[f"model.layers.0.{base}.scales"] = s
        weights[f"model.layers.0.{base}.qzeros"] = z
    return weights


def test_admission_of_a_whole_checkpoint(package, checkpoint):
    shape, tensors = checkpoint.admit(tiny_config(), tiny_awq_weights(package), "qwen3_awq")
    assert shape.quant_type == 1 and shape.qk_norm and not shape.qkv_bias and not shape.tied_embeddings
    assert shape.eos_token_id == 31 and shape.n_kv_heads == 1
    assert sorted(kind for kind, _ in tensors["wq0"]) == [checkpoint.QWEIGHT, checkpoint.SCALES, checkpoint.ZEROS]
    assert tensors["token_embeddings.weight"][0][1].dtype == np.uint16      # rounded to BF16 payloads
    tied_shape, tied = checkpoint.admit(tiny_config(tie_word_embeddings=True), tiny_awq_weights(package, tied=True),
                                        "qwen3_awq")
    assert tied_shape.tied_embeddings and "lm_head" not in tied
    with pytest.raises(ValueError, match="explicit lm_head"):
        checkpoint.admit(tiny_config(), tiny_awq_weights(package, tied=True), "qwen3_awq")
    incomplete = tiny_awq_weights(package)
    del incomplete["model.layers.0.mlp.up_proj.qzeros"]
    with pytest.raises(ValueError, match="Incomplete AWQ"):
        checkpoint.admit(tiny_config(), incomplete, "qwen3_awq")
    overlapping = tiny_awq_weights(package)
    overlapping["model.layers.0.mlp.up_proj.weight"] = np.zeros((256, 256), np.float32)
    with pytest.raises(ValueError, match="overlap"):
        checkpoint.admit(tiny_config(), overlapping, "qwen3_awq")
    wrong_type = tiny_awq_weights(package)
    wrong_type["model.layers.0.mlp.up_proj.qweight"] = wrong_type["model.layers.0.mlp.up_proj.qweight"].astype(np.int64)
    with pytest.raises(ValueError, match="int32"):
        checkpoint.admit(tiny_config(), wrong_type, "qwen3_awq")
    with pytest.raises(ValueError, match="require an AWQ model"):
        checkpoint.admit(tiny_config(), tiny_awq_weights(package), "qwen3_bf16")
    with pytest.raises(ValueError, match="rank mismatch"):
        checkpoint.admit(tiny_config(), dict(tiny_awq_weights(package), **{"model.norm.weight": np.ones((1, 256), np.float32)}),
                         "qwen3_awq")


def write_safetensors(path, tensors):
    header, offset, blobs = {}, 0, []
    for name, (dtype, array) in tensors.items():
        blob = np.ascontiguousarray(array).tobytes()
        header[name] = {"dtype": dtype, "shape": list(array.shape), "data_offsets": [offset, offset + len(blob)]}
        offset += len(blob)
        blobs.append(blob)
    encoded = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(encoded)) + encoded + b"".join(blobs))


def test_local_directory_with_sharded_safetensors(package, checkpoint, tmp_path):
    weights = tiny_awq_weights(package)
    names = sorted(weights)
    for shard, part in (("a.safetensors", names[::2]), ("b.safetensors", names[1::2])):
        write_safetensors(tmp_path / shard, {n: ("I32" if weights[n].dtype == np.int32 else
                                                 "BF16" if weights[n].dtype == np.uint16 else "F32", weights[n])
                                             for n in part})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {n: ("a.safetensors" if n in names[::2] else "b.safetensors") for n in names}}))
    (tmp_path / "config.json").write_text(json.dumps(tiny_config(quantization_config={"quant_method": "awq",
                                                                                       "version": "gemv", "bits": 4})))
    config, loaded = checkpoint.load_directory(tmp_path, "qwen3_awq")
    assert sorted(loaded) == names
    for name in names:
        assert np.array_equal(np.asarray(loaded[name]), weights[name]), name
    shape, tensors = checkpoint.admit(config, loaded, "qwen3_awq")
    assert shape.group_size == 128 and len(tensors) == 14
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {"x": "../outside.safetensors"}}))
    with pytest.raises((ValueError, FileNotFoundError)):
        checkpoint.load_directory(tmp_path, "qwen3_awq")
