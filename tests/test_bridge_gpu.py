"""The reference's Python binding surface over this library, on the GPU: a model admitted from an HF-named
checkpoint gives exactly what the same tensors give under their prepared names, and a speculative session
generates exactly the ordinary greedy tokens of the target (the reference's own criterion for its decoder,
runtime/tests/inference_generation_test.cpp:488-538)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HF_PROJECTIONS = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
                  "w_gate": "mlp.gate_proj", "w_up": "mlp.up_proj", "w_down": "mlp.down_proj"}
HF_SUFFIX = {0: "weight", 1: "qweight", 2: "scales", 3: "qzeros"}


def hf_checkpoint(shape, tensors):
    """The prepared-name tensors of synthetic.make_model under the names an HF / AutoAWQ checkpoint gives them."""
    config = {"vocab_size": shape.vocab_size, "num_hidden_layers": shape.n_layers, "num_attention_heads": shape.n_heads,
              "num_key_value_heads": shape.n_kv_heads, "hidden_size": shape.hidden_size, "head_dim": shape.head_dim,
              "intermediate_size": shape.intermediate_size, "max_position_embeddings": shape.max_position_embeddings,
              "rms_norm_eps": shape.rms_norm_eps, "rope_theta": shape.rope_theta, "eos_token_id": shape.vocab_size - 1,
              "tie_word_embeddings": shape.tied_embeddings}
    if shape.quant_type == 1:
        config["quantization_config"] = {"quant_method": "awq", "version": "GEMV", "bits": 4, "zero_point": True,
                                         "group_size": shape.group_size}
    weights = {}
    for name, kinds in tensors.items():
        for kind, data in kinds:
            if name == "token_embeddings.weight":
                key = "model.embed_tokens.weight"
            elif name == "rms_out_w":
                key = "model.norm.weight"
            elif name == "lm_head":
                key = "lm_head." + HF_SUFFIX[kind]
            elif name.startswith("layers."):
                key = "model." + name
            else:
                stem = name.rstrip("0123456789")
                layer = name[len(stem):]
                norm = {"rms_att_w": "input_layernorm", "rms_ffn_w": "post_attention_layernorm",
                        "q_norm": "self_attn.q_norm", "k_norm": "self_attn.k_norm"}
                if stem in norm:
                    key = f"model.layers.{layer}.{norm[stem]}.weight"
                else:
                    key = f"model.layers.{layer}.{HF_PROJECTIONS[stem]}.{HF_SUFFIX[kind]}"
            weights[key] = data
    return config, weights


@pytest.mark.parametrize("kind", ["qwen3_awq", "qwen_awq"])
def test_hf_named_checkpoint_equals_prepared_names(cuda, package, kind):
    syn = package.synthetic
    S = package.Shape
    shape = S(vocab_size=1024, n_layers=2, n_heads=4, n_kv_heads=2, hidden_size=512, intermediate_size=1024, quant_type=1,
              max_position_embeddings=256, qk_norm=kind == "qwen3_awq", qkv_bias=kind == "qwen_awq",
              eos_token_id=1023)
    tensors = syn.make_model(shape, seed=4, vary_norms=True)
    direct = package.Model(shape, tensors).new_session(128)
    config, weights = hf_checkpoint(shape, tensors)
    admitted_shape, admitted = package.checkpoint.admit(config, weights, kind)
    assert admitted_shape.qk_norm == shape.qk_norm and admitted_shape.qkv_bias == shape.qkv_bias
    bridged = package.Model(admitted_shape, admitted).new_session(128)
    prompt = syn.make_prompt(4, 33, shape.vocab_size)
    direct.prefill(prompt)
    bridged.prefill(prompt)
    assert np.array_equal(direct.read_logits(1), bridged.read_logits(1))


def test_speculative_session_generates_the_ordinary_greedy_tokens(cuda, package):
    syn, bridge = package.synthetic, package.model_bridge
    S = package.Shape
    target_shape = S(vocab_size=1024, n_layers=2, n_heads=4, n_kv_heads=2, hidden_size=512, intermediate_size=1024,
                     quant_type=1, max_position_embeddings=256, eos_token_id=1023)
    draft_shape = S(vocab_size=1024, n_layers=1, n_heads=2, n_kv_heads=1, hidden_size=256, intermediate_size=512,
                    max_position_embeddings=256, eos_token_id=1023)
    target = bridge.Model(*hf_checkpoint(target_shape, syn.make_model(target_shape, seed=5)), model_type="qwen3_awq")
    draft = bridge.Model(*hf_checkpoint(draft_shape, syn.make_model(draft_shape, seed=6)), model_type="qwen3_bf16")
    assert target.max_context_length == 256 and target.device == "cuda"
    prompt = [int(t) for t in syn.make_prompt(5, 19, 1024)]
    ordinary, speculative = [], []
    plain = target.new_session(128)
    plain.generate(prompt, ordinary.append, max_length=60)
    spec = target.new_speculative_session(draft, capacity=128, spec_length=4)
    assert spec.speculative and not plain.speculative and spec.capacity == 128
    spec.generate(prompt, speculative.append, max_length=60)
    assert len(ordinary) == 60 - len(prompt) and speculative == ordinary
    again = []
    spec.reset()
    spec.generate(prompt, again.append, max_length=60)              # a session is reusable after reset
    assert again == ordinary
    with pytest.raises(ValueError, match="greedy"):
        plain.generate(prompt, ordinary.append, max_length=60, temperature=0.8, top_k=50)
    with pytest.raises(ValueError):
        target.new_speculative_session(draft, spec_length=0)
