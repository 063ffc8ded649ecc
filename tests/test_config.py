"""Typed configuration and the registry (CPU)."""
import copy
import json

import pytest

from hi_b200.config import ConfigError, Llama4TextConfig, load_architecture, lookup, registered_architectures
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_every_key_is_read():
    a = Llama4TextConfig.from_json(TINY_A)
    assert (a.vocab_size, a.hidden_size, a.num_hidden_layers, a.num_attention_heads, a.num_key_value_heads,
            a.head_dim) == (256, 64, 2, 4, 2, 16)
    assert a.rms_norm_eps == 1e-5 and a.rope_theta == 10000.0 and a.rope_scaling is None
    assert a.attention_chunk_size == 32 and a.rope_layers == (True, False)
    assert a.use_qk_norm and a.attn_temperature_tuning and a.floor_scale == 16 and a.attn_scale == 0.1
    assert a.moe_layers == (True, True) and a.num_local_experts == 4 and a.num_experts_per_tok == 1
    assert a.intermediate_size == 128 and a.intermediate_size_mlp == 256 and a.eos_token_ids == (2,)
    b = Llama4TextConfig.from_json(TINY_B)          # nested text_config
    assert (b.vocab_size, b.hidden_size, b.num_hidden_layers, b.head_dim) == (515, 192, 6, 32)
    assert b.architectures == ("Llama4ForConditionalGeneration",) and b.model_type == "llama4"
    assert b.rope_scaling.factor == 8.0 and b.rope_scaling.original_max_position_embeddings == 64
    assert b.rope_layers == (True, True, True, False, True, True)
    assert b.moe_layers == (False, True, False, True, False, True)
    assert b.num_experts_per_tok == 2 and not b.use_qk_norm and not b.attn_temperature_tuning
    assert b.eos_token_ids == (1, 7) and b.tie_word_embeddings
    c = Llama4TextConfig.from_json(TINY_C)          # explicit lists win over intervals
    assert c.rope_layers == (True, False, True) and c.moe_layers == (True, False, True) and c.rope_interleaved


def test_defaults_follow_the_reference_parser():
    raw = {"model_type": "llama4_text", "hidden_size": 64, "num_attention_heads": 4, "vocab_size": 100,
           "num_hidden_layers": 4, "num_local_experts": 2, "intermediate_size": 32}
    c = Llama4TextConfig.from_json(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16          # config.rs:357, 120-128
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 1e6           # config.rs:424-433
    assert c.rope_layers == (True, True, True, False)               # models.rs:5953-5954
    assert c.moe_layers == (True,) * 4 and c.num_experts_per_tok == 1
    assert not c.use_qk_norm and c.qk_norm_eps == 1e-6 and c.attention_chunk_size == 8192


def test_generation_config_eos_ids_are_merged(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [2, 9, 11]}))
    _arch, cfg, _raw = load_architecture(str(tmp_path))
    assert cfg.eos_token_ids == (2, 9, 11)


@pytest.mark.parametrize("change,word", [
    ({"hidden_size": None}, "hidden_size"), ({"vocab_size": None}, "vocab_size"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"head_dim": 15}, "head_dim"),
    ({"attention_chunk_size": 0}, "attention_chunk_size"), ({"num_experts_per_tok": 5}, "num_experts_per_tok"),
    ({"num_local_experts": 0}, "num_local_experts"), ({"floor_scale": 0}, "floor_scale"),
    ({"rope_scaling": {"rope_type": "yarn"}}, "rope_scaling"), ({"hidden_act": "gelu"}, "hidden_act"),
    ({"no_rope_layers": [1]}, "no_rope_layers"), ({"moe_layers": [9]}, "moe_layers"),
    ({"num_hidden_layers": "two"}, "num_hidden_layers"),
])
def test_bad_configs_name_the_key(change, word):
    raw = copy.deepcopy(TINY_A)
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError) as e:
        Llama4TextConfig.from_json(raw)
    assert word in str(e.value)


def test_dense_layers_need_their_width():
    raw = copy.deepcopy(TINY_B)
    raw["text_config"].pop("intermediate_size_mlp")
    with pytest.raises(ConfigError, match="intermediate_size_mlp"):
        Llama4TextConfig.from_json(raw)


def test_registry_by_architecture_then_model_type():
    assert lookup({"architectures": ["Llama4ForConditionalGeneration"]}).name == "llama4_text"
    assert lookup({"architectures": ["Nope"], "model_type": "llama4_text"}).name == "llama4_text"
    assert lookup({"model_type": "llama4"}).name == "llama4_text"
    with pytest.raises(ConfigError) as e:
        lookup({"architectures": ["QwenForCausalLM"], "model_type": "qwen2"})
    assert "Llama4ForCausalLM" in str(e.value) and "Llama4ForCausalLM" in registered_architectures()


def test_spec_follows_the_configuration_layer_by_layer():
    arch = lookup(TINY_B)
    spec = arch.build_spec(arch.parse_config(TINY_B, None))
    kinds = [(l.mixer.params["window"], l.mixer.params["position"].kind, l.feed_forward.kind) for l in spec.layers]
    assert kinds[0] == (("chunk", 16), "rope", "dense_swiglu")
    assert kinds[3] == (None, "none", "moe_sigmoid")
    assert kinds[5] == (("chunk", 16), "rope", "moe_sigmoid")
    assert [e.layer for e in spec.schedule] == list(range(6))
    a = arch.build_spec(arch.parse_config(TINY_A, None))
    assert a.layers[1].mixer.params["temperature"] == (16.0, 0.1) and a.layers[0].mixer.params["temperature"] is None
    assert a.layers[0].mixer.params["qk_norm"] and not a.layers[1].mixer.params["qk_norm"]
    biased = arch.build_spec(arch.parse_config(dict(TINY_A, attention_bias=True), None))
    assert biased.layers[0].mixer.params["bias"] and not a.layers[0].mixer.params["bias"]
    with pytest.raises(ConfigError, match="head_dim"):
        arch.build_spec(arch.parse_config(dict(TINY_A, head_dim=24), None))
