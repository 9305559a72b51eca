"""Configuration and registry (no GPU)."""
import json

import pytest

from llm_serving_engine_b200.config import (ConfigError, Qwen2Config, known_architectures, load_config,
                                             register_architecture)
from llm_serving_engine_b200.models import expected_tensors
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_keys_of_config_json_are_read():
    config = Qwen2Config.from_dict(TINY_B)
    assert (config.vocab_size, config.hidden_size, config.intermediate_size) == (1000, 96, 256)
    assert (config.num_hidden_layers, config.num_attention_heads, config.num_key_value_heads) == (3, 3, 1)
    assert config.head_dim == 32 and config.rope_theta == 1e6 and config.rms_norm_eps == 1e-5
    assert config.tie_word_embeddings is False and config.attention_bias is True


def test_aliases_and_explicit_head_dim():
    values = dict(TINY_A)
    values["num_layers"] = values.pop("num_hidden_layers")
    values["max_seq_len"] = values.pop("max_position_embeddings")
    config = Qwen2Config.from_dict(values)
    assert config.num_hidden_layers == 2 and config.max_position_embeddings == 512
    assert Qwen2Config.from_dict(TINY_C).head_dim == 48


def test_missing_keys_are_named():
    values = dict(TINY_A)
    del values["rope_theta"], values["vocab_size"]
    with pytest.raises(ConfigError, match="rope_theta") as info:
        Qwen2Config.from_dict(values)
    assert "vocab_size" in str(info.value)


@pytest.mark.parametrize("change, message", [
    ({"use_sliding_window": True}, "sliding"),
    ({"num_key_value_heads": 3}, "divisible"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_scaling": {"type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"rope_pairing": "other"}, "rope_pairing"),
    ({"hidden_size": 66}, "divisible"),
])
def test_unsupported_configurations_are_refused(change, message):
    with pytest.raises(ConfigError, match=message):
        Qwen2Config.from_dict({**TINY_A, **change})


def test_registry_resolves_by_architecture_name(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    entry, config, spec = load_config(tmp_path)
    assert entry.name == "Qwen2ForCausalLM" and "Qwen2ForCausalLM" in known_architectures()
    assert spec.order == (0, 1) and len(spec.layers) == 2
    assert spec.layers[0].mixer.params["num_kv_heads"] == 2
    assert spec.layers[1].mixer.params["position"]["params"]["theta"] == 10000.0
    # model_type is the fallback when architectures is absent (the reference checks only that)
    values = dict(TINY_A)
    del values["architectures"]
    assert load_config(values)[0].name == "Qwen2ForCausalLM"
    with pytest.raises(ConfigError, match="unknown architecture"):
        load_config({**TINY_A, "architectures": ["NoSuchModel"]})


def test_expected_tensors_follow_the_configuration():
    _, _, spec = load_config(TINY_B)
    tensors = expected_tensors(spec)
    assert tensors["model.embed_tokens.weight"].shape == (1000, 96)
    assert tensors["model.layers.2.self_attn.k_proj.weight"].shape == (32, 96)
    assert tensors["model.layers.0.self_attn.q_proj.bias"].shape == (96,)
    assert tensors["model.layers.1.mlp.down_proj.weight"].shape == (96, 256)
    assert tensors["lm_head.weight"].shape == (1000, 96)
    _, _, tied = load_config(TINY_A)
    assert "lm_head.weight" not in expected_tensors(tied)
    _, _, nobias = load_config(TINY_C)
    assert "model.layers.0.self_attn.q_proj.bias" not in expected_tensors(nobias)
    assert expected_tensors(nobias)["model.layers.0.self_attn.o_proj.weight"].shape == (80, 480)


def test_another_architecture_can_be_registered():
    from llm_serving_engine_b200.models.qwen2 import build_qwen2_spec

    register_architecture("ToyAliasForCausalLM", Qwen2Config, build_qwen2_spec)
    entry, _, spec = load_config({**TINY_A, "architectures": ["ToyAliasForCausalLM"]})
    assert entry.name == "ToyAliasForCausalLM" and len(spec.layers) == 2
