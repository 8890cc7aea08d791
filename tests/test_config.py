"""Typed configuration from config.json keys, its errors, and the architecture registry."""

import json

import pytest

import tiny
from ampere_kv_engine_b200.config.model_config import ConfigError, read_config_json
from ampere_kv_engine_b200.models.registry import ARCHITECTURES, config_from_dict, load_config


def test_parses_both_tiny_configs_and_they_differ_everywhere():
    _, a = config_from_dict(tiny.config("A"))
    _, b = config_from_dict(tiny.config("B"))
    for key in ("num_hidden_layers", "hidden_size", "num_attention_heads", "head_dim", "intermediate_size",
                "vocab_size", "rope_theta", "rms_norm_eps", "max_position_embeddings", "tie_word_embeddings",
                "attention_bias", "use_sliding_window", "eos_token_id"):
        assert getattr(a, key) != getattr(b, key), key
    assert a.num_attention_heads // a.num_key_value_heads != b.num_attention_heads // b.num_key_value_heads
    assert a.num_attention_heads * a.head_dim == a.hidden_size and b.num_attention_heads * b.head_dim != b.hidden_size
    assert a.eos_token_id == (3,) and b.eos_token_id == (7, 9)
    assert [a.window_of_layer(i) for i in range(2)] == [None, None]
    assert [b.window_of_layer(i) for i in range(3)] == [None, 40, 40]


def test_defaults_follow_the_checkpoint_conventions():
    raw = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 100, "hidden_size": 64, "num_hidden_layers": 1,
           "num_attention_heads": 4, "intermediate_size": 96}
    _, c = config_from_dict(raw)
    assert c.num_key_value_heads == 4 and c.head_dim == 16 and c.rope_theta == 10000.0 and c.rms_norm_eps == 1e-6
    assert c.tie_word_embeddings is False and c.eos_token_id == ()


def test_layer_types_choose_the_window_layer_by_layer():
    raw = tiny.config("B")
    raw["layer_types"] = ["sliding_attention", "full_attention", "sliding_attention"]
    _, c = config_from_dict(raw)
    assert [c.window_of_layer(i) for i in range(3)] == [40, None, 40]


@pytest.mark.parametrize("change,match", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"head_dim": 15}, "head_dim"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"eos_token_id": "two"}, "eos_token_id"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_errors_name_the_key(change, match):
    raw = tiny.config("A")
    raw.update(change)
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_missing_key_and_unknown_architecture():
    raw = tiny.config("A")
    del raw["intermediate_size"]
    with pytest.raises(ConfigError, match="intermediate_size"):
        config_from_dict(raw)
    raw = tiny.config("A")
    raw["architectures"] = ["SomethingElseForCausalLM"]
    with pytest.raises(ConfigError, match="not registered.*Qwen3ForCausalLM"):
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in ARCHITECTURES


def test_reads_model_folder_and_generation_config(tmp_path):
    raw = tiny.config("A")
    del raw["eos_token_id"]
    (tmp_path / "config.json").write_text(json.dumps(raw))
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [5, 6]}))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Qwen3ForCausalLM" and cfg.eos_token_id == (5, 6)
    with pytest.raises(ConfigError, match="no config.json"):
        read_config_json(str(tmp_path / "nowhere"))


def test_round_trip_through_to_dict():
    _, b = config_from_dict(tiny.config("B"))
    _, again = config_from_dict(b.to_dict())
    assert again == b


def test_spec_is_layer_by_layer_data():
    _, b = config_from_dict(tiny.config("B"))
    spec = ARCHITECTURES["Qwen3ForCausalLM"].build_spec(b)
    assert [l.mixer.params["window"] for l in spec.layers] == [None, 40, 40]
    assert [e.layer for e in spec.schedule] == [0, 1, 2]
    assert spec.layers[1].mixer.prefix == "model.layers.1.self_attn"
    assert spec.head.params["tied"] is False
