"""Typed configuration and registry, after the reference's crates/llm-models/tests/qwen3_dense_config.rs."""
import copy
import json

import pytest

import kirai_b200
from kirai_b200.config import ConfigError, Qwen3Config
from kirai_b200.registry import config_from_dict, load_config, plan_for_config, registered_architectures, resolve
from tiny_configs import CONFIG_A, CONFIG_B


def test_parses_dense_config():
    cfg = config_from_dict(CONFIG_A)
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (64, 4, 2, 16)
    assert cfg.tie_word_embeddings and cfg.sliding_window is None
    assert all(cfg.window_for_layer(i) is None for i in range(cfg.num_hidden_layers))


def test_head_dim_defaults_to_hidden_over_heads():
    raw = copy.deepcopy(CONFIG_A)
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 16


def test_sliding_window_and_max_window_layers():
    cfg = config_from_dict(CONFIG_B)
    assert cfg.sliding_window == 16 and cfg.max_window_layers == 1
    assert [cfg.window_for_layer(i) for i in range(3)] == [None, 16, 16]
    raw = copy.deepcopy(CONFIG_B)
    del raw["max_window_layers"]  # the reference's behaviour: every layer windowed
    assert [config_from_dict(raw).window_for_layer(i) for i in range(3)] == [16, 16, 16]


def test_disabled_window_is_ignored():
    raw = copy.deepcopy(CONFIG_B)
    raw["use_sliding_window"] = False
    cfg = config_from_dict(raw)
    assert cfg.sliding_window is None and cfg.window_for_layer(2) is None


def test_enabled_window_without_value_is_invalid():
    raw = copy.deepcopy(CONFIG_B)
    del raw["sliding_window"]
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert err.value.code == "invalid_request"
    raw["sliding_window"] = 0
    with pytest.raises(ConfigError):
        config_from_dict(raw)


@pytest.mark.parametrize("key,value", [("hidden_act", "gelu"), ("attention_bias", True), ("rope_scaling", {"type": "yarn"})])
def test_rejects_unsupported_options(key, value):
    raw = copy.deepcopy(CONFIG_A)
    raw[key] = value
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert err.value.code == "unsupported_capability"


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "max_position_embeddings", "vocab_size", "rms_norm_eps", "rope_theta"])
def test_missing_required_field_names_it(key):
    raw = copy.deepcopy(CONFIG_A)
    del raw[key]
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert err.value.code == "unsupported_capability" and key in str(err.value)


def test_unknown_architecture_lists_registered():
    raw = copy.deepcopy(CONFIG_A)
    raw["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError) as err:
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in str(err.value)
    with pytest.raises(ConfigError):
        config_from_dict({"model_type": "qwen3"})
    raw = copy.deepcopy(CONFIG_A)
    raw["model_type"] = "qwen3_moe"
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_round_trip_through_config_json(tmp_path):
    for raw in (CONFIG_A, CONFIG_B):
        cfg = config_from_dict(raw)
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        assert load_config(str(tmp_path)) == cfg


def test_reference_fixture_shape():
    # fixtures/qwen3-dense-sliding-window/config.json of the reference
    raw = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "attention_bias": False, "hidden_act": "silu",
           "hidden_size": 1024, "intermediate_size": 3072, "max_position_embeddings": 40960, "num_attention_heads": 16,
           "num_hidden_layers": 2, "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_scaling": None,
           "rope_theta": 1000000, "sliding_window": 2048, "tie_word_embeddings": True, "use_sliding_window": True,
           "vocab_size": 151936}
    cfg = config_from_dict(raw)
    assert cfg.sliding_window == 2048 and cfg.window_for_layer(0) == 2048


def test_plan_follows_config():
    plan = plan_for_config(config_from_dict(CONFIG_B))
    specs = plan.weight_specs()
    assert specs["model.layers.2.self_attn.q_proj.weight"].shape == (192, 96)
    assert specs["model.layers.0.self_attn.k_norm.weight"].shape == (32,)
    assert specs["lm_head.weight"].shape == (384, 96)
    assert len(specs) == 3 * 11 + 3
    assert [need.window for need in plan.cache_needs] == [None, 16, 16]
    tied = plan_for_config(config_from_dict(CONFIG_A)).weight_specs()
    assert "lm_head.weight" not in tied and len(tied) == 2 * 11 + 2
    assert "Qwen3ForCausalLM" in registered_architectures() and resolve("Qwen3ForCausalLM")[0] is Qwen3Config
