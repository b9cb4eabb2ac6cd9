"""Configuration and registry (no GPU)."""

import json

import pytest

from starter_b200.config import (ARCHITECTURES, ConfigError, Qwen3Config, config_from_dict, load_config)
from tiny import TINY, TINY_A, TINY_B, TINY_C


def test_reads_every_size_from_config_json():
    for raw in TINY.values():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, Qwen3Config)
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim", "rms_norm_eps",
                    "rope_theta", "tie_word_embeddings"):
            assert getattr(cfg, key) == raw[key], key


def test_head_dim_defaults_to_hidden_over_heads():
    raw = dict(TINY_A)
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == raw["hidden_size"] // raw["num_attention_heads"]


def test_rope_theta_may_sit_in_rope_parameters():
    raw = dict(TINY_A)
    theta = raw.pop("rope_theta")
    raw["rope_parameters"] = {"rope_theta": theta, "rope_type": "default"}
    assert config_from_dict(raw).rope_theta == theta


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta"])
def test_missing_key_is_named(key):
    raw = dict(TINY_B)
    del raw[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(raw)


@pytest.mark.parametrize("change", [
    {"attention_bias": True}, {"hidden_act": "gelu"}, {"rope_scaling": {"rope_type": "yarn", "factor": 4.0}},
    {"num_key_value_heads": 3}, {"head_dim": 15}, {"use_sliding_window": True, "sliding_window": None},
    {"rms_norm_eps": 0.0}, {"layer_types": ["sliding_attention", "full_attention"]},
])
def test_unsupported_values_are_errors_not_ignored(change):
    raw = dict(TINY_A)
    raw.update(change)
    with pytest.raises(ConfigError):
        config_from_dict(raw)


def test_unknown_architecture_lists_known_ones():
    raw = dict(TINY_A, architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(raw)
    assert "Qwen3ForCausalLM" in ARCHITECTURES


def test_model_spec_follows_the_config_layer_by_layer():
    cfg = config_from_dict(TINY_C)
    spec = cfg.to_model_spec()
    assert len(spec.layers) == 4 and [e.layer for e in spec.schedule] == [0, 1, 2, 3]
    assert [l.mixer.window for l in spec.layers] == [None, None, 8, 8]
    m = spec.layers[0].mixer
    assert (m.num_heads, m.num_kv_heads, m.head_dim) == (5, 5, 48)
    assert m.scale == pytest.approx(48 ** -0.5)
    assert m.position.theta == 5e6 and m.qk_norm_eps == 1e-6
    assert spec.layers[0].feed_forward.intermediate_size == 176
    assert spec.tie_embeddings and spec.vocab_size == 515
    b = config_from_dict(TINY_B).to_model_spec()
    assert not b.tie_embeddings and b.final_norm.eps == 1e-5


def test_round_trip_through_config_json(tmp_path):
    cfg = config_from_dict(TINY_C)
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(str(tmp_path)) == cfg
    with pytest.raises(ConfigError):
        load_config(str(tmp_path / "nothing"))
