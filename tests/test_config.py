"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

from smolmoe_c99_b200.config import ConfigError, Qwen2Config, config_from_json, load_config, register_architecture
from tiny import TINY


@pytest.mark.parametrize("name", list(TINY))
def test_round_trip(name):
    cfg = config_from_json(TINY[name])
    assert isinstance(cfg, Qwen2Config)
    assert config_from_json(cfg.to_json()) == cfg
    spec = cfg.model_spec()
    assert len(spec.layers) == TINY[name]["num_hidden_layers"] and spec.order == tuple(range(len(spec.layers)))
    assert spec.vocab_size == TINY[name]["vocab_size"]
    assert (spec.head_name is None) == TINY[name]["tie_word_embeddings"]


def test_every_size_comes_from_the_file():
    a, b = config_from_json(TINY["A"]), config_from_json(TINY["B"])
    for field in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads",
                  "head_dim", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta", "tie_word_embeddings",
                  "use_sliding_window"):
        assert getattr(a, field) != getattr(b, field), field
    ma, mb = a.model_spec().layers[0].mixer, b.model_spec().layers[0].mixer
    assert abs(ma["scale"] - 16 ** -0.5) < 1e-12 and abs(mb["scale"] - 32 ** -0.5) < 1e-12
    assert ma["position"]["theta"] == 10000.0 and mb["position"]["theta"] == 1e6


def test_head_dim_default_and_override():
    assert config_from_json(TINY["A"]).head_dim == 16            # hidden / heads
    assert config_from_json(TINY["C"]).head_dim == 48            # given, and not hidden / heads (80 / 5)
    raw = dict(TINY["C"]); raw.pop("head_dim")
    assert config_from_json(raw).head_dim == 16


def test_window_layers():
    b = config_from_json(TINY["B"])
    assert [b.layer_window(i) for i in range(3)] == [None, 40, 40]
    assert [l.mixer["window"] for l in b.model_spec().layers] == [None, 40, 40]
    a = config_from_json(TINY["A"])
    assert all(a.layer_window(i) is None for i in range(2))
    raw = dict(TINY["B"]); raw.pop("sliding_window")
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_json(raw)


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "num_key_value_heads", "vocab_size", "max_position_embeddings", "rms_norm_eps",
                                 "rope_theta", "hidden_act", "tie_word_embeddings"])
def test_missing_key_is_named(key):
    raw = dict(TINY["A"]); raw.pop(key)
    with pytest.raises(ConfigError, match=key):
        config_from_json(raw)


def test_all_missing_keys_are_listed_at_once():
    raw = dict(TINY["A"]); raw.pop("rope_theta"); raw.pop("vocab_size")
    with pytest.raises(ConfigError) as e:
        config_from_json(raw)
    assert "rope_theta" in str(e.value) and "vocab_size" in str(e.value)


@pytest.mark.parametrize("change,word", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"rope_scaling": {"type": "linear", "factor": 2}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "num_key_value_heads"), ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"rms_norm_eps": 1.5}, "rms_norm_eps"), ({"rope_theta": 1.0}, "rope_theta"), ({"hidden_size": -4}, "hidden_size"),
    ({"vocab_size": 2.5}, "vocab_size"), ({"head_dim": 15}, "head_dim"), ({"model_type": "llama"}, "model_type"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"), ({"eos_token_id": 999}, "eos_token_id"),
    ({"hidden_size": 66}, "head_dim"),
])
def test_bad_values_name_the_key(change, word):
    raw = dict(TINY["A"]); raw.update(change)
    with pytest.raises(ConfigError, match=word):
        config_from_json(raw)


def test_registry():
    with pytest.raises(ConfigError, match="unsupported architecture: LlamaForCausalLM"):
        config_from_json(dict(TINY["A"], architectures=["LlamaForCausalLM"]))
    with pytest.raises(ConfigError, match="architectures"):
        config_from_json({k: v for k, v in TINY["A"].items() if k != "architectures"})

    class Other(Qwen2Config):
        pass
    register_architecture("OtherForCausalLM", Other)
    assert isinstance(config_from_json(dict(TINY["A"], architectures=["OtherForCausalLM"])), Other)


def test_load_config_from_folder(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY["B"]))
    assert load_config(str(tmp_path)) == config_from_json(TINY["B"])
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="no such file"):
        load_config(str(tmp_path / "absent"))


def test_model_spec_checks_order_and_cache_sharing():
    from dataclasses import replace
    spec = config_from_json(TINY["A"]).model_spec()
    with pytest.raises(ValueError, match="layer order"):
        replace(spec, order=(0, 5))
    shared = replace(spec.layers[1], cache_from=1)
    with pytest.raises(ValueError, match="not another layer"):
        replace(spec, layers=(spec.layers[0], shared))
    replace(spec, order=(0, 1, 1, 0))   # a layer may be named twice
