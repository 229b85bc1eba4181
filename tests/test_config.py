"""Configuration and registry (no GPU)."""
import copy
import os

import pytest

import helpers
from vt_transformer_b200.config import (ConfigError, Qwen2Config, config_from_dict, get_architecture,
                                        known_architectures, load_config, register_architecture,
                                        unregister_architecture)
from vt_transformer_b200.config.base import ModelConfig


def test_reads_every_size_from_the_keys():
    for name, d in helpers.CONFIGS.items():
        cfg = config_from_dict(d)
        assert isinstance(cfg, Qwen2Config)
        assert cfg.vocab_size == d["vocab_size"] and cfg.hidden_size == d["hidden_size"]
        assert cfg.intermediate_size == d["intermediate_size"] and cfg.num_hidden_layers == d["num_hidden_layers"]
        assert cfg.rms_norm_eps == d["rms_norm_eps"] and cfg.rope_theta == d["rope_theta"]
        assert cfg.head_dim == d.get("head_dim", d["hidden_size"] // d["num_attention_heads"])
        assert cfg.q_dim == cfg.num_attention_heads * cfg.head_dim
        assert cfg.kv_dim == cfg.num_key_value_heads * cfg.head_dim


def test_defaults_of_optional_keys():
    d = copy.deepcopy(helpers.CONFIGS["A"])
    del d["num_key_value_heads"], d["tie_word_embeddings"]
    cfg = config_from_dict(d)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.tie_word_embeddings is False and cfg.use_sliding_window is False
    assert all(cfg.layer_window(i) is None for i in range(cfg.num_hidden_layers))


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings"])
def test_missing_key_is_named(key):
    d = copy.deepcopy(helpers.CONFIGS["B"])
    del d[key]
    with pytest.raises(ConfigError, match=key):
        config_from_dict(d)


def test_wrong_types_are_named():
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d["hidden_size"] = "64"
    with pytest.raises(ConfigError, match="hidden_size"):
        config_from_dict(d)
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d["tie_word_embeddings"] = 1
    with pytest.raises(ConfigError, match="tie_word_embeddings"):
        config_from_dict(d)


def test_unknown_architecture_lists_the_known():
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d["architectures"] = ["NoSuchModel"]
    with pytest.raises(ConfigError, match="Qwen2ForCausalLM"):
        config_from_dict(d)
    del d["architectures"]
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(d)


def test_sizes_the_kernels_do_not_take_are_refused():
    for key, value, word in (("head_dim", 24, "head_dim"), ("head_dim", 272, "head_dim"),
                             ("hidden_size", 68, "hidden_size"), ("intermediate_size", 172, "intermediate_size"),
                             ("num_key_value_heads", 3, "num_key_value_heads"), ("hidden_act", "gelu", "hidden_act")):
        d = copy.deepcopy(helpers.CONFIGS["A"])
        d[key] = value
        if key == "hidden_size":
            d["head_dim"] = 16
        with pytest.raises(ConfigError, match=word):
            config_from_dict(d)


def test_rotation_scaling_is_refused_and_rope_parameters_are_read():
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d["rope_scaling"] = {"type": "yarn", "factor": 4.0}
    with pytest.raises(ConfigError, match="rope_scaling"):
        config_from_dict(d)
    d = copy.deepcopy(helpers.CONFIGS["A"])
    theta = d.pop("rope_theta")
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": theta}
    assert config_from_dict(d).rope_theta == theta


def test_window_by_layer():
    cfg = config_from_dict(helpers.CONFIGS["C"])
    assert [cfg.layer_window(i) for i in range(4)] == [None, None, 20, 20]
    d = copy.deepcopy(helpers.CONFIGS["C"])
    d["layer_types"] = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    cfg = config_from_dict(d)
    assert [cfg.layer_window(i) for i in range(4)] == [20, None, None, 20]
    d["use_sliding_window"] = False                      # switched off: layer_types gives no layer a window
    assert [config_from_dict(d).layer_window(i) for i in range(4)] == [None] * 4
    d["use_sliding_window"] = True
    d["layer_types"] = ["full_attention"]
    with pytest.raises(ConfigError, match="layer_types"):
        config_from_dict(d)
    d = copy.deepcopy(helpers.CONFIGS["C"])
    del d["sliding_window"]
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(d)
    # a 7B-style file: a window is given but switched off
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d.update(sliding_window=131072, use_sliding_window=False, max_window_layers=28)
    cfg = config_from_dict(d)
    assert all(cfg.layer_window(i) is None for i in range(cfg.num_hidden_layers))


def test_round_trip_through_a_folder(tmp_path):
    for name in helpers.CONFIGS:
        cfg = helpers.make_config(name)
        cfg.save(str(tmp_path / name))
        assert load_config(str(tmp_path / name)) == cfg
    with pytest.raises(ConfigError, match="config.json"):
        load_config(str(tmp_path / "nothing_here"))
    os.makedirs(tmp_path / "bad")
    (tmp_path / "bad" / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="JSON"):
        load_config(str(tmp_path / "bad"))


def test_eos_ids():
    d = copy.deepcopy(helpers.CONFIGS["A"])
    d["eos_token_id"] = [7, 9]
    assert config_from_dict(d).eos_token_id == (7, 9)
    d["eos_token_id"] = 5
    cfg = config_from_dict(d)
    assert cfg.eos_token_id == (5,) and config_from_dict(cfg.to_dict()) == cfg


def test_registry_takes_another_architecture():
    from dataclasses import dataclass

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        width: int = 8

        @classmethod
        def from_dict(cls, data, where="config.json"):
            return cls(architecture=data["architectures"][0], width=data["width"])

    register_architecture("ToyForTests", ToyConfig, lambda cfg: None)
    try:
        assert "ToyForTests" in known_architectures()
        cfg = config_from_dict({"architectures": ["ToyForTests"], "width": 24})
        assert isinstance(cfg, ToyConfig) and cfg.width == 24
        with pytest.raises(ValueError, match="registered already"):
            register_architecture("ToyForTests", ToyConfig, lambda cfg: None)
        assert get_architecture("ToyForTests").config_class is ToyConfig
    finally:
        unregister_architecture("ToyForTests")
    assert "ToyForTests" not in known_architectures()
