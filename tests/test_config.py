"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import tiny_models as tm
from litellmengine_b200.config import (ConfigError, ModelPlan, NormSpec, Qwen3Config, StageSpec,
                                       config_from_dict, load_config, register_architecture,
                                       registered_architectures, save_config, unregister_architecture)


def test_every_size_comes_from_config_json():
    for cfg in (tm.TINY_A, tm.TINY_B, tm.TINY_C):
        c = config_from_dict(cfg)
        assert isinstance(c, Qwen3Config)
        p = c.plan()
        assert p.hidden_size == cfg["hidden_size"] and p.vocab_size == cfg["vocab_size"]
        assert len(p.blocks) == len(p.order) == cfg["num_hidden_layers"]
        m = p.blocks[0].mixer
        assert (m.num_heads, m.num_kv_heads, m.head_dim) == (cfg["num_attention_heads"],
                                                             cfg["num_key_value_heads"], cfg["head_dim"])
        assert m.position.theta == cfg["rope_theta"] and m.qk_norm.eps == cfg["rms_norm_eps"]
        assert p.blocks[0].feed_forward.intermediate_size == cfg["intermediate_size"]
        assert p.tie_word_embeddings == cfg["tie_word_embeddings"] and p.max_position == cfg["max_position_embeddings"]


def test_defaults_follow_the_reference():
    d = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=10, hidden_size=32,
             intermediate_size=8, num_hidden_layers=1, num_attention_heads=2)
    c = config_from_dict(d)
    assert (c.num_key_value_heads, c.head_dim, c.max_position_embeddings) == (2, 16, 32768)
    assert c.rms_norm_eps == 1e-6 and c.rope_theta == 10000.0 and c.tie_word_embeddings is False


@pytest.mark.parametrize("key", ["model_type", "vocab_size", "hidden_size", "intermediate_size",
                                 "num_hidden_layers", "num_attention_heads"])
def test_missing_required_key(key):
    d = copy.deepcopy(tm.TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=f"Missing required config field: {key}"):
        config_from_dict(d)


@pytest.mark.parametrize("patch,msg", [
    ({"num_key_value_heads": 3}, "divisible"), ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
    ({"rope_theta": -1.0}, "rope_theta"), ({"vocab_size": 0}, "vocab_size"), ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"), ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn"}}, "rope_scaling"), ({"use_sliding_window": True}, "sliding"),
    ({"vocab_size": "many"}, "integer")])
def test_bad_values_are_refused(patch, msg):
    d = copy.deepcopy(tm.TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=msg):
        config_from_dict(d)


def test_unknown_architecture_lists_registered():
    d = copy.deepcopy(tm.TINY_A)
    d["architectures"] = ["NopeForCausalLM"]
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict(d)
    del d["architectures"]
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict(d)


def test_round_trip_through_a_folder(tmp_path):
    c = config_from_dict(tm.TINY_B)
    save_config(c, str(tmp_path))
    assert load_config(str(tmp_path)) == c
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        load_config(str(tmp_path))
    with pytest.raises(ConfigError, match="Failed to open"):
        load_config(str(tmp_path / "absent"))


def test_registering_another_architecture():
    @register_architecture("ToyForCausalLM")
    class ToyConfig:
        def __init__(self, d):
            self.d = d

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return self.d

        def plan(self):
            return config_from_dict(tm.TINY_A).plan()
    try:
        assert "ToyForCausalLM" in registered_architectures()
        assert isinstance(config_from_dict({"architectures": ["ToyForCausalLM"]}), ToyConfig)
    finally:
        unregister_architecture("ToyForCausalLM")


def test_plan_order_is_checked():
    p = config_from_dict(tm.TINY_A).plan()
    bad = ModelPlan(**{**p.__dict__, "order": (StageSpec(0), StageSpec(5))})
    with pytest.raises(ValueError, match="names layer 5"):
        bad.validate()
    bad = ModelPlan(**{**p.__dict__, "order": (StageSpec(0), StageSpec(1, cache_from=1))})
    with pytest.raises(ValueError, match="earlier stage"):
        bad.validate()
    ok = ModelPlan(**{**p.__dict__, "order": (StageSpec(0), StageSpec(1), StageSpec(0), StageSpec(1, cache_from=1))})
    ok.validate()
