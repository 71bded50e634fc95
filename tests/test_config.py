"""Typed configuration and the architecture registry
(pattern of crates/vllm-models/src/config.rs:117-136 and registry.rs:188-220)."""
import json

import pytest

import helpers
from railgun_b200.config.base import ConfigError
from railgun_b200.config.llama import LlamaConfig
from railgun_b200.config.registry import Architecture, architecture_of, known_architectures, load_config, \
    register_architecture


def test_llama_1b_like_json():
    cfg = LlamaConfig.from_dict({
        "architectures": ["LlamaForCausalLM"], "hidden_size": 2048, "num_attention_heads": 32,
        "num_key_value_heads": 8, "num_hidden_layers": 16, "intermediate_size": 8192, "vocab_size": 128256,
        "rope_theta": 500000.0, "tie_word_embeddings": True, "eos_token_id": [128001, 128008],
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
        "some_unknown_key": 7})
    assert cfg.head_dim == 64 and cfg.num_key_value_heads == 8
    assert cfg.rope_scaling.factor == 32.0 and cfg.tie_word_embeddings
    assert cfg.eos_token_id == (128001, 128008)


def test_defaults_follow_the_reference():
    cfg = LlamaConfig.from_dict(dict(hidden_size=64, num_attention_heads=4, num_hidden_layers=1,
                                     intermediate_size=128, vocab_size=100))
    assert cfg.num_key_value_heads == 4                 # defaults to the number of heads
    assert cfg.max_position_embeddings == 4096 and cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-5
    assert cfg.rope_scaling is None and cfg.tie_word_embeddings is False
    assert cfg.eos_token_id == ()


def test_head_dim_key_wins_over_quotient():
    cfg = LlamaConfig.from_dict(dict(hidden_size=96, num_attention_heads=3, num_hidden_layers=1,
                                     intermediate_size=128, vocab_size=100, head_dim=48))
    assert cfg.head_dim == 48


@pytest.mark.parametrize("patch, word", [
    ({"hidden_size": None}, "hidden_size"),
    ({"vocab_size": "many"}, "vocab_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "low_freq_factor"),
    ({"rms_norm_eps": -1.0}, "rms_norm_eps"),
    ({"tie_word_embeddings": "yes"}, "tie_word_embeddings"),
    ({"head_dim": 15}, "even"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
])
def test_bad_configs_are_refused(patch, word):
    data = dict(helpers.TINY_A)
    data.update(patch)
    with pytest.raises(ConfigError) as e:
        LlamaConfig.from_dict(data)
    assert word in str(e.value)


def test_round_trip_through_config_json(tmp_path):
    for name in ("A", "B", "C"):
        cfg = LlamaConfig.from_dict(helpers.TINY[name][0])
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        arch, back = load_config(tmp_path)
        assert arch.name == "LlamaForCausalLM"
        assert back.to_dict() == cfg.to_dict()


def test_registry_chooses_by_config_json(tmp_path):
    assert "LlamaForCausalLM" in known_architectures()
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["NoSuchModel"]}))
    with pytest.raises(ConfigError) as e:
        load_config(tmp_path)
    assert "unknown architecture: NoSuchModel" in str(e.value) and "LlamaForCausalLM" in str(e.value)
    (tmp_path / "config.json").write_text(json.dumps({"hidden_size": 4}))
    with pytest.raises(ConfigError):
        load_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        load_config(tmp_path)


def test_registering_another_architecture(tmp_path):
    arch = Architecture("ToyForCausalLM", lambda d, where="": dict(d), lambda cfg: None)
    register_architecture(arch, replace=True)
    with pytest.raises(ValueError):
        register_architecture(arch)
    assert architecture_of("ToyForCausalLM") is arch
    (tmp_path / "config.json").write_text(json.dumps({"architectures": ["ToyForCausalLM"], "x": 1}))
    got, cfg = load_config(tmp_path)
    assert got is arch and cfg["x"] == 1


def test_spec_holds_only_config_numbers():
    """Every size in the model description comes from the configuration."""
    from railgun_b200.models.llama import llama_model_spec
    for name in ("A", "B", "C"):
        raw = helpers.TINY[name][0]
        spec = llama_model_spec(LlamaConfig.from_dict(raw))
        assert len(spec.layers) == raw["num_hidden_layers"]
        m = spec.layers[0].mixer.params
        assert (m["num_heads"], m["num_kv_heads"], m["head_dim"]) == (
            raw["num_attention_heads"], raw["num_key_value_heads"], raw["head_dim"])
        assert spec.layers[0].ffn.params["intermediate_size"] == raw["intermediate_size"]
        assert spec.layers[0].mixer_norm.params["eps"] == raw["rms_norm_eps"]
        assert m["position"].params["theta"] == raw["rope_theta"]
        tied = raw["tie_word_embeddings"]
        assert (spec.head.params["name"] == spec.embedding.params["name"]) == tied
