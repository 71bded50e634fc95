"""Safetensors reading, the loader's one clear error, and random-weights mode."""
import json

import numpy as np
import pytest
import torch

import helpers
from plain_llama import read_safetensors
from railgun_b200.config.llama import LlamaConfig
from railgun_b200.models.llama import llama_model_spec
from railgun_b200.parts.model import expected_tensors
from railgun_b200.weights.loader import TensorSpec, WeightError, load_weights
from railgun_b200.weights.random_init import write_random_model
from railgun_b200.weights.safetensors_io import SafetensorsError, open_model_files, write_safetensors


def test_round_trip_and_stored_precision(tmp_path):
    t = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6).reshape(2, 3),
         "d": torch.randn(4).to(torch.float16)}
    write_safetensors(tmp_path / "model.safetensors", t)
    spec = {k: TensorSpec(tuple(v.shape)) for k, v in t.items()}
    got = load_weights(tmp_path, spec)
    assert got["a"].dtype == torch.bfloat16 and torch.equal(got["a"], t["a"])
    assert got["b"].dtype == torch.float32 and torch.equal(got["b"], t["b"])       # 32-bit stays 32-bit
    assert got["c"].dtype == torch.int32 and torch.equal(got["c"].long(), t["c"])  # integer tables: int32
    assert got["d"].dtype == torch.bfloat16
    # the plain reader (own code) agrees with the writer
    plain = read_safetensors(tmp_path / "model.safetensors")
    assert np.array_equal(plain["a"], t["a"].double().numpy())


def test_compatible_with_the_safetensors_library(tmp_path):
    st = pytest.importorskip("safetensors.torch")
    t = {"x": torch.randn(4, 4).to(torch.bfloat16), "y": torch.randn(2)}
    write_safetensors(tmp_path / "ours.safetensors", t)
    back = st.load_file(str(tmp_path / "ours.safetensors"))
    assert torch.equal(back["x"], t["x"]) and torch.equal(back["y"], t["y"])
    (tmp_path / "lib").mkdir()
    st.save_file(t, str(tmp_path / "lib" / "model.safetensors"))
    entries = open_model_files(tmp_path / "lib")
    assert torch.equal(entries["x"].read(), t["x"])


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    cfg = LlamaConfig.from_dict(helpers.TINY_B)
    expected = expected_tensors(llama_model_spec(cfg))
    full = read_safetensors(helpers.model_dir("B") / "model.safetensors")
    tensors = {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in full.items()}
    del tensors["model.layers.1.mlp.up_proj.weight"]
    del tensors["lm_head.weight"]
    tensors["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(96)
    tensors["model.norm.weight"] = torch.ones(95)
    tensors["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(32, 97)
    write_safetensors(tmp_path / "model.safetensors", tensors)
    with pytest.raises(WeightError) as e:
        load_weights(tmp_path, expected)
    err = e.value
    assert sorted(err.missing) == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.0.self_attn.q_proj.bias"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.layers.2.self_attn.k_proj.weight", "model.norm.weight"]
    text = str(err)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [96] got [95]", "q_proj.bias"):
        assert word in text


def test_tied_model_tolerates_an_lm_head_in_the_file(tmp_path):
    from railgun_b200.config.registry import load_config
    full = read_safetensors(helpers.model_dir("A") / "model.safetensors")
    tensors = {k: torch.tensor(v, dtype=torch.float32).to(torch.bfloat16) for k, v in full.items()}
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    write_safetensors(tmp_path / "model.safetensors", tensors)
    (tmp_path / "config.json").write_text((helpers.model_dir("A") / "config.json").read_text())
    arch, cfg = load_config(tmp_path)
    got = load_weights(tmp_path, expected_tensors(arch.model_spec(cfg)), allow_unexpected=arch.allow_unexpected(cfg))
    assert "lm_head.weight" not in got


def test_broken_files(tmp_path):
    with pytest.raises(WeightError):
        load_weights(tmp_path, {})                                  # no file at all
    (tmp_path / "model.safetensors").write_bytes(b"\x10\x00\x00")
    with pytest.raises(SafetensorsError):
        open_model_files(tmp_path)
    write_safetensors(tmp_path / "model.safetensors", {"a": torch.zeros(100)})
    blob = (tmp_path / "model.safetensors").read_bytes()
    (tmp_path / "model.safetensors").write_bytes(blob[:-50])        # truncated data
    with pytest.raises(SafetensorsError) as e:
        open_model_files(tmp_path)
    assert "truncated" in str(e.value)
    write_safetensors(tmp_path / "model.safetensors", {"a": torch.zeros(4)})
    write_safetensors(tmp_path / "other.safetensors", {"a": torch.zeros(4)})
    with pytest.raises(SafetensorsError) as e:
        open_model_files(tmp_path)
    assert "both" in str(e.value)


def test_random_weights_mode_is_seeded(tmp_path):
    cfg = LlamaConfig.from_dict(helpers.TINY_A)
    write_random_model(cfg, 5, tmp_path / "a")
    write_random_model(cfg, 5, tmp_path / "b")
    write_random_model(cfg, 6, tmp_path / "c")
    a, b, c = (read_safetensors(tmp_path / x / "model.safetensors") for x in "abc")
    assert set(a) == set(expected_tensors(llama_model_spec(cfg)))
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert not np.array_equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert json.loads((tmp_path / "a" / "config.json").read_text())["architectures"] == ["LlamaForCausalLM"]
    w = a["model.layers.0.mlp.down_proj.weight"]
    assert abs(w.std() - 0.02) < 0.002 and abs(w.mean()) < 0.002
    n = a["model.norm.weight"]
    assert n.min() >= 0.9 - 1e-2 and n.max() <= 1.1 + 1e-2 and n.std() > 0.01
    assert "lm_head.weight" not in a                               # tied
