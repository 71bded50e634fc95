"""The plain implementation against a second statement of the same formulas.

``tests/plain_llama.py`` (numpy, vectorised) is the oracle of every GPU test.
``tests/ref/llama_scalar.cpp`` states the decoder again, independently, as
scalar loops in C++; this test compiles it and compares whole-model logits of
the three tiny configurations (grouped and multi-query heads, a head size that
is not hidden / heads, llama3 frequency scaling in all its three branches, tied
and untied heads, three values of eps).  Both rest on the formulas, cited from
the reference in each file: the reference's own model code is Rust on the candle
crates and cannot be compiled where tests run, and model code of installed
packages is deliberately not used as a source.
"""
import shutil
import struct
import subprocess
from pathlib import Path

import numpy as np
import pytest

import helpers
import plain_llama as P

SRC = Path(__file__).resolve().parent / "ref" / "llama_scalar.cpp"


@pytest.fixture(scope="module")
def twin(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no C++ compiler")
    exe = tmp_path_factory.mktemp("twin") / "llama_scalar"
    subprocess.run([gxx, "-O2", "-std=c++17", str(SRC), "-o", str(exe)], check=True)
    return exe


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_numpy_and_scalar_statements_agree(name, twin, tmp_path):
    cfg = helpers.TINY[name][0]
    mdir = helpers.model_dir(name)
    plain = P.PlainLlama(mdir)
    ids = helpers.prompts(cfg["vocab_size"], [37], seed=40)[0]
    w = plain.w
    sc = cfg.get("rope_scaling") or {}
    header = struct.pack("<9i", plain.L, plain.H, plain.nh, plain.nkv, plain.d, cfg["intermediate_size"],
                         cfg["vocab_size"], len(ids), 1 if sc else 0)
    header += struct.pack("<6d", plain.eps, cfg["rope_theta"], sc.get("factor", 1.0), sc.get("low_freq_factor", 1.0),
                          sc.get("high_freq_factor", 1.0), sc.get("original_max_position_embeddings", 1))
    parts = [w["model.embed_tokens.weight"]]
    for i in range(plain.L):
        p = f"model.layers.{i}."
        parts += [w[p + n] for n in ("input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.weight",
                                     "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                     "post_attention_layernorm.weight", "mlp.gate_proj.weight", "mlp.up_proj.weight",
                                     "mlp.down_proj.weight")]
    parts += [w["model.norm.weight"], w["model.embed_tokens.weight"] if plain.tied else w["lm_head.weight"]]
    with open(tmp_path / "in.bin", "wb") as f:
        f.write(header)
        f.write(np.asarray(ids, dtype="<i4").tobytes())
        for t in parts:
            f.write(np.ascontiguousarray(t, dtype="<f8").tobytes())
    subprocess.run([str(twin), str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], check=True, timeout=300)
    got = np.fromfile(tmp_path / "out.bin", dtype="<f8").reshape(len(ids), cfg["vocab_size"])
    want = plain.forward(ids)
    assert np.abs(got - want).max() < 1e-9 * np.abs(want).max()
    if sc:                       # the test means something only if the scaling rule's three branches all occur
        inv = P.rope_inv_freq(plain.d, cfg["rope_theta"], None)
        wavelen = 2 * np.pi / inv
        lo, hi = sc["original_max_position_embeddings"] / sc["high_freq_factor"], sc["original_max_position_embeddings"] / sc["low_freq_factor"]
        assert (wavelen < lo).any() and (wavelen > hi).any() and ((wavelen >= lo) & (wavelen <= hi)).any()
