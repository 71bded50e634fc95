"""Parts that are not in the framework, defined here and registered from
outside: a mixer with state of its own (a decaying running sum kept in the
request's state slot), a feed-forward of another shape, and an architecture
made of them beside the built-in attention.  Nothing in the framework's files
changes; the model is built, stepped in several cuts and compared with a plain
statement of the same toy."""
import json

import numpy as np
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu

DECAY = 0.9


def register_toys():
    from railgun_b200 import ops
    from railgun_b200.cache.manager import StateNeed
    from railgun_b200.config.registry import Architecture, register_architecture
    from railgun_b200.parts import (FeedForward, LayerSpec, Mixer, ModelSpec, PartSpec, register_feed_forward,
                                    register_mixer)
    from railgun_b200.weights.loader import TensorSpec

    class DecayingSum(Mixer):
        """state_t = DECAY * state_{t-1} + x_t ; y_t = W state_t.  The state of
        each request lives in its slot between steps."""

        @classmethod
        def tensor_specs(cls, p, prefix):
            return {prefix + "toy.mix.weight": TensorSpec((p["hidden_size"], p["hidden_size"]))}

        @classmethod
        def cache_need(cls, p):
            return StateNeed((p["hidden_size"],), "float32")

        def __init__(self, p, prefix, env, tensors):
            super().__init__(p, prefix, env, tensors)
            self.w = tensors.get(prefix + "toy.mix.weight", env.dtype)

        def forward(self, x, batch, cache, writes=True):
            out = torch.empty_like(x, dtype=torch.float32)
            cu, starts, slots = batch.host_cu_seqlens, batch.host_start_pos, batch.host_state_slots
            for i in range(batch.num_requests):
                lo, hi = int(cu[i]), int(cu[i + 1])
                s = cache.state[int(slots[i])]
                if starts[i] == 0:
                    s.zero_()                       # a new (or recomputed) request starts from nothing
                for t in range(lo, hi):
                    s.mul_(DECAY).add_(x[t].float())
                    out[t] = s
            return ops.linear(out.to(x.dtype), self.w)

    class ReluMLP(FeedForward):
        @classmethod
        def tensor_specs(cls, p, prefix):
            return {prefix + "toy.up.weight": TensorSpec((p["inner"], p["hidden_size"])),
                    prefix + "toy.down.weight": TensorSpec((p["hidden_size"], p["inner"]))}

        def __init__(self, p, prefix, env, tensors):
            super().__init__(p, prefix, env, tensors)
            self.up = tensors.get(prefix + "toy.up.weight", env.dtype)
            self.down = tensors.get(prefix + "toy.down.weight", env.dtype)

        def forward(self, x, batch):
            return ops.linear(torch.relu(ops.linear(x, self.up)), self.down)

    register_mixer("toy_decaying_sum", DecayingSum, replace=True)
    register_feed_forward("toy_relu_mlp", ReluMLP, replace=True)

    def config_from_dict(d, where=""):
        from types import SimpleNamespace
        c = SimpleNamespace(**d)
        c.architecture = d["architectures"][0]
        c.to_dict = lambda: dict(d)
        return c

    def model_spec(c):
        H = c.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=c.eps, name=name))
        attn = PartSpec("paged_attention", dict(
            hidden_size=H, num_heads=c.heads, num_kv_heads=c.kv_heads, head_dim=c.head_dim, window=0, scale=None,
            position=PartSpec("rope", dict(head_dim=c.head_dim, theta=1000.0, scaling=None, max_position=c.max_pos))))
        toy = PartSpec("toy_decaying_sum", dict(hidden_size=H))
        swiglu = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.inner))
        relu = PartSpec("toy_relu_mlp", dict(hidden_size=H, inner=c.inner))
        layers = []
        for i, kind in enumerate(c.layer_kinds):             # mixers and feed-forwards differ layer by layer
            layers.append(LayerSpec(prefix=f"model.layers.{i}.", mixer=toy if kind == "toy" else attn,
                                    mixer_norm=norm("input_layernorm.weight"),
                                    ffn=relu if kind == "toy" else swiglu,
                                    ffn_norm=norm("post_attention_layernorm.weight")))
        return ModelSpec(hidden_size=H, vocab_size=c.vocab, max_position=c.max_pos,
                         embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=H, name="emb")),
                         layers=tuple(layers), final_norm=norm("model.norm.weight"),
                         head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=H, name="emb")))

    register_architecture(Architecture("ToyMixedForCausalLM", config_from_dict, model_spec), replace=True)


TOY_CFG = dict(architectures=["ToyMixedForCausalLM"], hidden_size=40, heads=2, kv_heads=1, head_dim=16, inner=72,
               vocab=90, eps=1e-5, max_pos=128, layer_kinds=["attn", "toy", "toy", "attn"])


def plain_toy_forward(model_dir, ids):
    cfg = json.loads((model_dir / "config.json").read_text())
    w = P.read_safetensors(model_dir / "model.safetensors")
    H, nh, nkv, d = cfg["hidden_size"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    T = len(ids)
    pos = np.arange(T)
    inv = P.rope_inv_freq(d, 1000.0, None)
    x = P.embedding(w["emb"], ids)
    for i, kind in enumerate(cfg["layer_kinds"]):
        p = f"model.layers.{i}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if kind == "toy":
            s, outs = np.zeros(H), []
            for t in range(T):
                s = DECAY * s + h[t]
                outs.append(s.copy())
            x = x + P.linear(np.stack(outs), w[p + "toy.mix.weight"])
            h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
            x = x + P.linear(np.maximum(P.linear(h, w[p + "toy.up.weight"]), 0), w[p + "toy.down.weight"])
        else:
            q = P.rope(P.linear(h, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, d), pos, inv)
            k = P.rope(P.linear(h, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, d), pos, inv)
            v = P.linear(h, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
            x = x + P.linear(P.attention(q, k, v, pos).reshape(T, nh * d), w[p + "self_attn.o_proj.weight"])
            h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
            x = x + P.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["emb"])


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_toy_architecture_with_a_stateful_mixer(mode, dtype, tol, tmp_path):
    from railgun_b200.config.registry import load_config
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    from railgun_b200.weights.random_init import write_random_model
    register_toys()
    mdir = tmp_path / "toy"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(TOY_CFG))
    arch, cfg = load_config(mdir)                             # chosen by config.json, as everywhere
    write_random_model(cfg, 3, mdir, std=0.15)
    (mdir / "config.json").write_text(json.dumps(TOY_CFG))
    reqs = {f"t{i}": p for i, p in enumerate(helpers.prompts(TOY_CFG["vocab"], [30, 9, 55, 41, 17], seed=8))}
    steps = {"whole": helpers.trace_whole, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, max_live=3, seed=2)}[mode](reqs)
    runner = ModelRunner(mdir, dtype=dtype, page_size=8, max_tokens=helpers.peak_tokens(steps, 64),
                         max_requests=3)
    assert len(runner.cache.state) == 2 and len(runner.cache.kv) == 2      # two stateful layers, two paged ones
    rp = Replayer(runner, tmp_path / "out")
    for s in steps:
        rp.feed(s)
    rows = helpers.collect(steps, tmp_path / "out", TOY_CFG["vocab"])
    for name, toks in reqs.items():
        ref = plain_toy_forward(mdir, toks)
        for p in range(len(toks)):
            assert np.abs(rows[(name, p)] - ref[p]).max() / np.abs(ref).max() < tol, (name, p)
    runner.alloc.check()


def test_unknown_part_kind_is_a_clear_error():
    from railgun_b200.parts.registry import MIXERS
    with pytest.raises(KeyError) as e:
        MIXERS.get("no_such_mixer")
    assert "paged_attention" in str(e.value)
