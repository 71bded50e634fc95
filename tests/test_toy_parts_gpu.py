"""Parts that are not in the framework, defined here and registered from
outside: a mixer with state of its own (a decaying running sum kept in the
request's state slot), once planned on the host and once written with device
operations only so that its steps replay from CUDA graphs, a layer with three
branches and three norms, a feed-forward of another shape, a feed-forward that
routes every token to one of several experts, a position encoding that is no
rotation, and architectures made of them beside the built-in attention.
Nothing in the framework's files changes; the models are built, stepped in
several cuts and compared with a plain statement of the same toys."""
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
    from railgun_b200.parts import (FeedForward, LayerSpec, Mixer, ModelSpec, PartSpec, SubLayer,
                                    register_feed_forward, register_mixer)
    from railgun_b200.weights.loader import TensorSpec

    class DecayingSum(Mixer):
        """state_t = DECAY * state_{t-1} + x_t ; y_t = W state_t.  The state of
        each request lives in its slot between steps.  This one walks the
        requests on the host, so it says that its steps cannot be captured."""
        graph_safe = False

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

    class DecayingSumOnDevice(DecayingSum):
        """The same mixer from the step's device-side description alone (token offsets, start positions and
        state slots as tensors; the longest portion as a number that the step's layout fixes): nothing is read
        back, so the model's steps can be captured and replayed.  Rows without a request (slot -1, the padding
        of a static decode batch) touch no state."""
        graph_safe = True

        def forward(self, x, batch, cache, writes=True):
            state = cache.state                                            # [slots, H] float32
            cu = batch.cu_seqlens.long()
            first, counts = cu[:-1], cu[1:] - cu[:-1]
            slots = batch.state_slots.long()
            live = slots >= 0
            slot = slots.clamp(min=0)
            fresh = (batch.start_pos == 0) & live
            out = torch.zeros_like(x, dtype=torch.float32)
            xf = x.float()
            last_row = x.shape[0] - 1
            for j in range(batch.max_query_len):
                on = live & (counts > j)
                row = (first + j).clamp(max=last_row)
                old = state[slot]
                base = torch.where(fresh[:, None], torch.zeros_like(old), old) if j == 0 else old
                new = DECAY * base + xf[row]
                # every live slot gets exactly one change, rows that are off add zero: duplicates cannot collide
                state.index_add_(0, slot, torch.where(on[:, None], new - old, torch.zeros_like(old)))
                out.index_add_(0, row, torch.where(on[:, None], new, torch.zeros_like(new)))
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
    register_mixer("toy_decaying_sum_on_device", DecayingSumOnDevice, replace=True)
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
        toy = PartSpec(getattr(c, "toy_mixer", "toy_decaying_sum"), dict(hidden_size=H))
        swiglu = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.inner))
        relu = PartSpec("toy_relu_mlp", dict(hidden_size=H, inner=c.inner))
        layers = []
        for i, kind in enumerate(c.layer_kinds):             # mixers and feed-forwards differ layer by layer
            if kind == "three":
                # a block of three branches, each behind a norm of its own: attention, then two feed-forwards
                layers.append(LayerSpec(prefix=f"model.layers.{i}.", sublayers=(
                    SubLayer(norm("input_layernorm.weight"), attn, "mixer"),
                    SubLayer(norm("post_attention_layernorm.weight"), relu, "ffn"),
                    SubLayer(norm("third_layernorm.weight"), swiglu, "ffn"))))
                continue
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
            if kind == "three":
                x = x + P.linear(np.maximum(P.linear(h, w[p + "toy.up.weight"]), 0), w[p + "toy.down.weight"])
                h = P.rms_norm(x, w[p + "third_layernorm.weight"], cfg["eps"])
            x = x + P.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["emb"])


def test_stateful_layers_and_three_branch_layers_replay_from_graphs(tmp_path):
    """The stateful mixer written with device operations only, beside attention layers and a layer of three
    branches with three norms: steps of single tokens replay CUDA graphs (static batches with padding rows),
    large repeated steps replay graphs captured for their layout, and every logit matches the plain statement."""
    from railgun_b200.config.registry import load_config
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    from railgun_b200.weights.random_init import write_random_model
    register_toys()
    cfg_dict = dict(TOY_CFG, toy_mixer="toy_decaying_sum_on_device", layer_kinds=["attn", "toy", "three", "toy"])
    mdir = tmp_path / "toy"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg_dict))
    arch, cfg = load_config(mdir)
    write_random_model(cfg, 3, mdir, std=0.15)
    (mdir / "config.json").write_text(json.dumps(cfg_dict))
    reqs = {f"t{i}": p for i, p in enumerate(helpers.prompts(TOY_CFG["vocab"], [30, 9, 55, 41, 17], seed=8))}
    for mode, make in (("tail", lambda r: helpers.trace_tail_decode(r, 12)),
                       ("mixed", lambda r: helpers.trace_mixed(r, max_live=3, seed=2))):
        steps = make(reqs)
        runner = ModelRunner(mdir, dtype="float32", page_size=8, max_tokens=helpers.peak_tokens(steps, 64),
                             max_requests=3)
        assert runner.use_graphs and len(runner.cache.state) == 2
        runner.shape_graph_min_tokens = 2
        rp = Replayer(runner, tmp_path / mode)
        for s in steps:
            rp.feed(s)
        assert runner._static, "no step of single tokens replayed a graph"
        rows = helpers.collect(steps, tmp_path / mode, TOY_CFG["vocab"])
        for name, toks in reqs.items():
            ref = plain_toy_forward(mdir, toks)
            for p in range(len(toks)):
                assert np.abs(rows[(name, p)] - ref[p]).max() / np.abs(ref).max() < 2e-5, (mode, name, p)
        runner.alloc.check()


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
    assert not runner.use_graphs                            # the mixer said that it plans on the host
    rp = Replayer(runner, tmp_path / "out")
    for s in steps:
        rp.feed(s)
    rows = helpers.collect(steps, tmp_path / "out", TOY_CFG["vocab"])
    for name, toks in reqs.items():
        ref = plain_toy_forward(mdir, toks)
        for p in range(len(toks)):
            assert np.abs(rows[(name, p)] - ref[p]).max() / np.abs(ref).max() < tol, (name, p)
    runner.alloc.check()


def register_routed_toys():
    """A feed-forward with a router (the expert with the largest 32-bit router logit takes the token,
    its output weighted by the softmax probability) and a position encoding that scales the
    coordinates of q and k by 1 + sin(position * (i + 1) / 7) / 2 instead of rotating them."""
    from railgun_b200 import ops
    from railgun_b200.config.registry import Architecture, register_architecture
    from railgun_b200.parts import (FeedForward, LayerSpec, ModelSpec, PartSpec, PositionEncoding,
                                    register_feed_forward, register_position_encoding)
    from railgun_b200.weights.loader import TensorSpec
    register_toys()

    class RoutedReluMLP(FeedForward):
        graph_safe = False                                  # how many kernels run depends on the routing: no graphs

        @classmethod
        def tensor_specs(cls, p, prefix):
            E, H, I = p["experts"], p["hidden_size"], p["inner"]
            specs = {prefix + "toy.router.weight": TensorSpec((E, H))}
            for e in range(E):
                specs[prefix + f"toy.experts.{e}.up.weight"] = TensorSpec((I, H))
                specs[prefix + f"toy.experts.{e}.down.weight"] = TensorSpec((H, I))
            return specs

        def __init__(self, p, prefix, env, tensors):
            super().__init__(p, prefix, env, tensors)
            self.router = tensors.get(prefix + "toy.router.weight", torch.float32)
            self.up = [tensors.get(prefix + f"toy.experts.{e}.up.weight", env.dtype) for e in range(p["experts"])]
            self.down = [tensors.get(prefix + f"toy.experts.{e}.down.weight", env.dtype) for e in range(p["experts"])]

        def forward(self, x, batch):
            logits = ops.linear(x.float(), self.router)                   # router logits in 32-bit
            prob, choice = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(len(self.up)):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    y = ops.linear(torch.relu(ops.linear(x[rows].contiguous(), self.up[e])), self.down[e])
                    out[rows] = (y.float() * prob[rows, None]).to(x.dtype)
            return out

    class ScalingEncoding(PositionEncoding):
        def apply(self, qkv, batch, nh, nkv, d, kv_dest):
            i = torch.arange(d, device=qkv.device, dtype=torch.float32)
            s = 1.0 + 0.5 * torch.sin(batch.positions.float()[:, None] * (i[None, :] + 1.0) / 7.0)       # [T, d]
            heads = qkv[:, :(nh + nkv) * d].view(qkv.shape[0], nh + nkv, d)
            heads.copy_((heads.float() * s[:, None, :]).to(qkv.dtype))
            return False                                                   # the mixer writes k and v to the cache

    register_feed_forward("toy_routed_relu_mlp", RoutedReluMLP, replace=True)
    register_position_encoding("toy_scaling", ScalingEncoding, replace=True)

    def config_from_dict(d, where=""):
        from types import SimpleNamespace
        c = SimpleNamespace(**d)
        c.architecture = d["architectures"][0]
        c.to_dict = lambda: dict(d)
        return c

    def model_spec(c):
        H = c.hidden_size
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=c.eps, name=name))
        def attn(position):
            return PartSpec("paged_attention", dict(hidden_size=H, num_heads=c.heads, num_kv_heads=c.kv_heads,
                                                    head_dim=c.head_dim, window=0, scale=None, position=position))
        rope = PartSpec("rope", dict(head_dim=c.head_dim, theta=1000.0, scaling=None, max_position=c.max_pos))
        scaling = PartSpec("toy_scaling", dict(head_dim=c.head_dim))
        mixers = {"attn_scaling": attn(scaling), "attn_rope": attn(rope), "toy": PartSpec("toy_decaying_sum", dict(hidden_size=H))}
        ffns = {"routed": PartSpec("toy_routed_relu_mlp", dict(hidden_size=H, inner=c.inner, experts=c.experts)),
                "swiglu": PartSpec("swiglu", dict(hidden_size=H, intermediate_size=c.inner))}
        layers = tuple(LayerSpec(prefix=f"model.layers.{i}.", mixer=mixers[m], mixer_norm=norm("input_layernorm.weight"),
                                 ffn=ffns[f], ffn_norm=norm("post_attention_layernorm.weight"))
                       for i, (m, f) in enumerate(c.layer_kinds))
        return ModelSpec(hidden_size=H, vocab_size=c.vocab, max_position=c.max_pos,
                         embedding=PartSpec("token_embedding", dict(vocab_size=c.vocab, hidden_size=H, name="emb")),
                         layers=layers, final_norm=norm("model.norm.weight"),
                         head=PartSpec("lm_head", dict(vocab_size=c.vocab, hidden_size=H, name="emb")))

    register_architecture(Architecture("ToyRoutedForCausalLM", config_from_dict, model_spec), replace=True)


ROUTED_CFG = dict(architectures=["ToyRoutedForCausalLM"], hidden_size=48, heads=3, kv_heads=3, head_dim=16, inner=56,
                  experts=3, vocab=70, eps=1e-6, max_pos=128,
                  layer_kinds=[["attn_scaling", "routed"], ["attn_rope", "swiglu"], ["attn_rope", "routed"]])


def plain_routed_forward(model_dir, ids):
    cfg = json.loads((model_dir / "config.json").read_text())
    w = P.read_safetensors(model_dir / "model.safetensors")
    H, nh, nkv, d, E = cfg["hidden_size"], cfg["heads"], cfg["kv_heads"], cfg["head_dim"], cfg["experts"]
    T = len(ids)
    pos = np.arange(T)
    inv = P.rope_inv_freq(d, 1000.0, None)
    scale = 1.0 + 0.5 * np.sin(pos[:, None] * (np.arange(d)[None, :] + 1.0) / 7.0)
    x = P.embedding(w["emb"], ids)
    margins = []
    for i, (mixer, ffn) in enumerate(cfg["layer_kinds"]):
        p = f"model.layers.{i}."
        h = P.rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"])
        if mixer == "toy":
            s, outs = np.zeros(H), []
            for t in range(T):
                s = DECAY * s + h[t]
                outs.append(s.copy())
            x = x + P.linear(np.stack(outs), w[p + "toy.mix.weight"])
        else:
            q = P.linear(h, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, d)
            k = P.linear(h, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, d)
            v = P.linear(h, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, d)
            if mixer == "attn_rope":
                q, k = P.rope(q, pos, inv), P.rope(k, pos, inv)
            else:
                q, k = q * scale[:, None, :], k * scale[:, None, :]
            x = x + P.linear(P.attention(q, k, v, pos).reshape(T, nh * d), w[p + "self_attn.o_proj.weight"])
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg["eps"])
        if ffn == "routed":
            logits = P.linear(h, w[p + "toy.router.weight"])
            prob = np.exp(logits - logits.max(-1, keepdims=True))
            prob /= prob.sum(-1, keepdims=True)
            srt = np.sort(logits, axis=-1)
            margins.append(float((srt[:, -1] - srt[:, -2]).min()))
            y = np.zeros_like(x)
            for t in range(T):
                e = int(np.argmax(logits[t]))
                up = np.maximum(P.linear(h[t:t + 1], w[p + f"toy.experts.{e}.up.weight"]), 0)
                y[t] = prob[t, e] * P.linear(up, w[p + f"toy.experts.{e}.down.weight"])[0]
            x = x + y
        else:
            x = x + P.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                             w[p + "mlp.down_proj.weight"])
    return P.linear(P.rms_norm(x, w["model.norm.weight"], cfg["eps"]), w["emb"]), min(margins)


@pytest.mark.parametrize("mode", ["whole", "portions", "mixed"])
def test_toy_architecture_with_routing_and_another_position_encoding(mode, tmp_path):
    """32-bit only: a router's choice is discontinuous, so bfloat16 rounding of its input would flip near
    ties; here the smallest margin between the two best experts is checked to be far above the tolerance."""
    from railgun_b200.config.registry import load_config
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    from railgun_b200.weights.random_init import write_random_model
    register_routed_toys()
    mdir = tmp_path / "routed"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(ROUTED_CFG))
    arch, cfg = load_config(mdir)
    write_random_model(cfg, 5, mdir, std=0.2)
    (mdir / "config.json").write_text(json.dumps(ROUTED_CFG))
    reqs = {f"r{i}": p for i, p in enumerate(helpers.prompts(ROUTED_CFG["vocab"], [26, 7, 49, 38], seed=4))}
    steps = {"whole": helpers.trace_whole, "portions": helpers.trace_portions,
             "mixed": lambda r: helpers.trace_mixed(r, max_live=3, seed=6)}[mode](reqs)
    runner = ModelRunner(mdir, dtype="float32", page_size=8, max_tokens=helpers.peak_tokens(steps, 64), max_requests=3)
    assert len(runner.cache.kv) == 3 and not runner.cache.state
    assert not runner.use_graphs                            # the routed feed-forward said that it plans on the host
    rp = Replayer(runner, tmp_path / "out")
    for s in steps:
        rp.feed(s)
    rows = helpers.collect(steps, tmp_path / "out", ROUTED_CFG["vocab"])
    for name, toks in reqs.items():
        ref, margin = plain_routed_forward(mdir, toks)
        assert margin > 1e-4, "a router tie in the test's own data: change the seed"
        for p in range(len(toks)):
            assert np.abs(rows[(name, p)] - ref[p]).max() / np.abs(ref).max() < 2e-5, (name, p)
    runner.alloc.check()


def test_unknown_part_kind_is_a_clear_error():
    from railgun_b200.parts.registry import MIXERS
    with pytest.raises(KeyError) as e:
        MIXERS.get("no_such_mixer")
    assert "paged_attention" in str(e.value)
