"""Each part alone against its plain function, built from a PartSpec with
sizes unlike the tiny models', and the schedule as data: a layer named twice
and a layer that reads another layer's cache."""
import numpy as np
import pytest
import torch

import helpers
import plain_llama as P

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def bank_of(arrays, dtype):
    from railgun_b200.parts.model import TensorBank
    return TensorBank({k: torch.tensor(v, dtype=torch.float32).to(dtype) for k, v in arrays.items()}, DEV)


def env_of(dtype, H):
    from railgun_b200.parts.spec import BuildEnv
    return BuildEnv(device=DEV, dtype=dtype, hidden_size=H, max_position=512)


def rounded(arrays, dtype):
    """The values the part really holds (bfloat16 storage rounds them)."""
    return {k: torch.tensor(v, dtype=torch.float32).to(dtype).double().numpy() for k, v in arrays.items()}


def rel(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else got
    return np.abs(got - ref).max() / np.abs(ref).max()


TOL = {torch.float32: 5e-6, torch.bfloat16: 2e-2}
DTYPES = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_part(dtype):
    from railgun_b200.parts.registry import NORMS
    rng = np.random.default_rng(0)
    H = 200
    w = {"x.weight": 1 + 0.1 * rng.normal(size=H)}
    part = NORMS.get("rmsnorm")(dict(size=H, eps=3e-6, name="weight"), "x.", env_of(dtype, H), bank_of(w, dtype))
    assert NORMS.get("rmsnorm").tensor_specs(dict(size=H, eps=3e-6, name="weight"), "x.")["x.weight"].shape == (H,)
    resid = torch.tensor(rng.normal(size=(6, H)), dtype=torch.float32, device=DEV)
    pend = torch.tensor(rng.normal(size=(6, H)), dtype=torch.float32).to(dtype).to(DEV)
    ref = P.rms_norm(resid.double().cpu().numpy() + pend.double().cpu().numpy(), rounded(w, dtype)["x.weight"], 3e-6)
    out = part.add_norm(resid, pend)
    assert out.dtype == dtype and rel(out, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
def test_feed_forward_part(dtype):
    from railgun_b200.parts.registry import FEED_FORWARDS
    rng = np.random.default_rng(1)
    H, I = 72, 200
    w = {"l.mlp.gate_proj.weight": rng.normal(size=(I, H)) * 0.2, "l.mlp.up_proj.weight": rng.normal(size=(I, H)) * 0.2,
         "l.mlp.down_proj.weight": rng.normal(size=(H, I)) * 0.2}
    cls = FEED_FORWARDS.get("swiglu")
    p = dict(hidden_size=H, intermediate_size=I)
    assert {k: v.shape for k, v in cls.tensor_specs(p, "l.").items()} == {k: v.shape for k, v in w.items()}
    part = cls(p, "l.", env_of(dtype, H), bank_of(w, dtype))
    x = torch.tensor(rng.normal(size=(9, H)), dtype=torch.float32).to(dtype).to(DEV)
    r = rounded(w, dtype)
    ref = P.swiglu(x.double().cpu().numpy(), r["l.mlp.gate_proj.weight"], r["l.mlp.up_proj.weight"],
                   r["l.mlp.down_proj.weight"])
    assert rel(part.forward(x, None), ref) < TOL[dtype]


@pytest.mark.parametrize("rows", [1, 5, 8, 12])
def test_prenorm_block_hands_unfinished_values_only_to_parts_that_take_them(rows):
    """At small decode batches the built-in parts pass products and norms on unfinished (the residual addition
    and the norm then run inside the products' kernels).  Parts that did not ask for that see tensors only, and
    both routes give the block's result."""
    from railgun_b200 import ops
    from railgun_b200.parts.base import Mixer, Norm, Stream
    from railgun_b200.parts.block import PreNorm
    from railgun_b200.parts.model import Branch, Layer
    from railgun_b200.parts.registry import FEED_FORWARDS, NORMS
    dtype, H, I, eps = torch.bfloat16, 72, 200, 1e-5
    rng = np.random.default_rng(rows)
    w = {}
    for l in ("a.", "b."):
        w.update({l + "n1": 1 + 0.1 * rng.normal(size=H), l + "n2": 1 + 0.1 * rng.normal(size=H),
                  l + "mix1": rng.normal(size=(H, H)) * 0.2, l + "mix2": rng.normal(size=(H, H)) * 0.2,
                  l + "mlp.gate_proj.weight": rng.normal(size=(I, H)) * 0.2,
                  l + "mlp.up_proj.weight": rng.normal(size=(I, H)) * 0.2,
                  l + "mlp.down_proj.weight": rng.normal(size=(H, I)) * 0.2})
    r = rounded(w, dtype)
    x0 = rng.normal(size=(rows, H))
    ref = x0.copy()
    for l in ("a.", "b."):
        ref = ref + P.linear(P.linear(P.rms_norm(ref, r[l + "n1"], eps), r[l + "mix1"]), r[l + "mix2"])
        ref = ref + P.swiglu(P.rms_norm(ref, r[l + "n2"], eps), r[l + "mlp.gate_proj.weight"],
                             r[l + "mlp.up_proj.weight"], r[l + "mlp.down_proj.weight"])
    seen = []

    class TwoLinears(Mixer):
        def __init__(self, prefix, tensors, lazy):
            self.w1, self.w2 = tensors.get(prefix + "mix1", dtype), tensors.get(prefix + "mix2", dtype)
            self.takes_normed_rows = self.defers_output = lazy

        def forward(self, x, batch, cache, writes=True, defer=False):
            seen.append(("mixer", type(x).__name__))
            y = ops.linear(x, self.w1)
            return ops.PendingLinear(y, self.w2) if defer else ops.linear(y, self.w2)

    class PlainNorm(Norm):
        def __init__(self, weight):
            self.weight = weight

        def add_norm(self, resid, pending, rows=None):
            seen.append(("norm", type(pending).__name__))
            return ops.add_rmsnorm(resid, pending, self.weight, eps, dtype, rows)

    def run(lazy):
        seen.clear()
        env, tensors = env_of(dtype, H), bank_of(w, dtype)
        layers = []
        for l in ("a.", "b."):
            norm = lambda name: (NORMS.get("rmsnorm")(dict(size=H, eps=eps, name=name), l, env, tensors) if lazy
                                 else PlainNorm(tensors.get(l + name, torch.float32)))
            layers.append(Layer(branches=[
                Branch(norm("n1"), TwoLinears(l, tensors, lazy), "mixer"),
                Branch(norm("n2"), FEED_FORWARDS.get("swiglu")(dict(hidden_size=H, intermediate_size=I), l, env, tensors),
                       "ffn")], arrangement=PreNorm()))
        stream = Stream(torch.tensor(x0, dtype=torch.float32, device=DEV))
        for layer in layers:
            layer.arrangement.run(layer, stream, None, None, True)
        pending = stream.pending.materialize() if isinstance(stream.pending, ops.PendingLinear) else stream.pending
        return stream.resid.double().cpu().numpy() + pending.double().cpu().numpy(), list(seen)

    out_lazy, seen_lazy = run(True)
    out_plain, seen_plain = run(False)
    assert rel(out_lazy, ref) < TOL[dtype] and rel(out_plain, ref) < TOL[dtype]
    assert all(kind == "Tensor" or kind == "NoneType" for _, kind in seen_plain)
    small = rows <= ops.SKINNY_AUTO_ROWS
    assert seen_lazy == [("mixer", "Tensor"), ("mixer", "NormedRows" if small else "Tensor")]


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts_share_a_tied_tensor(dtype):
    from railgun_b200.parts.registry import EMBEDDINGS, HEADS
    rng = np.random.default_rng(2)
    V, H = 300, 40
    w = {"emb": rng.normal(size=(V, H))}
    bank = bank_of(w, dtype)
    p = dict(vocab_size=V, hidden_size=H, name="emb")
    emb = EMBEDDINGS.get("token_embedding")(p, "", env_of(dtype, H), bank)
    head = HEADS.get("lm_head")(p, "", env_of(dtype, H), bank)
    assert emb.table.data_ptr() == head.weight.data_ptr()
    ids = torch.tensor([5, 299, 0, 5], dtype=torch.int32, device=DEV)
    r = rounded(w, dtype)["emb"]
    assert np.array_equal(emb.embed(ids).cpu().numpy(), r[[5, 299, 0, 5]].astype(np.float32))
    h = torch.tensor(rng.normal(size=(3, H)), dtype=torch.float32).to(dtype).to(DEV)
    lg = head.logits(h)
    assert lg.dtype == torch.float32 and rel(lg, h.double().cpu().numpy() @ r.T) < (5e-6 if dtype == torch.float32 else 1e-5)


def _attention_fixture(dtype, window, page, seed):
    """An attention mixer alone: two requests run in two steps each through
    the cache, compared with the plain attention over the whole sequences."""
    from railgun_b200.cache.manager import CacheManager
    from railgun_b200.engine.batch import StepEntry, build_step_batch
    from railgun_b200.engine.runner import _CacheViews
    from railgun_b200.parts.registry import MIXERS
    from railgun_b200.parts.spec import PartSpec
    rng = np.random.default_rng(seed)
    H, nh, nkv, d = 56, 6, 3, 16
    pos = PartSpec("rope", dict(head_dim=d, theta=12345.0, scaling=None, max_position=512))
    p = dict(hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=d, window=window, scale=None, position=pos)
    cls = MIXERS.get("paged_attention")
    w = {"L.self_attn.q_proj.weight": rng.normal(size=(nh * d, H)) * 0.3,
         "L.self_attn.k_proj.weight": rng.normal(size=(nkv * d, H)) * 0.3,
         "L.self_attn.v_proj.weight": rng.normal(size=(nkv * d, H)) * 0.3,
         "L.self_attn.o_proj.weight": rng.normal(size=(H, nh * d)) * 0.3}
    assert {k: v.shape for k, v in cls.tensor_specs(p, "L.").items()} == {k: v.shape for k, v in w.items()}
    part = cls(p, "L.", env_of(dtype, H), bank_of(w, dtype))
    cache = CacheManager({0: cls.cache_need(p)}, page, 256, 4, dtype, DEV)
    views = _CacheViews(cache)
    lens = {1: 37, 2: 50}
    xs = {r: torch.tensor(rng.normal(size=(n, H)), dtype=torch.float32).to(dtype) for r, n in lens.items()}
    got = {r: [] for r in lens}
    cuts = {1: [(0, 20), (20, 37)], 2: [(0, 49), (49, 50)]}
    for step in range(2):
        entries = [StepEntry(r, [0] * (cuts[r][step][1] - cuts[r][step][0]), []) for r in lens]
        batch = build_step_batch(entries, cache.alloc, [page], 10, 512, DEV)
        x = torch.cat([xs[r][cuts[r][step][0]:cuts[r][step][1]] for r in lens]).to(DEV)
        y = part.forward(x, batch, views.view(0), True)
        off = 0
        for e in entries:
            got[e.request_id].append(y[off:off + len(e.tokens)].double().cpu().numpy())
            off += len(e.tokens)
            cache.alloc.commit(e.request_id, cache.alloc.num_computed(e.request_id) + len(e.tokens))
    r_w = rounded(w, dtype)
    inv = P.rope_inv_freq(d, 12345.0, None)
    worst = 0.0
    for r, n in lens.items():
        x = xs[r].double().numpy()
        posn = np.arange(n)
        q = P.rope(P.linear(x, r_w["L.self_attn.q_proj.weight"]).reshape(n, nh, d), posn, inv)
        k = P.rope(P.linear(x, r_w["L.self_attn.k_proj.weight"]).reshape(n, nkv, d), posn, inv)
        v = P.linear(x, r_w["L.self_attn.v_proj.weight"]).reshape(n, nkv, d)
        ref = P.linear(P.attention(q, k, v, posn, window=window or None).reshape(n, nh * d),
                       r_w["L.self_attn.o_proj.weight"])
        worst = max(worst, rel(np.concatenate(got[r]), ref))
    return worst


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,page", [(0, 16), (0, 4), (11, 8)])
def test_attention_mixer_part(dtype, window, page):
    assert _attention_fixture(dtype, window, page, seed=window + page) < TOL[dtype] * 2


def _runner_with_spec(name, dtype, spec_fn, page, max_tokens=512):
    from railgun_b200.engine.runner import ModelRunner
    return ModelRunner(helpers.model_dir(name), dtype=dtype, page_size=page, max_tokens=max_tokens, max_requests=4,
                       spec_override=spec_fn)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_schedule_names_a_layer_twice_and_shares_a_cache(dtype, tmp_path):
    """Order is data: layer 0, layer 1, layer 0 again (its own cache), then
    layer 2 reading the cache the first entry wrote."""
    import dataclasses
    from railgun_b200.models.llama import llama_model_spec
    from railgun_b200.parts.spec import ScheduleEntry
    from railgun_b200.replay import Replayer
    order = [(0, 0, True), (1, 1, True), (0, 2, True), (2, 0, False)]

    def spec_fn(cfg):
        return dataclasses.replace(llama_model_spec(cfg), schedule=tuple(ScheduleEntry(*o) for o in order))

    cfg = helpers.TINY_B
    runner = _runner_with_spec("B", dtype, spec_fn, page=8)
    assert sorted(runner.cache.kv) == [0, 1, 2]
    reqs = {f"s{i}": p for i, p in enumerate(helpers.prompts(cfg["vocab_size"], [45, 70], seed=21))}
    plain = P.PlainLlama(helpers.model_dir("B"), schedule=order)
    steps = helpers.trace_portions(reqs, sizes=(13, 2, 30, 5))
    rp = Replayer(runner, tmp_path)
    for s in steps:
        rp.feed(s)
    rows = helpers.collect(steps, tmp_path, cfg["vocab_size"])
    tol = 2e-5 if dtype == "float32" else 3e-2
    for name, toks in reqs.items():
        ref = plain.forward(toks)
        for p in range(len(toks)):
            assert np.abs(rows[(name, p)] - ref[p]).max() / np.abs(ref).max() < tol, (name, p)
    # the default order gives other numbers: the schedule was really used
    assert np.abs(P.PlainLlama(helpers.model_dir("B")).forward(reqs["s0"]) - plain.forward(reqs["s0"])).max() > 1e-3


def test_bad_schedules_are_refused():
    import dataclasses
    from railgun_b200.models.llama import llama_model_spec
    from railgun_b200.parts.spec import ScheduleEntry
    for order in ([(0, 0, True), (1, 0, True)], [(0, 1, False)], [(7, 0, True)]):
        def spec_fn(cfg, order=order):
            return dataclasses.replace(llama_model_spec(cfg), schedule=tuple(ScheduleEntry(*o) for o in order))
        with pytest.raises(ValueError):
            _runner_with_spec("A", "float32", spec_fn, page=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_attention_through_the_engine_frees_pages(dtype, tmp_path):
    """The attention part with a window, chosen layer by layer: layer 0 keeps
    every key, the others a window of 24; the windowed group's pages come back
    while the request is still running, and the logits still match."""
    import dataclasses
    from railgun_b200.models.llama import llama_model_spec
    from railgun_b200.parts.spec import PartSpec
    from railgun_b200.replay import Replayer
    W = 24

    def spec_fn(cfg):
        spec = llama_model_spec(cfg)
        layers = list(spec.layers)
        for i in range(1, len(layers)):
            mp = dict(layers[i].mixer.params, window=W)
            layers[i] = dataclasses.replace(layers[i], mixer=PartSpec("paged_attention", mp))
        return dataclasses.replace(spec, layers=tuple(layers))

    cfg = helpers.TINY_B
    runner = _runner_with_spec("B", dtype, spec_fn, page=8, max_tokens=160)
    assert len(runner.cache.groups) == 2 and runner.cache.groups[1].need.window == W
    toks = helpers.prompts(cfg["vocab_size"], [150], seed=31)[0]

    class WindowedPlain(P.PlainLlama):
        def forward(self, ids, start_pos=0):
            T = len(ids)
            pos = np.arange(T)
            x = P.embedding(self.w["model.embed_tokens.weight"], ids)
            for li in range(self.L):
                lw = self.layer_weights(li)
                h = P.rms_norm(x, lw["ln1"], self.eps)
                q = P.rope(P.linear(h, lw["q"]).reshape(T, self.nh, self.d), pos, self.inv_freq)
                k = P.rope(P.linear(h, lw["k"]).reshape(T, self.nkv, self.d), pos, self.inv_freq)
                v = P.linear(h, lw["v"]).reshape(T, self.nkv, self.d)
                a = P.attention(q, k, v, pos, window=None if li == 0 else W).reshape(T, self.nh * self.d)
                x = x + P.linear(a, lw["o"])
                x = x + P.swiglu(P.rms_norm(x, lw["ln2"], self.eps), lw["gate"], lw["up"], lw["down"])
            x = P.rms_norm(x, self.w["model.norm.weight"], self.eps)
            return P.linear(x, self.w["lm_head.weight"])

    ref = WindowedPlain(helpers.model_dir("B")).forward(toks)
    steps = helpers.trace_portions({"w": toks}, sizes=(9, 2, 17, 1, 1, 30, 3))
    rp = Replayer(runner, tmp_path)
    min_free = []
    for s in steps:
        rp.feed(s)
        if not s["end"]:
            rid = rp._ids["w"]
            held = int((runner.alloc.block_table(rid, 1) >= 0).sum())
            assert held <= -(-(W + 30) // 8) + 1
            min_free.append(held)
    rows = helpers.collect(steps, tmp_path, cfg["vocab_size"])
    tol = 2e-5 if dtype == "float32" else 3e-2
    for p in range(len(toks)):
        assert np.abs(rows[("w", p)] - ref[p]).max() / np.abs(ref).max() < tol, p
    runner.alloc.check()
