"""The model at the layer sizes that bench.py times (Llama 3.2 1B: hidden
2,048, 32 query and 8 key/value heads of size 64, intermediate 8,192,
vocabulary 128,256, tied head, llama3 frequency scaling), with 2 of its 16
layers.  These sizes take code that the tiny configurations do not reach: the
tcgen05 attention kernel inside real steps, the exact head-size-64
specialisations, the tcgen05 gate|up product on pairs of CTAs from 1,024 rows
on, the library products between 17 and 1,023 rows, the fused decode products
at their compiled widths, and graphs captured for repeated large layouts.

The 32-bit path is held to the plain implementation; bfloat16 is held to the
32-bit path run on the same stored weights (the packed forward of
crates/vllm-models/src/llama/architecture.rs:141-156 either way), in every cut
of the work, with a tolerance taken from the measured rounding noise."""
import numpy as np
import pytest

import helpers
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

BENCH_SIZES = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    head_dim=64, num_hidden_layers=2, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072, torch_dtype="bfloat16")
PAGE = 16
LENGTHS = [2200, 300, 150, 40, 1100, 77]
# bfloat16 against the 32-bit path: the largest difference in a row as a fraction of the largest absolute logit
# of the request, and the row's root-mean-square difference as a fraction of its root-mean-square logit.
# Measured on a B200 over every cut below (bfloat16 rounds activations to 8 bits of mantissa between kernels;
# two layers; 128,256 logits a row): worst rows 1.3e-2 and 1.1e-2; the bounds leave a factor of two.
BF16_VS_F32 = 2.6e-2
BF16_VS_F32_RMS = 2.2e-2
F32_VS_PLAIN = 2e-5

_made: dict = {}


def test_these_are_the_sizes_bench_times():
    import bench                                                  # the repository's root is on the path (conftest)
    for key, value in bench.LLAMA_3_2_1B.items():
        if key != "num_hidden_layers":
            assert BENCH_SIZES[key] == value, key


def folder():
    if "dir" not in _made:
        import tempfile
        from pathlib import Path
        from railgun_b200.config.llama import LlamaConfig
        from railgun_b200.weights.random_init import write_random_model
        d = Path(tempfile.mkdtemp(prefix="rg_bench_sizes_"))
        write_random_model(LlamaConfig.from_dict(BENCH_SIZES), 7, d)
        _made["dir"] = d
    return _made["dir"]


def requests():
    if "reqs" not in _made:
        toks = helpers.prompts(BENCH_SIZES["vocab_size"], LENGTHS, seed=21)
        reqs = {f"r{i}": t for i, t in enumerate(toks)}
        # logits are wanted at every 37th position, at both sides of every 128-row tile edge and at the end
        keep = {}
        for name, t in reqs.items():
            n = len(t)
            places = set(range(0, n, 37)) | set(range(max(0, n - 8), n))
            for edge in range(128, n, 128):
                places |= {edge - 1, edge}
            keep[name] = places
        _made["reqs"] = (reqs, keep)
    return _made["reqs"]


def restrict_want(steps, keep):
    """The same steps, asking only for the logits at the absolute positions in ``keep[request]``."""
    pos = {}
    for s in steps:
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            e["want"] = [w for w in range(len(e["tokens"])) if start + w in keep[e["id"]]]
            pos[e["id"]] = start + len(e["tokens"])
        for name in s["end"]:
            pos.pop(name, None)
    return steps


def replay(dtype, steps, tmp_path, max_requests=4, min_graph_tokens=None):
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    runner = ModelRunner(folder(), dtype=dtype, page_size=PAGE, max_tokens=helpers.peak_tokens(steps, 64),
                         max_requests=max_requests)
    if min_graph_tokens is not None:
        runner.shape_graph_min_tokens = min_graph_tokens
    out = tmp_path / dtype
    rp = Replayer(runner, out)
    for s in steps:
        rp.feed(s)
    runner.check_device_errors()
    runner.alloc.check()
    assert runner.alloc.num_requests() == 0
    rows = helpers.collect(steps, out, BENCH_SIZES["vocab_size"])
    del rp, runner
    import torch
    torch.cuda.empty_cache()
    return rows


def reference_rows(tmp_path):
    """The 32-bit path, every request alone and whole: (request, position) -> logits row."""
    if "f32" not in _made:
        reqs, keep = requests()
        _made["f32"] = replay("float32", restrict_want(helpers.trace_whole(reqs), keep), tmp_path / "ref")
    return _made["f32"]


def rms_error(got, want):
    return float(np.sqrt(np.mean((got - want) ** 2)) / np.sqrt(np.mean(want ** 2)))


def compare(rows, ref, what, tol, tol_rms=None):
    reqs, keep = requests()
    worst, worst_rms, flips = 0.0, 0.0, 0
    for name in reqs:
        places = sorted(p for p in keep[name] if (name, p) in rows)
        assert places, f"{what}: no rows of request {name}"
        scale = max(np.abs(ref[(name, p)]).max() for p in places)
        for p in places:
            got, want = rows[(name, p)], ref[(name, p)]
            err = np.abs(got - want).max() / scale
            if err > tol:
                raise AssertionError(f"{what}: request {name} (length {len(reqs[name])}) first differs at position "
                                     f"{p}: relative error {err:.3e} > {tol:.1e}")
            worst = max(worst, err)
            if tol_rms is not None:
                rms = rms_error(got, want)
                assert rms < tol_rms, f"{what}: request {name} position {p}: rms error {rms:.3e} > {tol_rms:.1e}"
                worst_rms = max(worst_rms, rms)
            top2 = np.sort(want)[-2:]
            if top2[1] - top2[0] > 2 * tol * scale:                  # a clear winner stays the winner
                assert int(np.argmax(got)) == int(np.argmax(want)), f"{what}: {name} position {p}: another argmax"
            else:
                flips += 1
    print(f"{what}: worst relative error {worst:.3e}, worst rms error {worst_rms:.3e} "
          f"({flips} rows without a clear winner)")
    return worst


def test_float32_path_matches_plain_at_bench_sizes(tmp_path):
    """A 96-token prompt whole, in portions and with its tail decoded, 32-bit, against the plain implementation."""
    toks = helpers.prompts(BENCH_SIZES["vocab_size"], [96], seed=22)[0]
    plain = PlainLlama(folder()).forward(toks)
    scale = np.abs(plain).max()
    reqs = {"p": toks}
    for cut, steps in (("whole", helpers.trace_whole(reqs)),
                       ("portions", helpers.trace_portions(reqs, sizes=(40, 2, 17, 37))),
                       ("tail", helpers.trace_tail_decode(reqs, 12))):
        rows = None
        from railgun_b200.engine.runner import ModelRunner
        from railgun_b200.replay import Replayer
        runner = ModelRunner(folder(), dtype="float32", page_size=PAGE, max_tokens=128, max_requests=2)
        rp = Replayer(runner, tmp_path / cut)
        for s in steps:
            rp.feed(s)
        runner.check_device_errors()
        rows = helpers.collect(steps, tmp_path / cut, BENCH_SIZES["vocab_size"])
        for p in range(len(toks)):
            err = np.abs(rows[("p", p)] - plain[p]).max() / scale
            assert err < F32_VS_PLAIN, f"float32 {cut}: position {p}: relative error {err:.3e}"
        del rp, runner


def cut_steps(mode):
    reqs, keep = requests()
    if mode == "whole":
        steps = helpers.trace_whole(reqs)
    elif mode == "tail":
        steps = helpers.trace_tail_decode(reqs, 32)
    elif mode == "portions":
        # the longest request begins with one portion of 2,048 tokens; the others cross the attention tiles
        steps = helpers.trace_portions(reqs, sizes=(2048, 2, 130, 64, 7, 128, 3, 600, 65, 2, 33))
    elif mode == "mixed":
        steps = helpers.trace_mixed(reqs, max_live=4, seed=9, sizes=(5, 1, 2, 70, 1, 1, 3, 140, 1, 600, 128, 17, 1100))
    else:
        raise ValueError(mode)
    return restrict_want(steps, keep)


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_bfloat16_matches_the_float32_path_at_bench_sizes(mode, tmp_path):
    ref = reference_rows(tmp_path)
    rows = replay("bfloat16", cut_steps(mode), tmp_path)
    compare(rows, ref, f"bench sizes bfloat16 {mode}", BF16_VS_F32, BF16_VS_F32_RMS)


def test_float32_path_is_the_same_in_every_cut_at_bench_sizes(tmp_path):
    ref = reference_rows(tmp_path)
    rows = replay("float32", cut_steps("mixed"), tmp_path)
    compare(rows, ref, "bench sizes float32 mixed", F32_VS_PLAIN)


def test_repeated_large_layouts_replay_graphs_at_bench_sizes(tmp_path):
    """Portions of 256 tokens of two requests, one after the other: the layout repeats, so the steps run eagerly,
    are captured and replay; the tcgen05 kernels run inside the captured graph."""
    reqs, keep = requests()
    steps, n = [], 0
    for name in ("r0", "r4"):
        toks = reqs[name][:1024]
        for p in range(4):
            steps.append({"step": n, "entries": [{"id": name, "tokens": toks[256 * p:256 * p + 256], "want": []}],
                          "end": [name] if p == 3 else []})
            n += 1
    restrict_want(steps, keep)
    ref = reference_rows(tmp_path)
    rows = replay("bfloat16", steps, tmp_path)
    for (name, p), row in rows.items():
        scale = np.abs(ref[(name, p)]).max()
        assert np.abs(row - ref[(name, p)]).max() / scale < BF16_VS_F32, (name, p)
        assert rms_error(row, ref[(name, p)]) < BF16_VS_F32_RMS, (name, p)
    assert len(rows) > 40


def test_forty_requests_decode_together_at_bench_sizes(tmp_path):
    """Forty live requests: their prompts in steps of several requests, then decode steps of forty rows (the
    products of 17 to 64 rows, SiLU-mul on interleaved storage, split attention over forty contexts), bfloat16
    against the 32-bit path fed the same tokens."""
    V = BENCH_SIZES["vocab_size"]
    lengths = [20 + (7 * i) % 50 for i in range(40)]
    toks = helpers.prompts(V, [n + 4 for n in lengths], seed=23)
    steps, n = [], 0
    for lo in range(0, 40, 10):                                     # ten prompts a step
        steps.append({"step": n, "entries": [{"id": f"q{i}", "tokens": toks[i][:lengths[i]], "want": [lengths[i] - 1]}
                                             for i in range(lo, lo + 10)], "end": []})
        n += 1
    for k in range(4):                                              # four decode steps of all forty
        steps.append({"step": n, "entries": [{"id": f"q{i}", "tokens": [toks[i][lengths[i] + k]], "want": [0]}
                                             for i in range(40)], "end": []})
        n += 1
    steps[-1]["end"] = [f"q{i}" for i in range(40)]
    got = {}
    for dtype in ("float32", "bfloat16"):
        from railgun_b200.engine.runner import ModelRunner
        from railgun_b200.replay import Replayer
        runner = ModelRunner(folder(), dtype=dtype, page_size=PAGE, max_tokens=40 * 80, max_requests=40)
        rp = Replayer(runner, tmp_path / dtype)
        for s in steps:
            rp.feed(s)
        runner.check_device_errors()
        got[dtype] = helpers.collect(steps, tmp_path / dtype, V)
        del rp, runner
    worst, worst_rms = 0.0, 0.0
    for key, want in got["float32"].items():
        err = np.abs(got["bfloat16"][key] - want).max() / np.abs(want).max()
        rms = rms_error(got["bfloat16"][key], want)
        worst, worst_rms = max(worst, err), max(worst_rms, rms)
        assert err < BF16_VS_F32, f"request {key[0]} position {key[1]}: relative error {err:.3e}"
        assert rms < BF16_VS_F32_RMS, f"request {key[0]} position {key[1]}: rms error {rms:.3e}"
    print(f"forty requests: worst relative error {worst:.3e}, worst rms error {worst_rms:.3e}")
