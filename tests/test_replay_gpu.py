"""Trace replay on the GPU against the plain implementation: every request
whole, with the last 32 tokens decoded one by one, in portions of changing
size, and mixed with other requests in a pool so small that pages are used
again; in 32-bit and in bfloat16, for every tiny configuration (the third has
head size 64 and prompts of several hundred tokens, which the tcgen05
attention kernel with its 128-row tiles takes)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import helpers
from plain_llama import PlainLlama

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 100, 131, 64, 48], "B": [1, 9, 40, 63, 100, 200, 77, 129],
           "C": [300, 392, 400, 129, 257, 64, 395, 390]}
# portion sizes of the "portions" and "mixed" cuts; C's cross the 64- and 128-row tiles of the attention kernels
PORTIONS = {"C": (130, 2, 64, 7, 128, 3, 65, 2, 33, 129)}
MIXED = {"C": (5, 1, 2, 70, 1, 1, 3, 140, 1, 2, 128, 17)}
# Largest absolute logit difference allowed, as a fraction of the largest
# absolute logit of the row's sequence.  32-bit differs from the 64-bit plain
# implementation by accumulated rounding only; bfloat16 rounds activations to
# 8 bits of mantissa between kernels.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}

_oracle_cache: dict = {}


def oracle(name):
    if name not in _oracle_cache:
        cfg = helpers.TINY[name][0]
        reqs = {f"r{i}": p for i, p in enumerate(helpers.prompts(cfg["vocab_size"], LENGTHS[name], seed=11))}
        plain = PlainLlama(helpers.model_dir(name))
        _oracle_cache[name] = (reqs, {k: plain.forward(v) for k, v in reqs.items()})
    return _oracle_cache[name]


def make_trace(mode, reqs, name="A"):
    if mode == "whole":
        return helpers.trace_whole(reqs)
    if mode == "tail":
        return helpers.trace_tail_decode(reqs, 32)
    if mode == "portions":
        return helpers.trace_portions(reqs, **({"sizes": PORTIONS[name]} if name in PORTIONS else {}))
    if mode == "mixed":
        return helpers.trace_mixed(reqs, max_live=4, seed=5, **({"sizes": MIXED[name]} if name in MIXED else {}))
    raise ValueError(mode)


def compare(rows, reqs, logits, dtype, what):
    worst = 0.0
    for name, toks in reqs.items():
        ref = logits[name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            got = rows[(name, p)]
            err = np.abs(got - ref[p]).max() / scale
            if err > TOL[dtype]:
                raise AssertionError(f"{what}: request {name} (length {len(toks)}) first differs at position {p}: "
                                     f"relative error {err:.3e} > {TOL[dtype]:.1e}")
            worst = max(worst, err)
    return worst


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_replay_matches_plain(name, dtype, mode, tmp_path):
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    cfg, _, page = helpers.TINY[name]
    reqs, logits = oracle(name)
    steps = make_trace(mode, reqs, name)
    max_tokens = helpers.peak_tokens(steps, 64)
    runner = ModelRunner(helpers.model_dir(name), dtype=dtype, page_size=page, max_tokens=max_tokens,
                         max_requests=4)
    rp = Replayer(runner, tmp_path)
    for s in steps:
        rp.feed(s)
    runner.check_device_errors()
    runner.alloc.check()
    assert runner.alloc.num_requests() == 0
    rows = helpers.collect(steps, tmp_path, cfg["vocab_size"])
    worst = compare(rows, reqs, logits, dtype, f"tiny {name} {dtype} {mode}")
    print(f"tiny {name} {dtype} {mode}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_steps_of_a_repeated_layout_replay_a_graph(name, dtype, tmp_path):
    """Large steps whose packed layout repeats are captured the second time and replayed from then on.  With
    the threshold lowered to two tokens, equal portions of several requests (alone, and beside single tokens of
    another request) go through the eager run, the capture and the replays, over pages that are used again; every
    logit is compared with the plain implementation."""
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    cfg, _, page = helpers.TINY[name]
    reqs, logits = oracle(name)
    P = 130 if name == "C" else 21                               # C: a tile of 128 rows and one of 2 in every portion
    names = [k for k, v in reqs.items() if len(v) >= 3 * P][:4]
    decoder = next(k for k, v in reqs.items() if len(v) >= 40 and k not in names)
    steps, n = [], 0
    # the decoder's prompt but for its last 12 tokens, then it decodes beside the others' portions
    dt = reqs[decoder]
    steps.append({"step": n, "entries": [{"id": decoder, "tokens": dt[:len(dt) - 12], "want": list(range(len(dt) - 12))}],
                  "end": []})
    n += 1
    fed = len(dt) - 12
    for r in names:
        toks = reqs[r][:3 * P]                                   # three portions of P tokens: the same layout 12 times
        for p in range(3):
            entries = [{"id": r, "tokens": toks[P * p:P * p + P], "want": list(range(P))}]
            if fed < len(dt):
                entries.append({"id": decoder, "tokens": [dt[fed]], "want": [0]})
                fed += 1
            steps.append({"step": n, "entries": entries, "end": [r] if p == 2 else []})
            n += 1
    steps[-1]["end"].append(decoder)
    runner = ModelRunner(helpers.model_dir(name), dtype=dtype, page_size=page,
                         max_tokens=helpers.peak_tokens(steps, 64), max_requests=4)
    runner.shape_graph_min_tokens = 2
    rp = Replayer(runner, tmp_path)
    for s in steps:
        rp.feed(s)
    assert len(runner._shape_steps) >= 1                          # something was captured ...
    assert any(v >= 2 for v in runner._shape_seen.values())
    runner.check_device_errors()
    runner.alloc.check()
    rows = helpers.collect(steps, tmp_path, cfg["vocab_size"])
    some = {r: reqs[r][:3 * P] for r in names}
    some[decoder] = dt
    ref = {r: logits[r][:len(t)] for r, t in some.items()}
    # rows of a prefix do not depend on what follows it, so the prefix's reference rows are the request's own
    compare(rows, some, ref, dtype, f"repeated layouts {name} {dtype}")


def test_pages_are_used_again(tmp_path):
    """The mixed trace needs more pages over its life than the pool has."""
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    cfg, _, page = helpers.TINY["B"]
    reqs, _ = oracle("B")
    steps = make_trace("mixed", reqs)
    max_tokens = helpers.peak_tokens(steps, 64)
    assert sum(-(-len(t) // page) for t in reqs.values()) * page > max_tokens
    runner = ModelRunner(helpers.model_dir("B"), dtype="float32", page_size=page, max_tokens=max_tokens,
                         max_requests=4)
    rp = Replayer(runner, tmp_path)
    held, freed, reused = {}, set(), set()
    for s in steps:
        rp.feed(s)
        now = {rid: {int(p) for p in runner.alloc.block_table(rid, 0)} for rid in rp._ids.values()}
        for rid, pages in now.items():
            reused |= (pages - held.get(rid, set())) & freed     # a page handed out now that an ended request gave back
        for rid, pages in held.items():
            if rid not in now:
                freed |= pages
        held = now
    assert reused, "no page that an ended request gave back was handed to a later request"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype, tmp_path):
    """bin/trace_run as a user runs it: steps on standard input, files out."""
    cfg, _, page = helpers.TINY["A"]
    reqs, logits = oracle("A")
    some = {k: reqs[k] for k in list(reqs)[:4]}
    steps = helpers.trace_mixed(some, max_live=3, seed=1)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(helpers.model_dir("A")),
         "--dtype", dtype, "--out", str(out), "--max-tokens", str(helpers.peak_tokens(steps, 64))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    rows = helpers.collect(steps, out, cfg["vocab_size"])
    compare(rows, some, logits, dtype, f"trace_run {dtype}")
