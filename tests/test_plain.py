"""The plain implementation checked against direct, loop-level statements of
the formulas and against its own invariants."""
import math

import numpy as np
import pytest

import helpers
import plain_llama as P


def test_rms_norm_against_loops():
    rng = np.random.default_rng(0)
    x, w = rng.normal(size=(3, 10)), rng.normal(size=10)
    got = P.rms_norm(x, w, 1e-6)
    for t in range(3):
        ms = sum(v * v for v in x[t]) / 10
        for i in range(10):
            assert abs(got[t, i] - w[i] * x[t, i] / math.sqrt(ms + 1e-6)) < 1e-12


def test_rope_llama3_scaling_hits_all_three_branches():
    sc = helpers.TINY_B["rope_scaling"]
    d, theta = helpers.TINY_B["head_dim"], helpers.TINY_B["rope_theta"]
    base = P.rope_inv_freq(d, theta, None)
    scaled = P.rope_inv_freq(d, theta, sc)
    lam = 2 * math.pi / base
    kept = lam < 64 / 4
    divided = lam > 64 / 1
    mid = ~kept & ~divided
    assert kept.any() and divided.any() and mid.any()
    assert np.allclose(scaled[kept], base[kept]) and np.allclose(scaled[divided], base[divided] / 8)
    for i in np.where(mid)[0]:
        s = (64 / lam[i] - 1) / (4 - 1)
        assert abs(scaled[i] - ((1 - s) * base[i] / 8 + s * base[i])) < 1e-15
        assert base[i] / 8 < scaled[i] < base[i]


def test_rope_rotates_pairs_and_depends_on_distance_only():
    rng = np.random.default_rng(1)
    inv = P.rope_inv_freq(8, 10000.0, None)
    x = rng.normal(size=(1, 1, 8))
    y = P.rope(x, [3], inv)
    for i in range(4):                                   # pairs (i, i + d/2), crates/vllm-cuda/src/kernels/rope.cu:30-41
        c, s = math.cos(3 * inv[i]), math.sin(3 * inv[i])
        assert abs(y[0, 0, i] - (x[0, 0, i] * c - x[0, 0, i + 4] * s)) < 1e-12
        assert abs(y[0, 0, i + 4] - (x[0, 0, i + 4] * c + x[0, 0, i] * s)) < 1e-12
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    dots = [float((P.rope(q, [a], inv) * P.rope(k, [a - 5], inv)).sum()) for a in (5, 9, 100)]
    assert max(dots) - min(dots) < 1e-9
    assert abs(np.linalg.norm(y) - np.linalg.norm(x)) < 1e-12


def test_attention_against_loops_with_groups_and_window():
    rng = np.random.default_rng(2)
    T, nh, nkv, d = 7, 4, 2, 6
    q, k, v = rng.normal(size=(T, nh, d)), rng.normal(size=(T, nkv, d)), rng.normal(size=(T, nkv, d))
    for window in (None, 3):
        got = P.attention(q, k, v, np.arange(T), window=window)
        for t in range(T):
            for h in range(nh):
                kh = h // (nh // nkv)
                lo = 0 if not window else max(0, t - window + 1)
                s = [float(q[t, h] @ k[j, kh]) / math.sqrt(d) for j in range(lo, t + 1)]
                m = max(s)
                p = [math.exp(x - m) for x in s]
                o = sum(pj * v[lo + j, kh] for j, pj in enumerate(p)) / sum(p)
                assert np.abs(got[t, h] - o).max() < 1e-12


def test_model_is_causal_and_tied_or_untied():
    for name in ("A", "B", "C"):
        cfg = helpers.TINY[name][0]
        m = P.PlainLlama(helpers.model_dir(name))
        ids = helpers.prompts(cfg["vocab_size"], [12], seed=4)[0]
        full = m.forward(ids)
        assert full.shape == (12, cfg["vocab_size"])
        assert np.abs(m.forward(ids[:7]) - full[:7]).max() < 1e-10
        other = list(ids)
        other[9] = (other[9] + 1) % cfg["vocab_size"]
        assert np.abs(m.forward(other)[:9] - full[:9]).max() < 1e-10
        assert np.abs(m.forward(other)[9:] - full[9:]).max() > 1e-6
        assert m.tied == cfg["tie_word_embeddings"]
        assert ("lm_head.weight" in m.w) == (not m.tied)


def test_greedy_keeps_the_stop_token():
    m = P.PlainLlama(helpers.model_dir("A"))
    out = m.greedy([1, 2, 3], 6)
    assert len(out) == 6
    stopped = m.greedy([1, 2, 3], 6, stop_ids=(out[2],))
    assert stopped == out[:out.index(out[2]) + 1]


def test_sampling_rules():
    rng = np.random.default_rng(3)
    logits = rng.normal(size=50) * 3
    assert P.sample(logits, 0.0, 1, 0) == int(np.argmax(logits))
    top2 = set(np.argsort(-logits)[:2].tolist())
    for c in range(20):                                   # crates/vllm-engine/src/sampling.rs:73-116
        assert P.sample(logits, 1.0, 7, c, top_k=1) == int(np.argmax(logits))
        assert P.sample(logits, 1.0, 7, c, top_k=2) in top2
    assert np.allclose(P.filtered_probs(logits, 0.7, top_k=80), P.filtered_probs(logits, 0.7))   # k >= V: no filter
    p = P.filtered_probs(logits, 1.0, top_p=0.6)
    full = P.filtered_probs(logits, 1.0)
    kept = np.where(p > 0)[0]
    assert full[kept].sum() >= 0.6 and full[kept].sum() - full[kept].min() < 0.6      # the smallest such set
    assert abs(p.sum() - 1) < 1e-12
    us = [P.uniform_from_counter(5, c) for c in range(2000)]
    assert 0 <= min(us) and max(us) < 1 and abs(np.mean(us) - 0.5) < 0.03
    assert us[:5] == [P.uniform_from_counter(5, c) for c in range(5)]
    assert P.uniform_from_counter(6, 0) != us[0]
    # the draws follow the distribution
    counts = np.bincount([P.sample(logits, 1.0, 11, c) for c in range(4000)], minlength=50) / 4000
    assert np.abs(counts - full).max() < 0.03
