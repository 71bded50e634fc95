"""Shared test fixtures: the two tiny configurations, model folders, traces."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import numpy as np

# Tiny configurations that differ in every size and option.  A and B have head sizes 16 and 32; C has the head
# size 64 (with more query features than the hidden size) that selects the tcgen05 attention kernel and the exact
# head-size specialisations of the other kernels.
TINY_A = dict(
    architectures=["LlamaForCausalLM"], hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, num_hidden_layers=2, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
    rope_scaling=None, tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=256)
TINY_B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=96, num_attention_heads=3, num_key_value_heads=1,
    head_dim=32, num_hidden_layers=3, intermediate_size=256, vocab_size=500, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=64),
    tie_word_embeddings=False, rms_norm_eps=1e-6, max_position_embeddings=512)
TINY_C = dict(
    architectures=["LlamaForCausalLM"], hidden_size=192, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, num_hidden_layers=2, intermediate_size=320, vocab_size=384, rope_theta=50000.0,
    rope_scaling=dict(rope_type="llama3", factor=4.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=128),
    tie_word_embeddings=True, rms_norm_eps=2e-5, max_position_embeddings=1024)
TINY = {"A": (TINY_A, 0, 16), "B": (TINY_B, 2, 8), "C": (TINY_C, 4, 16)}      # config, weight seed, page size

_made: dict = {}


def model_dir(name: str, std: float = 0.1) -> Path:
    """A model folder with random weights for TINY[name] (made once per process,
    in a temporary folder).  std 0.1 rather than 0.02 so that attention is far
    from uniform and a wrong key changes the logits visibly."""
    key = (name, std)
    if key not in _made:
        from railgun_b200.config.llama import LlamaConfig
        from railgun_b200.weights.random_init import write_random_model
        cfg, seed, _ = TINY[name]
        d = Path(tempfile.mkdtemp(prefix=f"rg_tiny_{name}_"))
        write_random_model(LlamaConfig.from_dict(cfg), seed, d, std=std)
        _made[key] = d
    return _made[key]


def prompts(vocab: int, lengths, seed: int):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, size=n).tolist() for n in lengths]


# ---- traces: lists of step records as bin/trace_run reads them ----------------------------

def trace_whole(reqs: dict) -> list:
    """Each request alone and whole, logits everywhere."""
    steps = []
    for i, (name, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": name, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [name]})
    return steps


def trace_tail_decode(reqs: dict, tail: int = 32) -> list:
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    steps, k = [], 0
    for name, toks in reqs.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": k, "entries": [{"id": name, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        k += 1
        for j in range(head, len(toks)):
            steps.append({"step": k, "entries": [{"id": name, "tokens": [toks[j]], "want": [0]}],
                          "end": [name] if j == len(toks) - 1 else []})
            k += 1
        if head == len(toks):
            steps[-1]["end"] = [name]
    return steps


def trace_portions(reqs: dict, sizes=(7, 2, 16, 3, 2, 5, 11, 2, 9)) -> list:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps, k = [], 0
    for name, toks in reqs.items():
        pos, i = 0, 0
        while pos < len(toks):
            n = min(sizes[i % len(sizes)], len(toks) - pos)
            steps.append({"step": k, "entries": [{"id": name, "tokens": toks[pos:pos + n],
                                                  "want": list(range(n))}],
                          "end": [name] if pos + n == len(toks) else []})
            pos += n
            i += 1
            k += 1
    return steps


def trace_mixed(reqs: dict, max_live: int = 4, seed: int = 0, sizes=(5, 1, 2, 9, 1, 1, 3, 17, 1, 2)) -> list:
    """Up to ``max_live`` requests at a time, portions of some beside single
    tokens of others; a request that ends frees its pages for the next one."""
    rng = np.random.default_rng(seed)
    waiting = list(reqs.items())
    live: dict = {}
    steps, k = [], 0
    while waiting or live:
        while waiting and len(live) < max_live:
            name, toks = waiting.pop(0)
            live[name] = [toks, 0]
        entries, ended = [], []
        for name in list(live):
            toks, pos = live[name]
            if len(live) > 1 and rng.random() < 0.2:
                continue                      # left out of this step, goes on later
            n = min(int(sizes[int(rng.integers(0, len(sizes)))]), len(toks) - pos)
            entries.append({"id": name, "tokens": toks[pos:pos + n], "want": list(range(n))})
            live[name][1] = pos + n
            if pos + n == len(toks):
                ended.append(name)
                del live[name]
        steps.append({"step": k, "entries": entries, "end": ended})
        k += 1
    return steps


def peak_tokens(steps: list, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: dict = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-v // round_to) * round_to for v in held.values()))
        for name in s["end"]:
            held.pop(name, None)
    return peak


def collect(steps: list, out_dir, vocab: int) -> dict:
    """(request, position) -> logits row, from the files a replay wrote."""
    pos: dict = {}
    rows: dict = {}
    for s in steps:
        wanted = []
        for e in s["entries"]:
            start = pos.get(e["id"], 0)
            wanted += [(e["id"], start + w) for w in e.get("want", [])]
            pos[e["id"]] = start + len(e["tokens"])
        for name in s["end"]:
            pos.pop(name, None)
        if wanted:
            arr = np.fromfile(Path(out_dir) / f"{s['step']}.f32", dtype="<f4").reshape(len(wanted), vocab)
            for key, row in zip(wanted, arr):
                rows[key] = row
    return rows
