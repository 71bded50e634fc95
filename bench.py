#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama 3.2 1B with random weights:
decode at batch 8 with 1,024 tokens of context per request (the headline
``value``, decoded tokens per second), the same through the Python entry point
with host tokens in and out (``e2e``), decode at batch 1 and 64 (``points``),
one 2,048-token prefill (``prefill``) and the decode step's memory roofline
(``roofline``).  One JSON line is printed.  A step is one decode step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_3_2_1B = dict(
    architectures=["LlamaForCausalLM"], hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
    head_dim=64, num_hidden_layers=16, intermediate_size=8192, vocab_size=128256, rope_theta=500000.0,
    rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                      original_max_position_embeddings=8192),
    tie_word_embeddings=True, rms_norm_eps=1e-5, max_position_embeddings=131072, torch_dtype="bfloat16")
CONTEXT = 1024            # tokens each decoding request holds
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)     # used only if MEASURED_PEAKS.json is absent


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            data = json.load(open(path))
            return dict(hbm_gbs=float(data["hbm_gbs"]), bf16_tflops=float(data["bf16_tflops"]),
                        bf16_tflops_sustained=float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.samples, self.proc = [], None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons}


def model_folder(cfg_dict, seed=0):
    """The model folder with random weights (written once per machine into the temporary folder)."""
    from railgun_b200.config.llama import LlamaConfig
    from railgun_b200.weights.random_init import write_random_model
    tag = f"rg_bench_L{cfg_dict['num_hidden_layers']}_H{cfg_dict['hidden_size']}_V{cfg_dict['vocab_size']}_s{seed}"
    d = os.path.join(tempfile.gettempdir(), tag)
    if not (os.path.exists(os.path.join(d, "model.safetensors")) and os.path.exists(os.path.join(d, "config.json"))):
        tmp = d + f".tmp{os.getpid()}"
        write_random_model(LlamaConfig.from_dict(cfg_dict), seed, tmp)
        if os.path.exists(d):
            import shutil
            shutil.rmtree(d, ignore_errors=True)
        os.replace(tmp, d)
    return d


def decode_bytes(cfg, batch, context, kv_bytes_per_token):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * d * H + nh * d * H + 3 * I * H + 2 * H
    weights = (L * per_layer + V * H + H) * 2              # the head's matrix once, tied or not
    embedding_rows = batch * H * 2                          # of the embedding table only the tokens' rows
    return weights + embedding_rows + batch * context * kv_bytes_per_token


def prefill_flops(cfg, T):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * T * L * ((nh + 2 * nkv) * d * H + nh * d * H + 3 * I * H)
    attn = L * nh * 2 * 2 * d * (T * (T + 1) // 2)          # causal: QK^T and PV
    return linear + attn + 2 * V * H


def run_ours(args):
    import numpy as np
    import torch
    from railgun_b200.engine.batch import StepEntry
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    from railgun_b200 import ops

    cfg = dict(LLAMA_3_2_1B)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk, pk_src = peaks()
    mdir = model_folder(cfg)
    page = 16
    pool_tokens = 64 * 8192                                # the cache pool: 64 sequences x 8,192 tokens
    eng = Engine(mdir, dtype="bfloat16", block_size=page, num_gpu_blocks=pool_tokens // page, max_num_seqs=64,
                 max_num_batched_tokens=8192, max_model_len=8192)
    runner = eng.runner
    V = cfg["vocab_size"]
    rng = np.random.default_rng(0)
    kv_per_token = runner.cache.bytes_per_token()
    launches = ops.launch_counter()

    def fill_contexts(batch, first_id, context=CONTEXT):
        """Prefill ``batch`` requests of ``context`` tokens each; returns their ids and first sampled tokens."""
        ids = list(range(first_id, first_id + batch))
        toks = []
        for rid in ids:
            prompt = rng.integers(0, V, size=context).tolist()
            lg = runner.step([StepEntry(rid, prompt, [context - 1])])
            toks.append(int(ops.argmax(lg).item()))
        return np.asarray(ids, dtype=np.int64), np.asarray(toks, dtype=np.int32)

    class DecodeLoop:
        """Decode steps for requests in the cache, launched as generation launches them (``Engine.step``): the
        first from host tokens, every later one while the one before it runs, its token ids staying on the
        device; but no step's tokens are read here.  ``log`` [n, rows] receives every step's tokens."""

        def __init__(self, ids, toks, log=None):
            self.ids, self.log, self.done, self.follow = ids, log, 0, None
            runner.decode_step_flat(ids, toks)
            self._note(runner.last_greedy)

        def _note(self, sampled):
            if self.log is not None:
                self.log[self.done, :len(self.ids)].copy_(sampled[:len(self.ids)])
            self.done += 1

        def run(self, n):
            for _ in range(n):
                nxt = runner.decode_follow(self.ids, self.follow)
                if nxt is None:
                    raise RuntimeError("the cache has no room for the timed decode steps")
                if self.follow is not None:
                    runner.alloc.advance(self.ids, 1)      # the step before is committed once its successor is packed
                self.follow = nxt
                self._note(nxt.static.sampled)

        def close(self):
            if self.follow is not None:
                runner.alloc.advance(self.ids, 1)
            torch.cuda.synchronize()

    def time_decode(batch, steps, warmup, first_id, context=CONTEXT, min_seconds=0.3):
        """Windows of exactly ``steps`` decode steps each, timed with CUDA events, until ``min_seconds`` are
        covered (three windows at least); before each window the requests go back to ``context`` tokens, so every
        window reads the same amount of cache.  Returns the median window."""
        ids, toks = fill_contexts(batch, first_id, context)
        back = np.full(batch, context, dtype=np.int32)
        windows, n_launch, total = [], 0, 0.0
        while len(windows) < 3 or (total < min_seconds and len(windows) < 200):
            runner.alloc.commit_many(ids, back)
            loop = DecodeLoop(ids, toks)
            loop.run(warmup - 1)
            torch.cuda.synchronize()
            n0 = launches.value
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            loop.run(steps)
            t1.record()
            torch.cuda.synchronize()
            loop.close()
            n_launch = launches.value - n0
            ms = t0.elapsed_time(t1)
            windows.append(ms / steps)
            total += ms * 1e-3
        runner.check_device_errors()
        runner.end(ids.tolist())
        ms = sorted(windows)[len(windows) // 2]
        return batch / ms * 1e3, ms, n_launch, len(windows)

    def hbm_frac(batch, ms, steps, warmup, context=CONTEXT):
        bytes_step = decode_bytes(cfg, batch, context + warmup + steps // 2, kv_per_token)
        achieved = bytes_step / (ms * 1e-3) / 1e9
        return achieved, achieved / pk["hbm_gbs"]

    def e2e_window(prompts, steps, warmup):
        """``steps`` calls of Engine.step with every request decoding: host tokens in, host tokens out."""
        rids = [eng.add_request(p, SamplingParams(max_new_tokens=steps + warmup + 2)) for p in prompts]
        tokens = {r: [] for r in rids}
        while True:                                        # until all prompts are in the cache
            out = eng.step()
            for r, t in out or ():
                tokens[r].append(t)
            if out is not None and len(out) == len(prompts):
                break
        for _ in range(warmup):
            for r, t in eng.step():
                tokens[r].append(t)
        torch.cuda.synchronize()
        w0 = time.perf_counter()
        for _ in range(steps):
            for r, t in eng.step():
                tokens[r].append(t)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - w0
        h2d = eng.runner.last_h2d_bytes
        for r in rids:
            eng.abort(r)
            eng.collect(r)
        return seconds * 1e3 / steps, h2d, [tokens[r] for r in rids]

    def check_tokens(prompts, n=24):
        """The timed loop against the entry point: the same prompts through Engine.step, token by token on the
        host, and through ``DecodeLoop`` after the same prefill; every token of every step must be equal."""
        _, _, by_engine = e2e_window(prompts, n - 1, 1)
        rids = [eng.add_request(p, SamplingParams(max_new_tokens=n + 2)) for p in prompts]
        while True:
            out = eng.step()
            if out is not None and len(out) == len(prompts):
                break
        first = dict(out)
        ids = np.asarray(rids, dtype=np.int64)
        log = torch.zeros((n, len(rids)), dtype=torch.int32, device=runner.device)
        loop = DecodeLoop(ids, np.asarray([first[r] for r in rids], dtype=np.int32), log)
        loop.run(n - 1)
        loop.close()
        by_loop = log.cpu().numpy()
        for r in rids:
            eng.abort(r)
            eng.collect(r)
        return all([first[r]] + by_loop[:, i].tolist() == by_engine[i][:n + 1] for i, r in enumerate(rids))

    if args.mode == "decode":                              # a short run of one decode batch (for profiling)
        tok_s, ms_step, n_launch, _ = time_decode(args.batch, args.steps, args.warmup, 1000, args.context,
                                                  min_seconds=0.0 if args.windows == 1 else 0.3)
        print(json.dumps({"mode": "decode", "batch": args.batch, "context": args.context, "tok_s": round(tok_s, 1),
                          "hbm_frac": round(hbm_frac(args.batch, ms_step, args.steps, args.warmup, args.context)[1], 4),
                          "ms_per_step": round(ms_step, 4), "gpu_launches": n_launch,
                          "layers": cfg["num_hidden_layers"]}))
        return 0
    if args.mode == "prefill":
        prompt = rng.integers(0, V, size=args.tokens).tolist()
        times = []
        for i in range(args.warmup + args.steps):
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            runner.step([StepEntry(7000 + i, prompt, [args.tokens - 1])])
            t1.record()
            torch.cuda.synchronize()
            runner.end([7000 + i])
            times.append(t0.elapsed_time(t1))
        ms = sorted(times[args.warmup:])[len(times[args.warmup:]) // 2]
        print(json.dumps({"mode": "prefill", "tokens": args.tokens, "ms": round(ms, 3),
                          "tok_s": round(args.tokens / ms * 1e3, 1), "layers": cfg["num_hidden_layers"],
                          "frac": round(prefill_flops(cfg, args.tokens) / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}))
        return 0

    prompts = [rng.integers(0, V, size=CONTEXT).tolist() for _ in range(8)]
    checked = bool(check_tokens(prompts))
    with ClockSampler() as clocks:
        tok_s, ms_step, n_launch, n_windows = time_decode(8, args.steps, args.warmup, 1000)
    clock_summary = clocks.summary()
    points = {}
    for b in (1, 64):
        b_tok_s, b_ms, _, _ = time_decode(b, args.steps, args.warmup, 2000 + 100 * b)
        points[f"decode_b{b}"] = round(b_tok_s, 1)
        points[f"decode_b{b}_ms_per_step"] = round(b_ms, 4)
        points[f"decode_b{b}_frac"] = round(hbm_frac(b, b_ms, args.steps, args.warmup)[1], 4)

    # prefill of 2,048 tokens, logits at the last position
    prompt = rng.integers(0, V, size=PREFILL_TOKENS).tolist()
    pf_ms = []
    for i in range(args.warmup + 9):
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        runner.step([StepEntry(5000 + i, prompt, [PREFILL_TOKENS - 1])])
        t1.record()
        torch.cuda.synchronize()
        runner.end([5000 + i])
        if i >= args.warmup:
            pf_ms.append(t0.elapsed_time(t1))
    runner.check_device_errors()
    pf = sorted(pf_ms)[len(pf_ms) // 2]
    flops = prefill_flops(cfg, PREFILL_TOKENS)

    # end to end through the entry point: host tokens in, host tokens out, every step; the median window
    e2e, seconds = [], 0.0
    while len(e2e) < 3 or (seconds < 0.3 and len(e2e) < 200):
        ms, h2d, _ = e2e_window(prompts, args.steps, args.warmup)
        e2e.append(ms)
        seconds += ms * args.steps * 1e-3
    e2e_ms = sorted(e2e)[len(e2e) // 2]
    d2h = 8 * 4

    achieved, frac = hbm_frac(8, ms_step, args.steps, args.warmup)
    line = {
        "metric": "decode tok/s at batch 8 (Llama 3.2 1B sizes, 1,024-token contexts)",
        "value": round(tok_s, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights and uniform random token ids",
        "impl": "ours", "checked": checked,
        "config": {
            "model": "Llama-3.2-1B sizes, random weights", "layers": cfg["num_hidden_layers"],
            "layers_of_named_config": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": 8,
            "seq_len": CONTEXT, "block_size": page, "kv_pool_tokens": pool_tokens, "parallelism": "none (1 GPU)",
            "l2": "inputs larger than L2 (2.5 GB of weights per step)", "peaks": pk_src,
            "timing": f"median of {n_windows} windows of {args.steps} steps",
        },
        "e2e": {"value": round(8 / e2e_ms * 1e3, 1), "unit": "tok/s", "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "frac": round(hbm_frac(8, e2e_ms, args.steps, args.warmup)[1], 4), "windows": len(e2e)},
        "gpu_launches": int(n_launch),
        "prefill": {"value": round(PREFILL_TOKENS / pf * 1e3, 1), "tokens": PREFILL_TOKENS, "ms": round(pf, 3),
                    "frac": round(flops / (pf * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(frac, 4)},
        "points": points,
        "clocks": clock_summary,
    }
    print(json.dumps(line))
    return 0


def run_kernels(args):
    """Times the hot kernels one by one, each as a CUDA graph of 16 calls over 16 different operand sets (so
    that weights and caches come from HBM, not L2), with CUDA events around replays.  One JSON line per case."""
    import torch
    from railgun_b200 import ops
    dev, L = "cuda:0", 16
    cfg = LLAMA_3_2_1B
    H, I, nh, nkv, d = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    QKV, page = (nh + 2 * nkv) * d, 16

    def timed(fn, reps=20):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(reps):
            g.replay()
        t1.record()
        torch.cuda.synchronize()
        ops.tc_gemm_check()
        return t0.elapsed_time(t1) / reps * 1e3 / L          # microseconds per call

    def weights(n, k):
        return [(torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16) for _ in range(L)]

    def out(case, us, **more):
        print(json.dumps(dict(case=case, us=round(us, 2), **more)), flush=True)

    want = set(args.cases.split(",")) if args.cases else None
    on = lambda name: want is None or name in want

    if on("decode_gemm"):
        for M in (1, 8):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            resid, nw = torch.randn(M, H, device=dev), torch.ones(H, device=dev)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                us = timed(lambda: [ops.skinny_gemm(inp, w, silu_mul=silu) for w in ws])
                us_lib = timed(lambda: [torch.mm(inp, w.t()) for w in ws])
                more = {}
                if name in ("o", "down"):
                    more["residual_epilogue_us"] = round(timed(lambda: [ops.skinny_gemm_residual(inp, w, resid, nw, 1e-5) for w in ws]), 2)
                else:
                    rows = ops.skinny_gemm_residual(x, weights(H, H)[0], resid, nw, 1e-5)
                    more["norm_finishing_us"] = round(timed(lambda: [ops.skinny_gemm_scaled(rows, w, silu_mul=silu) for w in ws]), 2)
                out(f"decode product {name} M{M} ({n} x {k})", us, GBs=round(n * k * 2 / us / 1e3, 1), cublas_us=round(us_lib, 2), **more)
    if on("decode_gemm_mid"):
        # decode batches of 17 to 64 rows: the swapped-operand tcgen05 product against the library
        for M in (32, 64):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                res = {}
                for sp in (0, 1, 2, 4, 8):
                    res[f"splits{sp}"] = round(timed(lambda: [ops.tc_stream_gemm(inp, w, silu_mul=silu, splits=sp) for w in ws]), 2)
                us_lib = timed(lambda: [ops.silu_mul(torch.mm(inp, w.t()), interleaved=True) if silu else torch.mm(inp, w.t()) for w in ws])
                out(f"decode product {name} M{M} ({n} x {k})", res["splits0"], GBs=round(n * k * 2 / res["splits0"] / 1e3, 1),
                    cublas_us=round(us_lib, 2), **res)
    if on("decode_attention"):
        for B, ctx in ((1, 1024), (8, 1024), (64, 1024), (8, 8192)):
            blocks = -(-ctx // page)
            kvs = [torch.randn(B * blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks).contiguous()
            q = torch.randn(B, QKV, device=dev).to(torch.bfloat16)
            o = torch.empty(B, nh * d, dtype=torch.bfloat16, device=dev)
            req = torch.arange(B, dtype=torch.int32, device=dev)
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
            splits = ops.decode_splits(B, nkv, ctx)
            us = timed(lambda: [ops.decode_attention(q, QKV, o, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, splits)
                                for kv in kvs])
            more = {}
            if 2 <= splits <= 8:     # beside the engine's way (a second kernel adds the splits): the splits as a cluster
                more["cluster_us"] = round(timed(lambda: [ops.decode_attention(
                    q, QKV, o, kv, bt, None, B, req, pos, nh, nkv, d, 0, d ** -0.5, splits, cluster=True) for kv in kvs]), 2)
            out(f"decode attention B{B} ctx{ctx} splits{splits}", us, GBs=round(B * ctx * nkv * d * 4 / us / 1e3, 1), **more)
    if on("sampling"):
        V = cfg["vocab_size"]
        for rows in (8, 64):
            logits = [torch.randn(rows, V, device=dev) * 9.0 for _ in range(L)]      # peaked rows, as a trained model's
            seed = torch.arange(rows, dtype=torch.int64, device=dev)
            counter = torch.zeros(rows, dtype=torch.int64, device=dev)
            res = {"argmax": round(timed(lambda: [ops.argmax(l) for l in logits]), 1)}
            for name, T, k, p in (("temperature", 0.8, 0, 1.0), ("top_k_50", 0.8, 50, 1.0), ("top_p_0.9", 0.8, 0, 0.9),
                                  ("top_k_50_top_p_0.9", 0.8, 50, 0.9), ("top_k_2000", 0.8, 2000, 1.0)):
                t = torch.full((rows,), T, device=dev)
                kk = torch.full((rows,), k, dtype=torch.int32, device=dev)
                pp = torch.full((rows,), p, device=dev)
                res[name] = round(timed(lambda: [ops.sample(l, t, kk, pp, seed, counter) for l in logits]), 1)
            out(f"sampling {rows} rows x {V} logits", res["temperature"], **res)
    if on("prefill_gemm"):
        for M in (2048, 8192):
            x = torch.randn(M, H, device=dev).to(torch.bfloat16)
            xi = torch.randn(M, I, device=dev).to(torch.bfloat16)
            for name, n, k, silu in (("qkv", QKV, H, False), ("o", H, H, False), ("gate_up", 2 * I, H, True), ("down", H, I, False)):
                ws = weights(n, k)
                inp = xi if k == I else x
                fl = 2 * M * n * k
                res = {}
                for tile in ops.TC_TILES:
                    us = timed(lambda: [ops.tc_gemm(inp, w, silu_mul=silu, tile=tile) for w in ws])
                    res[tile] = f"{us:.1f} us, {fl / us / 1e6:.0f} TFLOP/s"
                us_lib = timed(lambda: [ops.silu_mul(torch.mm(inp, w.t()), interleaved=True) if silu else torch.mm(inp, w.t()) for w in ws])
                out(f"prefill product {name} M{M} ({n} x {k})", us_lib, cublas_TFLOPs=round(fl / us_lib / 1e6), **res)
    if on("primitives"):
        # cycles of the building blocks of the tcgen05 kernels (per warp instruction and scheduler, per MMA, per wait)
        print(json.dumps({"case": "sm_100a primitives, cycles", **ops.probe_sm100(dev)}), flush=True)
    if on("prefill_attention"):
        for T in (2048, 8192):
            blocks = -(-T // page)
            kvs = [torch.randn(blocks, 2, nkv, page, d, device=dev).to(torch.bfloat16) for _ in range(L)]
            bt = torch.arange(blocks, dtype=torch.int32, device=dev).view(1, blocks).contiguous()
            q = torch.randn(T, QKV, device=dev).to(torch.bfloat16)
            o = torch.empty(T, nh * d, dtype=torch.bfloat16, device=dev)
            pos = torch.arange(T, dtype=torch.int32, device=dev)
            t128 = torch.tensor([(k, min(128, T - k), 0) for k in range(0, T, 128)], dtype=torch.int32, device=dev)
            t64 = torch.tensor([(k, min(64, T - k), 0) for k in range(0, T, 64)], dtype=torch.int32, device=dev)
            fl = nh * 4 * d * T * (T + 1) / 2
            us = timed(lambda: [ops.prefill_attention_tc(q, o, kv, bt, t128, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            us2 = timed(lambda: [ops.prefill_attention(q, QKV, o, kv, bt, t64, pos, nh, nkv, d, 0, d ** -0.5) for kv in kvs])
            out(f"prefill attention T{T} tcgen05", us, TFLOPs=round(fl / us / 1e6, 1), mma_sync_us=round(us2, 2))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the named configuration (0: all)")
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill", "kernels"],
                    help="all: the contract's line; decode / prefill: one short measurement (for profiling); "
                         "kernels: the hot kernels one by one")
    ap.add_argument("--cases", default="", help="--mode kernels: comma-separated subset of sampling, decode_gemm, "
                    "decode_gemm_mid, decode_attention, prefill_gemm, prefill_attention, primitives")
    ap.add_argument("--batch", type=int, default=8, help="--mode decode: requests in the batch")
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS, help="--mode prefill: prompt length")
    ap.add_argument("--context", type=int, default=CONTEXT, help="--mode decode: tokens each request holds")
    ap.add_argument("--windows", type=int, default=0, help="--mode decode: 1 times three windows only (for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust workspace on the candle crates: pip finds neither setup.py nor "
                          "pyproject.toml, and cargo/rustc are not installed"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.mode == "kernels":
        return run_kernels(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
