"""Plain, slow implementation of the dense GQA Llama decoder, used only by tests.

It rests on the formulas, not on the reference's output: the reference's model
code is Rust on the candle crates and can neither be imported nor compiled
where these tests run, and its forward pass leaves out the rotary embedding
(crates/vllm-cuda/src/kernels/paged_attn_op.rs:236 has no call site), so the
formulas below are the architecture's own, with the reference cited for the
order of operations, tensor names and conventions.

Three of the reference's CUDA kernels do compile as host C++ through a small
stand-in header; ``tests/golden/make_reference_kernel_golden.py`` ran them once
and ``tests/test_golden.py`` holds ``attention`` and ``rope`` below against
their stored outputs (cache layout, head grouping, softmax-weighted values for
a single query, rotation of pairs (i, i + d/2)).  Everything else (RMSNorm with
eps inside the root, SiLU and the gated feed-forward, the llama3 frequency
scaling, the causal mask inside a prompt, head grouping in a whole model, the
tied or untied head) rests on the formulas alone; for those the whole model is
stated a second time, independently, as scalar loops in C++
(``tests/ref/llama_scalar.cpp``), and ``tests/test_plain_twin.py`` holds the two
statements' logits together.  Model code of installed packages is not used as
a source for either.

Whole sequences, no cache, float64 arithmetic, one function per part.  It
shares no code with ``railgun_b200``: it reads config.json and
model.safetensors itself.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np

# --------------------------------------------------------------------------
# reading a model folder (own reader; the product's loader is not used)
# --------------------------------------------------------------------------


def _bf16_to_f64(raw: np.ndarray) -> np.ndarray:
    u32 = raw.astype(np.uint32) << 16
    return u32.view(np.float32).astype(np.float64)


def read_safetensors(path) -> dict[str, np.ndarray]:
    """name -> float64 / int64 array.  Layout: u64 little-endian header length,
    JSON header {name: {dtype, shape, data_offsets}}, then the bytes."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8:8 + hlen])
    data = blob[8 + hlen:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = data[lo:hi]
        dt = meta["dtype"]
        if dt == "BF16":
            arr = _bf16_to_f64(np.frombuffer(buf, dtype=np.uint16))
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype=np.float16).astype(np.float64)
        elif dt == "F32":
            arr = np.frombuffer(buf, dtype=np.float32).astype(np.float64)
        elif dt in ("I32", "I64"):
            arr = np.frombuffer(buf, dtype=np.int32 if dt == "I32" else np.int64).astype(np.int64)
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(meta["shape"])
    return out


def read_model(model_dir):
    model_dir = Path(model_dir)
    cfg = json.loads((model_dir / "config.json").read_text())
    weights = read_safetensors(model_dir / "model.safetensors")
    return cfg, weights


def round_bf16(x: np.ndarray) -> np.ndarray:
    """Round float64 values to the nearest bfloat16 (ties to even), as float64."""
    f = np.asarray(x, dtype=np.float32)
    u = f.view(np.uint32).astype(np.uint64)
    bias = ((u >> 16) & 1) + 0x7FFF
    u = ((u + bias) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(x))


# --------------------------------------------------------------------------
# the parts, one function each
# --------------------------------------------------------------------------


def embedding(table: np.ndarray, ids) -> np.ndarray:
    """x = embed_tokens[input_ids], no scaling
    (crates/vllm-models/src/llama/architecture.rs:150)."""
    return table[np.asarray(ids, dtype=np.int64)]


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """y = w * x / sqrt(mean(x^2) + eps), eps inside the root.  The reference
    builds it with candle_nn::rms_norm(H, eps)
    (crates/vllm-models/src/llama/architecture.rs:27-28,108); eps default 1e-5
    (crates/vllm-models/src/config.rs:66-68)."""
    ms = np.mean(x * x, axis=-1, keepdims=True)
    return x / np.sqrt(ms + eps) * w


def linear(x: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y = x W^T with W stored [out, in], no bias
    (crates/vllm-models/src/llama/attention.rs:94-96,133)."""
    return x @ w.T


def rope_inv_freq(head_dim: int, theta: float, scaling: dict | None) -> np.ndarray:
    """inv_freq_i = theta^(-2i/d), i < d/2; rope_theta default 10000
    (crates/vllm-models/src/config.rs:63-65).  With rope_scaling of type
    "llama3" (factor f, low_freq_factor a, high_freq_factor b, original length
    P): wavelengths below P/b are kept, above P/a divided by f, and between
    them blended linearly in P/wavelength.  The reference cannot read the key
    (crates/vllm-models/src/llama/model.rs:49 sets it to None), so this rule is
    the architecture's published one."""
    i = np.arange(0, head_dim, 2, dtype=np.float64)
    inv = 1.0 / (float(theta) ** (i / head_dim))
    if not scaling:
        return inv
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind in (None, "default"):
        return inv
    if kind != "llama3":
        raise ValueError(f"plain rope: unknown rope_type {kind!r}")
    f = float(scaling["factor"])
    a = float(scaling["low_freq_factor"])
    b = float(scaling["high_freq_factor"])
    P = float(scaling["original_max_position_embeddings"])
    out = np.empty_like(inv)
    for k, v in enumerate(inv):
        wavelen = 2.0 * math.pi / v
        if wavelen < P / b:
            out[k] = v
        elif wavelen > P / a:
            out[k] = v / f
        else:
            s = (P / wavelen - a) / (b - a)
            out[k] = (1.0 - s) * v / f + s * v
    return out


def rope(x: np.ndarray, positions, inv_freq: np.ndarray) -> np.ndarray:
    """Rotate pairs (i, i + d/2) of every head by angle pos * inv_freq_i:
    x'[i] = x[i] c - x[i+d/2] s ; x'[i+d/2] = x[i+d/2] c + x[i] s
    (crates/vllm-cuda/src/kernels/rope.cu:30-41).  x is [T, heads, d]."""
    pos = np.asarray(positions, dtype=np.float64)
    ang = pos[:, None] * inv_freq[None, :]              # [T, d/2]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    return np.concatenate([lo * c - hi * s, hi * c + lo * s], axis=-1)


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, positions,
              window: int | None = None, scale: float | None = None) -> np.ndarray:
    """Causal grouped-query attention over one whole sequence.
    q [T, nh, d]; k, v [T, nkv, d].  kv_head = head // (nh / nkv)
    (crates/vllm-cuda/src/kernels/paged_attention.cu:40); score =
    scale * q.k with scale = d^-0.5 (crates/vllm-models/src/llama/attention.rs:69);
    softmax over the keys at positions <= the query's (and, with a window w,
    > position - w); out = sum p v / sum p
    (crates/vllm-cuda/src/kernels/paged_attention.cu:66-69,103-107)."""
    T, nh, d = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    if scale is None:
        scale = d ** -0.5
    pos = np.asarray(positions, dtype=np.int64)
    allowed = pos[None, :] <= pos[:, None]
    if window:
        allowed &= pos[None, :] > pos[:, None] - window
    out = np.zeros_like(q)
    for h in range(nh):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].T) * scale        # [T, T]
        s = np.where(allowed, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        out[:, h, :] = (p @ v[:, kh, :]) / p.sum(axis=-1, keepdims=True)
    return out


def silu(x: np.ndarray) -> np.ndarray:
    return x / (1.0 + np.exp(-x))


def swiglu(x: np.ndarray, w_gate, w_up, w_down) -> np.ndarray:
    """down(silu(gate(x)) * up(x))
    (crates/vllm-models/src/llama/architecture.rs:81-85)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------


class PlainLlama:
    """Whole-sequence forward of LlamaForCausalLM from a model folder.

    Order of operations per layer: x + attn(norm(x)), then x + mlp(norm(x))
    (crates/vllm-models/src/llama/architecture.rs:47-58); final norm and
    lm_head, which is the embedding matrix when tied (:110-118,154-155).
    ``schedule`` optionally lists (layer, cache_of, writes) triples: the order
    layers run in, whose keys and values each one reads, and whether it adds
    its own; by default every layer once, on its own keys."""

    def __init__(self, model_dir, act_rounding=None, schedule=None, window=None):
        self.cfg, self.w = read_model(model_dir)
        c = self.cfg
        self.H = c["hidden_size"]
        self.nh = c["num_attention_heads"]
        self.nkv = c.get("num_key_value_heads", self.nh)
        self.d = c.get("head_dim") or self.H // self.nh
        self.L = c["num_hidden_layers"]
        self.eps = c.get("rms_norm_eps", 1e-5)
        self.inv_freq = rope_inv_freq(self.d, c.get("rope_theta", 10000.0), c.get("rope_scaling"))
        self.tied = bool(c.get("tie_word_embeddings", False))
        self.schedule = schedule or [(i, i, True) for i in range(self.L)]
        self.window = window

    def layer_weights(self, i):
        p = f"model.layers.{i}."
        w = self.w
        return dict(
            ln1=w[p + "input_layernorm.weight"], ln2=w[p + "post_attention_layernorm.weight"],
            q=w[p + "self_attn.q_proj.weight"], k=w[p + "self_attn.k_proj.weight"],
            v=w[p + "self_attn.v_proj.weight"], o=w[p + "self_attn.o_proj.weight"],
            gate=w[p + "mlp.gate_proj.weight"], up=w[p + "mlp.up_proj.weight"],
            down=w[p + "mlp.down_proj.weight"])

    def forward(self, ids, start_pos: int = 0) -> np.ndarray:
        """Logits [T, V] (float64) of one sequence, every position."""
        T = len(ids)
        pos = np.arange(start_pos, start_pos + T)
        x = embedding(self.w["model.embed_tokens.weight"], ids)
        kv = {}
        for (li, cache_of, writes) in self.schedule:
            lw = self.layer_weights(li)
            h = rms_norm(x, lw["ln1"], self.eps)
            q = rope(linear(h, lw["q"]).reshape(T, self.nh, self.d), pos, self.inv_freq)
            if writes:
                k = rope(linear(h, lw["k"]).reshape(T, self.nkv, self.d), pos, self.inv_freq)
                v = linear(h, lw["v"]).reshape(T, self.nkv, self.d)
                kv[cache_of] = (k, v)
            k, v = kv[cache_of]
            a = attention(q, k, v, pos, window=self.window).reshape(T, self.nh * self.d)
            x = x + linear(a, lw["o"])
            h = rms_norm(x, lw["ln2"], self.eps)
            x = x + swiglu(h, lw["gate"], lw["up"], lw["down"])
        x = rms_norm(x, self.w["model.norm.weight"], self.eps)
        head = self.w["model.embed_tokens.weight"] if self.tied else self.w["lm_head.weight"]
        return linear(x, head)

    def greedy(self, prompt, n_new: int, stop_ids=()) -> list[int]:
        """Greedy continuation, recomputing the whole sequence for each token,
        as crates/vllm-models/src/llama/model.rs:221-243 does; ties go to the
        lowest index.  A stop token is kept in the output and ends it
        (crates/vllm-scheduler/src/request.rs:180-192)."""
        ids = list(prompt)
        out = []
        for _ in range(n_new):
            tok = int(np.argmax(self.forward(ids)[-1]))
            out.append(tok)
            ids.append(tok)
            if tok in stop_ids:
                break
        return out


# --------------------------------------------------------------------------
# sampling
# --------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


def uniform_from_counter(seed: int, counter: int) -> float:
    """The engine's counter-based generator, restated: splitmix64 of
    seed + (counter + 1) * golden-ratio constant, top 24 bits -> [0, 1)."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def filtered_probs(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0) -> np.ndarray:
    """softmax(logits / T) restricted by top-k, then top-p.  top-k keeps every
    logit >= the k-th largest, ties kept, k >= V is no filter
    (crates/vllm-engine/src/sampling.rs:50-62).  top-p keeps the probabilities
    >= t, t being the largest value whose kept mass reaches top_p (the
    smallest set whose mass reaches top_p, ties kept;
    crates/vllm-scheduler/src/request.rs:49-53)."""
    z = np.asarray(logits, dtype=np.float64) / temperature
    if top_k and top_k < z.size:
        thr = np.sort(z)[-top_k]
        z = np.where(z >= thr, z, -np.inf)
    p = np.exp(z - z.max())
    p = p / p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        csum = np.cumsum(p[order])
        n_keep = int(np.searchsorted(csum, top_p, side="left")) + 1
        t = p[order[min(n_keep, p.size) - 1]]
        p = np.where(p >= t, p, 0.0)
        p = p / p.sum()
    return p


def sample(logits: np.ndarray, temperature: float, seed: int, counter: int,
           top_k: int = 0, top_p: float = 1.0) -> int:
    """temperature 0 is greedy (crates/vllm-scheduler/src/request.rs:42-46);
    otherwise the first index whose cumulative probability exceeds u."""
    if temperature == 0.0:
        return int(np.argmax(logits))
    p = filtered_probs(logits, temperature, top_k, top_p)
    u = uniform_from_counter(seed, counter)
    c = np.cumsum(p)
    idx = int(np.searchsorted(c, u * c[-1], side="right"))
    return min(idx, p.size - 1)
