"""Choosing the next token from 32-bit logits: greedy, temperature, top-k, top-p.

Greedy is argmax, ties to the lowest index
(crates/vllm-models/src/llama/model.rs:210-218); temperature 0 means greedy
(crates/vllm-scheduler/src/request.rs:42-46); top-k keeps logits >= the k-th
largest (crates/vllm-engine/src/sampling.rs:50-62); top-p keeps the smallest
set of tokens whose probability reaches top_p.  The random number of a draw
depends only on the request's seed and on how many tokens it has generated,
so a request gets the same tokens alone, in any batch, and after preemption.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample(self, logits: torch.Tensor, params: list, counters: list) -> np.ndarray:
        """One token per logits row; ``params[i]`` is row i's SamplingParams and
        ``counters[i]`` the number of tokens its request has generated so far.
        Returns int32 token ids on the host."""
        rows = logits.shape[0]
        if rows != len(params) or rows != len(counters):
            raise ValueError(f"{rows} rows of logits for {len(params)} parameter sets")
        return self.sample_arrays(logits, dict(
            temperature=np.array([p.temperature for p in params], dtype=np.float32),
            top_k=np.array([p.top_k for p in params], dtype=np.int32),
            top_p=np.array([p.top_p for p in params], dtype=np.float32),
            seed=np.array([_as_i64(p.seed) for p in params], dtype=np.int64),
            counter=np.array([int(c) for c in counters], dtype=np.int64)))

    def sample_arrays(self, logits: torch.Tensor, sp: dict) -> np.ndarray:
        """The same from arrays of one entry per row: ``temperature`` float32, ``top_k`` int32, ``top_p``
        float32, ``seed`` int64 (the bits of an unsigned seed), ``counter`` int64 (the number of the draw)."""
        rows = logits.shape[0]
        if any(len(sp[k]) != rows for k in ("temperature", "top_k", "top_p", "seed", "counter")):
            raise ValueError(f"{rows} rows of logits, but the parameter arrays have other lengths")
        if not (sp["temperature"] != 0.0).any():
            return ops.argmax(logits).cpu().numpy()
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(self.device, non_blocking=True)
        out = ops.sample(logits, dev(sp["temperature"]), dev(sp["top_k"]), dev(sp["top_p"]), dev(sp["seed"]),
                         dev(sp["counter"]))
        return out.cpu().numpy()


def _as_i64(seed: int) -> int:
    """An unsigned 64-bit seed stored in a signed 64-bit tensor (same bits)."""
    seed &= (1 << 64) - 1
    return seed - (1 << 64) if seed >= (1 << 63) else seed
