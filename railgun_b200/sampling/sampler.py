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
        if all(p.temperature == 0.0 for p in params):
            return ops.argmax(logits).cpu().numpy()
        temperature = torch.tensor([p.temperature for p in params], dtype=torch.float32)
        top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32)
        top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32)
        seed = torch.tensor([_as_i64(p.seed) for p in params], dtype=torch.int64)
        counter = torch.tensor([int(c) for c in counters], dtype=torch.int64)
        dev = lambda t: t.to(self.device, non_blocking=True)
        out = ops.sample(logits, dev(temperature), dev(top_k), dev(top_p), dev(seed), dev(counter))
        return out.cpu().numpy()


def _as_i64(seed: int) -> int:
    """An unsigned 64-bit seed stored in a signed 64-bit tensor (same bits)."""
    seed &= (1 << 64) - 1
    return seed - (1 << 64) if seed >= (1 << 63) else seed
