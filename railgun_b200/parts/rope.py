"""Rotary position encoding with the optional "llama3" frequency scaling.

inv_freq_i = theta^(-2i/d); with rope_scaling of type llama3 (factor f,
low_freq_factor a, high_freq_factor b, original length P): wavelengths below
P/b are kept, above P/a divided by f, between them blended linearly in
P/wavelength.  Angles are position * inv_freq, computed in 64-bit on the host
and stored as a 32-bit table [max_position, d] = cos | sin, the layout of the
reference's kernel (crates/vllm-cuda/src/kernels/rope.cu:8,30-41), indexed by
absolute position, so a token is rotated the same way however the work is cut.
The reference never builds the table nor calls the kernel
(crates/vllm-cuda/src/kernels/paged_attn_op.rs:236 has no caller) and cannot
read rope_scaling (crates/vllm-models/src/llama/model.rs:49).
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding
from .registry import register_position_encoding


def rope_inverse_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    i = torch.arange(0, head_dim, 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (i / head_dim))
    if not scaling:
        return inv
    f = float(scaling["factor"])
    a = float(scaling["low_freq_factor"])
    b = float(scaling["high_freq_factor"])
    P = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (P / wavelen - a) / (b - a)
    blended = (1.0 - smooth) * inv / f + smooth * inv
    out = torch.where(wavelen > P / a, inv / f, blended)
    out = torch.where(wavelen < P / b, inv, out)
    return out


def rope_table(head_dim: int, theta: float, scaling: dict | None, max_position: int) -> torch.Tensor:
    inv = rope_inverse_frequencies(head_dim, theta, scaling)
    ang = torch.arange(max_position, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).to(torch.float32)


class RotaryEncoding(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``scaling`` (dict or None), ``max_position``."""

    def __init__(self, params, prefix, env, tensors):
        super().__init__(params, prefix, env, tensors)
        if params["head_dim"] % 2:
            raise ValueError(f"rotary encoding needs an even head size, got {params['head_dim']}")
        self.table = rope_table(params["head_dim"], params["theta"], params.get("scaling"),
                                params["max_position"]).to(env.device)

    @property
    def rotary_table(self):
        """[max_position, d] = cos | sin: lets a mixer rotate inside its own kernels."""
        return self.table

    def apply(self, qkv, batch, nh, nkv, d, kv_dest, paired8: bool = False) -> bool:
        kv, slots = kv_dest if kv_dest is not None else (None, None)
        page_size = kv.shape[3] if kv is not None else 1
        ops.rope_cache_write(qkv, self.table, batch.positions, slots, kv, nh, nkv, d, page_size, batch.err_flag,
                             paired8=paired8)
        return kv is not None


register_position_encoding("rope", RotaryEncoding)
