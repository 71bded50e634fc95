"""Block arrangements: how a layer's parts sit around the residual stream.

"prenorm": x = x + mixer(norm(x)); x = x + ffn(norm(x))
(crates/vllm-models/src/llama/architecture.rs:47-58).  Each addition is done
inside the next norm's kernel, in 32-bit.
"""
from __future__ import annotations

from .base import Arrangement
from .registry import register_arrangement


class PreNorm(Arrangement):
    def run(self, layer, stream, batch, cache, writes):
        h = layer.mixer_norm.add_norm(stream.resid, stream.pending)
        stream.pending = layer.mixer.forward(h, batch, cache, writes)
        h = layer.ffn_norm.add_norm(stream.resid, stream.pending)
        stream.pending = layer.ffn.forward(h, batch)


register_arrangement("prenorm", PreNorm)
