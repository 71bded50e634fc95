"""Block arrangements: how a layer's parts sit around the residual stream.

"prenorm": x = x + mixer(norm(x)); x = x + ffn(norm(x))
(crates/vllm-models/src/llama/architecture.rs:47-58).  Each addition is done
inside the next norm's kernel, in 32-bit; at small decode batches the
addition moves into the kernel of the product before it and the norm into the
kernel of the product after it (ops.PendingLinear, ops.NormedRows).
"""
from __future__ import annotations

from .base import Arrangement, normed_input
from .registry import register_arrangement


class PreNorm(Arrangement):
    def run(self, layer, stream, batch, cache, writes):
        h = normed_input(layer.mixer_norm, layer.mixer, stream)
        if getattr(layer.mixer, "defers_output", False):
            stream.pending = layer.mixer.forward(h, batch, cache, writes, defer=True)
        else:
            stream.pending = layer.mixer.forward(h, batch, cache, writes)
        h = normed_input(layer.ffn_norm, layer.ffn, stream)
        if getattr(layer.ffn, "defers_output", False):
            stream.pending = layer.ffn.forward(h, batch, defer=True)
        else:
            stream.pending = layer.ffn.forward(h, batch)


register_arrangement("prenorm", PreNorm)
