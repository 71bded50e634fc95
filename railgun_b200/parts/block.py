"""Block arrangements: how a layer's parts sit around the residual stream.

"prenorm": for every branch of the layer in turn, x = x + part(norm(x)); the
usual block is x = x + mixer(norm(x)); x = x + ffn(norm(x))
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
        for b in layer.branches:
            h = normed_input(b.norm, b.part, stream)
            more = dict(defer=True) if getattr(b.part, "defers_output", False) else {}
            if b.role == "mixer":
                stream.pending = b.part.forward(h, batch, cache, writes, **more)
            else:
                stream.pending = b.part.forward(h, batch, **more)


register_arrangement("prenorm", PreNorm)
