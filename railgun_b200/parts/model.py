"""A decoder model put together from a ``ModelSpec``.

Embedding, then the layers in the order the schedule lists, then the final
norm and the head on the rows whose logits are wanted
(crates/vllm-models/src/llama/architecture.rs:141-156 is the reference's
packed forward).  The class knows no architecture: it reads the spec.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import CacheView, Stream, normed_input
from .registry import ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS
from .spec import BuildEnv, ModelSpec
# importing the modules registers the built-in parts
from . import attention as _attention, block as _block, embedding as _embedding  # noqa: F401
from . import mlp as _mlp, norm as _norm, rope as _rope  # noqa: F401


def expected_tensors(spec: ModelSpec) -> dict:
    """Every tensor the model reads: name -> TensorSpec."""
    out = {}
    out.update(EMBEDDINGS.get(spec.embedding.kind).tensor_specs(spec.embedding.params, ""))
    for layer in spec.layers:
        for reg, part in ((NORMS, layer.mixer_norm), (MIXERS, layer.mixer),
                          (NORMS, layer.ffn_norm), (FEED_FORWARDS, layer.ffn)):
            out.update(reg.get(part.kind).tensor_specs(part.params, layer.prefix))
    out.update(NORMS.get(spec.final_norm.kind).tensor_specs(spec.final_norm.params, ""))
    out.update(HEADS.get(spec.head.kind).tensor_specs(spec.head.params, ""))
    return out


class TensorBank:
    """The loaded tensors, handed to parts.  ``get(name, dtype)`` returns the
    tensor cast to ``dtype`` (memoised, so tied tensors are shared);
    ``shared_part`` memoises whole parts (one rotary table for all layers)."""

    def __init__(self, tensors: dict, device):
        self._raw = dict(tensors)
        self._cast: dict = {}
        self._parts: dict = {}
        self.device = device

    def has(self, name: str) -> bool:
        return name in self._raw

    def get(self, name: str, dtype=None):
        t = self._raw[name]
        key = (name, dtype or t.dtype)
        if key not in self._cast:
            self._cast[key] = t.to(device=self.device, dtype=key[1])
        return self._cast[key]

    def drop(self, *names):
        for n in names:
            self._raw.pop(n, None)
            for key in [k for k in self._cast if k[0] == n]:
                del self._cast[key]

    def shared_part(self, key, factory):
        if key not in self._parts:
            self._parts[key] = factory()
        return self._parts[key]


@dataclass
class Layer:
    mixer_norm: object
    mixer: object
    ffn_norm: object
    ffn: object
    arrangement: object


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv, tensors: TensorBank):
        self.spec = spec
        self.env = env
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, "", env, tensors)
        self.layers = []
        for ls in spec.layers:
            self.layers.append(Layer(
                mixer_norm=NORMS.get(ls.mixer_norm.kind)(ls.mixer_norm.params, ls.prefix, env, tensors),
                mixer=MIXERS.get(ls.mixer.kind)(ls.mixer.params, ls.prefix, env, tensors),
                ffn_norm=NORMS.get(ls.ffn_norm.kind)(ls.ffn_norm.params, ls.prefix, env, tensors),
                ffn=FEED_FORWARDS.get(ls.ffn.kind)(ls.ffn.params, ls.prefix, env, tensors),
                arrangement=ARRANGEMENTS.get(ls.arrangement)(),
            ))
        self.final_norm = NORMS.get(spec.final_norm.kind)(spec.final_norm.params, "", env, tensors)
        self.head = HEADS.get(spec.head.kind)(spec.head.params, "", env, tensors)
        self.order = spec.run_order()
        seen_writer = set()
        for e in self.order:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}; the model has {len(self.layers)}")
            if e.writes:
                if e.cache in seen_writer:
                    raise ValueError(f"cache {e.cache} is written by two schedule entries")
                seen_writer.add(e.cache)
            elif e.cache not in seen_writer:
                raise ValueError(f"schedule entry reads cache {e.cache} before anything wrote it")

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def parts(self):
        yield self.embedding
        for layer in self.layers:
            yield from (layer.mixer_norm, layer.mixer, layer.ffn_norm, layer.ffn)
        yield self.final_norm
        yield self.head

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph: every part says so."""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def cache_needs(self) -> dict:
        """cache id -> what the writing layer's mixer keeps between steps."""
        needs = {}
        for e in self.order:
            if e.writes:
                ls = self.spec.layers[e.layer]
                needs[e.cache] = MIXERS.get(ls.mixer.kind).cache_need(ls.mixer.params)
        for e in self.order:
            if not e.writes:
                ls = self.spec.layers[e.layer]
                need = MIXERS.get(ls.mixer.kind).cache_need(ls.mixer.params)
                if need != needs[e.cache]:
                    raise ValueError(f"layer {e.layer} reads cache {e.cache} whose geometry {needs[e.cache]} "
                                     f"differs from its own {need}")
        return needs

    def forward(self, batch, cache):
        """Run the step's tokens; return float32 logits [wanted rows, vocab] or None."""
        stream = Stream(self.embedding.embed(batch.token_ids))
        for e in self.order:
            layer = self.layers[e.layer]
            layer.arrangement.run(layer, stream, batch, cache.view(e.cache), e.writes)
        if batch.num_wanted == 0:
            return None
        h = normed_input(self.final_norm, None, stream, rows=batch.want_rows)
        return self.head.logits(h)
