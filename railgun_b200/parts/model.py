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


def _part_registry(role: str):
    return MIXERS if role == "mixer" else FEED_FORWARDS


def expected_tensors(spec: ModelSpec) -> dict:
    """Every tensor the model reads: name -> TensorSpec."""
    out = {}
    out.update(EMBEDDINGS.get(spec.embedding.kind).tensor_specs(spec.embedding.params, ""))
    for layer in spec.layers:
        for b in layer.branches():
            out.update(NORMS.get(b.norm.kind).tensor_specs(b.norm.params, layer.prefix))
            out.update(_part_registry(b.role).get(b.part.kind).tensor_specs(b.part.params, layer.prefix))
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
class Branch:
    norm: object
    part: object
    role: str                       # "mixer" or "ffn"


@dataclass
class Layer:
    """A built block: its branches in order, and how they are wired."""
    branches: list
    arrangement: object

    def _first(self, role, what):
        for b in self.branches:
            if b.role == role:
                return getattr(b, what)
        return None

    # the usual block's parts by name
    mixer = property(lambda self: self._first("mixer", "part"))
    mixer_norm = property(lambda self: self._first("mixer", "norm"))
    ffn = property(lambda self: self._first("ffn", "part"))
    ffn_norm = property(lambda self: self._first("ffn", "norm"))


class DecoderModel:
    def __init__(self, spec: ModelSpec, env: BuildEnv, tensors: TensorBank):
        self.spec = spec
        self.env = env
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(spec.embedding.params, "", env, tensors)
        self.layers = []
        for ls in spec.layers:
            self.layers.append(Layer(
                branches=[Branch(NORMS.get(b.norm.kind)(b.norm.params, ls.prefix, env, tensors),
                                 _part_registry(b.role).get(b.part.kind)(b.part.params, ls.prefix, env, tensors),
                                 b.role) for b in ls.branches()],
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
            for b in layer.branches:
                yield b.norm
                yield b.part
        yield self.final_norm
        yield self.head

    @property
    def graph_safe(self) -> bool:
        """Whether a step of this model can be captured in a CUDA graph: every part says so."""
        return all(getattr(p, "graph_safe", True) for p in self.parts())

    def cache_needs(self) -> dict:
        """cache id -> what the writing layer's mixer keeps between steps."""
        def need_of(layer_index):
            """What the layer's mixers keep between steps: a schedule entry names one cache, so one of them at most."""
            found = [n for n in (MIXERS.get(b.part.kind).cache_need(b.part.params)
                                 for b in self.spec.layers[layer_index].branches() if b.role == "mixer") if n is not None]
            if len(found) > 1:
                raise ValueError(f"layer {layer_index} has {len(found)} mixers that keep something between steps; "
                                 "a layer's schedule entry names one cache")
            return found[0] if found else None

        needs = {}
        for e in self.order:
            if e.writes:
                needs[e.cache] = need_of(e.layer)
        for e in self.order:
            if not e.writes:
                need = need_of(e.layer)
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
