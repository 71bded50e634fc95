"""Registries of part kinds: mixers, feed-forwards, norms, position encodings,
block arrangements, embeddings and heads.

Adding a part is ``register_mixer("name", Class)`` (and so on) from any
module; a ``PartSpec(kind="name", ...)`` in a model description then builds it.
The reference keeps one registry, from architecture name to model factory
(crates/vllm-models/src/registry.rs:90-154); parts there are fixed Rust types.
"""
from __future__ import annotations


class PartRegistry:
    def __init__(self, what: str):
        self.what = what
        self._kinds: dict = {}

    def register(self, kind: str, cls, replace: bool = False):
        if kind in self._kinds and not replace and self._kinds[kind] is not cls:
            raise ValueError(f"{self.what} kind {kind!r} is already registered")
        self._kinds[kind] = cls
        return cls

    def unregister(self, kind: str):
        self._kinds.pop(kind, None)

    def get(self, kind: str):
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"unknown {self.what} kind {kind!r}; known: {sorted(self._kinds)}") from None

    def kinds(self):
        return sorted(self._kinds)


MIXERS = PartRegistry("mixer")
FEED_FORWARDS = PartRegistry("feed-forward")
NORMS = PartRegistry("norm")
POSITION_ENCODINGS = PartRegistry("position encoding")
ARRANGEMENTS = PartRegistry("block arrangement")
EMBEDDINGS = PartRegistry("embedding")
HEADS = PartRegistry("head")

register_mixer = MIXERS.register
register_feed_forward = FEED_FORWARDS.register
register_norm = NORMS.register
register_position_encoding = POSITION_ENCODINGS.register
register_arrangement = ARRANGEMENTS.register
register_embedding = EMBEDDINGS.register
register_head = HEADS.register
