"""Descriptions of a model as data: which parts, with which sizes, in which order.

An architecture turns its typed configuration into a ``ModelSpec``; nothing
below that knows which model it is in.  Each part is named by ``kind`` (looked
up in the part registries) and carries its sizes and constants in ``params``.
Layers may differ from one another, and the order layers run in is a list of
its own (``schedule``), which may name a layer twice or let a layer read the
cache another one wrote.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: dict = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class LayerSpec:
    """One block: a mixer and a feed-forward, each behind its norm."""
    prefix: str                     # tensor-name prefix, e.g. "model.layers.3."
    mixer: PartSpec
    mixer_norm: PartSpec
    ffn: PartSpec
    ffn_norm: PartSpec
    arrangement: str = "prenorm"


@dataclass(frozen=True)
class ScheduleEntry:
    """Run ``layer`` using cache ``cache``; ``writes`` False means the layer
    only reads what another entry with the same cache id wrote."""
    layer: int
    cache: int
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: tuple
    final_norm: PartSpec
    head: PartSpec
    schedule: tuple = ()

    def run_order(self) -> tuple:
        if self.schedule:
            return tuple(self.schedule)
        return tuple(ScheduleEntry(i, i, True) for i in range(len(self.layers)))


@dataclass
class BuildEnv:
    """Where and in which precision a model is built."""
    device: object
    dtype: object                   # activations and matrices: torch.bfloat16 or torch.float32
    hidden_size: int
    max_position: int
