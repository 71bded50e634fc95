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
class SubLayer:
    """One branch of a block around the residual stream: ``part`` (a mixer or a
    feed-forward; ``role`` says which interface it has) behind ``norm``."""
    norm: PartSpec
    part: PartSpec
    role: str                       # "mixer" or "ffn"

    def __post_init__(self):
        if self.role not in ("mixer", "ffn"):
            raise ValueError(f"a sub-layer's role is 'mixer' or 'ffn', not {self.role!r}")


@dataclass(frozen=True)
class LayerSpec:
    """One block: a list of branches (norm, part) that its arrangement wires
    around the residual stream.  The usual block, a mixer and a feed-forward
    each behind its norm, can be given by the four fields of those names;
    ``sublayers`` gives any other list: a single mixer, two feed-forwards,
    three norms."""
    prefix: str                     # tensor-name prefix, e.g. "model.layers.3."
    mixer: PartSpec | None = None
    mixer_norm: PartSpec | None = None
    ffn: PartSpec | None = None
    ffn_norm: PartSpec | None = None
    arrangement: str = "prenorm"
    sublayers: tuple = ()

    def __post_init__(self):
        if self.sublayers and (self.mixer or self.ffn or self.mixer_norm or self.ffn_norm):
            raise ValueError("a LayerSpec is given by `sublayers` or by mixer / ffn with their norms, not both")
        if not self.sublayers and ((self.mixer is None) != (self.mixer_norm is None)
                                   or (self.ffn is None) != (self.ffn_norm is None)):
            raise ValueError("a part and its norm are given together")
        if not self.branches():
            raise ValueError("a layer needs at least one branch")

    def branches(self) -> tuple:
        """The block's branches in the order they run."""
        if self.sublayers:
            return tuple(self.sublayers)
        out = []
        if self.mixer is not None:
            out.append(SubLayer(self.mixer_norm, self.mixer, "mixer"))
        if self.ffn is not None:
            out.append(SubLayer(self.ffn_norm, self.ffn, "ffn"))
        return tuple(out)


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
