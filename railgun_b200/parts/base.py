"""The interfaces parts must have.

Every part class has
  * ``tensor_specs(params, prefix) -> {tensor name: TensorSpec}`` (a class
    method: the names and shapes it reads from the model folder), and
  * ``__init__(params, prefix, env, tensors)`` taking those tensors (already on
    the device, in stored precision) and casting what it computes with.
Sizes and constants come only from ``params``.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import ops


class Part:
    # False for a part that plans on the host while it runs (reads device values back, launches a number of
    # kernels that depends on the data): steps of a model with such a part are never captured in a CUDA graph.
    graph_safe = True

    @classmethod
    def tensor_specs(cls, params: dict, prefix: str) -> dict:
        return {}

    def __init__(self, params: dict, prefix: str, env, tensors: dict):
        self.params = params
        self.prefix = prefix
        self.env = env


class Norm(Part):
    """``add_norm(resid, pending, rows=None)``: add ``pending`` (or nothing) to
    the 32-bit residual stream in place and return the normed rows in the
    activation dtype.  With ``rows`` only those rows are returned and the
    residual is left as it was.

    A norm that sets ``fuses_pending_linear`` also takes ``pending`` as an
    ``ops.PendingLinear`` (a product not computed yet) and may return
    ``ops.NormedRows`` (a norm not computed yet); ``normed_input`` below keeps
    both away from parts that did not ask for them."""

    fuses_pending_linear = False

    def add_norm(self, resid, pending, rows=None):
        raise NotImplementedError


class PositionEncoding(Part):
    """``apply(qkv, batch, nh, nkv, d, kv_dest)`` encodes positions into the q
    and k heads of ``qkv`` [T, (nh+2nkv)d] in place.  ``kv_dest`` is None or
    ``(kv tensor, slot mapping)``; an encoding that can write k and v to the
    cache in the same pass does so and returns True, otherwise it returns False
    and the mixer writes them.

    Optional: an encoding that is a rotation of pairs (i, i + d/2) by angles from
    a table [max_position, d] = cos | sin may expose it as ``rotary_table`` and
    take a keyword ``paired8`` in ``apply``; the attention part then keeps its q
    and k rows in ``ops.rope_pair_order`` and, for a few single tokens, rotates
    inside the projection's kernel."""

    rotary_table = None

    def apply(self, qkv, batch, nh, nkv, d, kv_dest) -> bool:
        raise NotImplementedError


def normed_input(norm, part, stream, rows=None):
    """The rows that ``part`` reads: ``norm`` of the stream with what is pending
    added.  Values that are not computed yet pass only between a norm and a
    part that both declare that they take them."""
    pending = stream.pending
    if isinstance(pending, ops.PendingLinear) and not getattr(norm, "fuses_pending_linear", False):
        pending = pending.materialize()
    h = norm.add_norm(stream.resid, pending) if rows is None else norm.add_norm(stream.resid, pending, rows=rows)
    if isinstance(h, ops.NormedRows) and not getattr(part, "takes_normed_rows", False):
        h = h.materialize()
    return h


class Mixer(Part):
    """Mixes information between positions of a request.

    ``cache_need(params)`` (class method) says what it keeps between steps: a
    ``PagedKVNeed``, a ``StateNeed`` or None.  ``forward(x, batch, cache,
    writes)`` takes the normed rows [T, H] of the step's tokens and returns
    [T, H]; ``cache`` is a ``CacheView`` of what the need asked for; ``writes``
    False means the layer reads a cache that another layer fills.

    Optional, for mixers and feed-forwards alike: ``takes_normed_rows`` = True
    says that ``x`` may be an ``ops.NormedRows`` (which ``ops.linear`` takes in
    place of a tensor); ``defers_output`` = True says that ``forward`` has a
    keyword ``defer`` and, when it is True, may return its last product as an
    ``ops.PendingLinear``."""

    takes_normed_rows = False
    defers_output = False

    @classmethod
    def cache_need(cls, params: dict):
        return None

    def forward(self, x, batch, cache, writes: bool = True):
        raise NotImplementedError


class FeedForward(Part):
    """``forward(x, batch)``: [T, H] -> [T, H], each row on its own."""

    takes_normed_rows = False
    defers_output = False

    def forward(self, x, batch):
        raise NotImplementedError


class Embedding(Part):
    """``embed(ids)``: int32 [T] -> the 32-bit residual stream [T, H]."""

    def embed(self, ids):
        raise NotImplementedError


class Head(Part):
    """``logits(h)``: normed rows [W, H] -> float32 [W, V]."""

    def logits(self, h):
        raise NotImplementedError


@dataclass
class CacheView:
    """What one schedule entry sees of the cache."""
    cache_id: int
    group: int = -1            # page group of a PagedKVNeed, else -1
    kv: object = None          # [pages, 2, kv_heads, page_size, head_dim]
    page_size: int = 0
    state: object = None       # [max_requests, *shape] of a StateNeed


class Stream:
    """The residual stream during a step: the 32-bit sum and the last part's
    output, not yet added (it is added inside the next norm's kernel)."""

    __slots__ = ("resid", "pending")

    def __init__(self, resid):
        self.resid = resid
        self.pending = None


class Arrangement:
    """How a layer's parts are wired around the residual stream.
    ``run(layer, stream, batch, cache, writes)`` updates the stream."""

    def run(self, layer, stream, batch, cache, writes):
        raise NotImplementedError
