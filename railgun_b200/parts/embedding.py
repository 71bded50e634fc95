"""Token embedding and output head.

x = embed_tokens[ids], no scaling (crates/vllm-models/src/llama/architecture.rs:150);
logits = h W^T with W = lm_head.weight, or the embedding matrix when the
embeddings are tied (:110-118).  Logits are computed only for the rows asked
for and come out in 32-bit; the reference computes them for every row (:154-155).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Embedding, Head
from .registry import register_embedding, register_head


class TokenEmbedding(Embedding):
    """params: ``vocab_size``, ``hidden_size``, ``name`` (full tensor name)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        return {p["name"]: TensorSpec((p["vocab_size"], p["hidden_size"]))}

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.table = tensors.get(p["name"], env.dtype)
        self.vocab_size = p["vocab_size"]

    def embed(self, ids):
        return ops.embedding(ids, self.table)


class LMHead(Head):
    """params: ``vocab_size``, ``hidden_size``, ``name`` (full tensor name; the
    embedding's name when tied, so both share one tensor)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        return {p["name"]: TensorSpec((p["vocab_size"], p["hidden_size"]))}

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.weight = tensors.get(p["name"], env.dtype)

    def logits(self, h):
        return ops.linear(h, self.weight, out_dtype=torch.float32)


register_embedding("token_embedding", TokenEmbedding)
register_head("lm_head", LMHead)
