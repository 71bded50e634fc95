"""RMSNorm, fused with the residual add that precedes it.

y = w * r / sqrt(mean(r^2) + eps), r = residual (+ pending), all in 32-bit
with one rounding at the end.  The reference builds the norm with
candle_nn::rms_norm(H, eps) (crates/vllm-models/src/llama/architecture.rs:27-28,108)
and adds residuals with separate ops (:53,58).
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Norm
from .registry import register_norm


class RMSNorm(Norm):
    """params: ``size``, ``eps``, ``name`` (weight tensor name after the prefix)."""

    @classmethod
    def tensor_specs(cls, params, prefix):
        return {prefix + params["name"]: TensorSpec((params["size"],), init="norm")}

    def __init__(self, params, prefix, env, tensors):
        super().__init__(params, prefix, env, tensors)
        self.eps = float(params["eps"])
        self.weight = tensors.get(prefix + params["name"], torch.float32)

    fuses_pending_linear = True

    def add_norm(self, resid, pending, rows=None):
        if isinstance(pending, ops.PendingLinear):
            # small decode batches: the product adds its result to the residual itself and prepares this
            # norm; the product that reads the result finishes it
            if rows is None and self.env.dtype == torch.bfloat16 and ops.skinny_fused_ok(pending.x, pending.weight, resid):
                return ops.skinny_gemm_residual(pending.x, pending.weight, resid, self.weight, self.eps)
            if rows is None and self.env.dtype == torch.bfloat16 and ops.tc_stream_fused_ok(pending.x, pending.weight, resid):
                return ops.tc_stream_gemm_residual(pending.x, pending.weight, resid, self.weight, self.eps)
            pending = pending.materialize()
        return ops.add_rmsnorm(resid, pending, self.weight, self.eps, self.env.dtype, rows)


register_norm("rmsnorm", RMSNorm)
