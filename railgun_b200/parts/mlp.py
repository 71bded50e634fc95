"""Dense gated feed-forward: down(silu(gate(x)) * up(x))
(crates/vllm-models/src/llama/architecture.rs:75-85).  gate and up are one
matrix here, stacked by rows at load.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import FeedForward
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        H, I = p["hidden_size"], p["intermediate_size"]
        return {
            prefix + "mlp.gate_proj.weight": TensorSpec((I, H)),
            prefix + "mlp.up_proj.weight": TensorSpec((I, H)),
            prefix + "mlp.down_proj.weight": TensorSpec((H, I)),
        }

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        m = prefix + "mlp."
        gate, up = tensors.get(m + "gate_proj.weight", env.dtype), tensors.get(m + "up_proj.weight", env.dtype)
        # bfloat16 with I % 8 == 0: gate and up rows interleaved in blocks of 8, which lets the decode
        # product apply SiLU-mul in its epilogue; otherwise gate rows, then up rows
        self.interleaved = env.dtype == torch.bfloat16 and p["intermediate_size"] % 8 == 0
        self.w_gate_up = (ops.interleave_gate_up(gate, up) if self.interleaved
                          else torch.cat([gate, up], dim=0).contiguous())
        tensors.drop(m + "gate_proj.weight", m + "up_proj.weight")
        self.w_down = tensors.get(m + "down_proj.weight", env.dtype)

    takes_normed_rows = True
    defers_output = True

    def forward(self, x, batch, defer=False):
        if isinstance(x, ops.NormedRows):
            if self.interleaved and ops.skinny_scaled_ok(x, self.w_gate_up):
                act = ops.skinny_gemm_scaled(x, self.w_gate_up, silu_mul=True)   # decode: norm, product and SiLU-mul in one
                return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)
            if self.interleaved and ops.tc_stream_scaled_ok(x, self.w_gate_up):
                act = ops.tc_stream_gemm(x, self.w_gate_up, silu_mul=True)       # the same for 17 to 64 rows
                return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)
            x = x.materialize()
        if self.interleaved and x.shape[0] <= ops.SKINNY_AUTO_ROWS and ops.skinny_gemm_ok(x, self.w_gate_up):
            act = ops.skinny_gemm(x, self.w_gate_up, silu_mul=True)              # decode: weights streamed once
        elif (self.interleaved and x.shape[0] <= ops.TC_STREAM_AUTO_ROWS and ops.tc_stream_ok(x, self.w_gate_up)):
            # decode batches of 17 to 32 rows: the swapped-operand tcgen05 product, SiLU-mul in its epilogue
            act = ops.tc_stream_gemm(x, self.w_gate_up, silu_mul=True)
        elif self.interleaved and x.shape[0] >= ops.TC_GEMM_MIN_ROWS and ops.tc_gemm_ok(x, self.w_gate_up):
            # prefill: tcgen05 on CTA pairs, SiLU-mul in the epilogue
            act = ops.tc_gemm(x, self.w_gate_up, silu_mul=True, tile="256x256")
        else:
            act = ops.silu_mul(ops.linear(x, self.w_gate_up), interleaved=self.interleaved)
        return ops.PendingLinear(act, self.w_down) if defer else ops.linear(act, self.w_down)


register_feed_forward("swiglu", SwiGLU)
