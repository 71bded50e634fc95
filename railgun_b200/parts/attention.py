"""Grouped-query attention over the paged cache.

q, k, v = x Wq^T, x Wk^T, x Wv^T (crates/vllm-models/src/llama/attention.rs:94-96);
positions are encoded into q and k, k and v go to the cache, then every query
attends its request's keys up to its own position (and not further back than
the window, if there is one), and the result goes through Wo (:133).  The
three projections are one matrix here, stacked by rows at load, which gives
the same numbers as three products.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorSpec
from .base import Mixer
from .registry import register_mixer, POSITION_ENCODINGS


# The tcgen05 flash kernel takes portions of prompts when the head size is 64 and pages hold 8..128 tokens;
# RAILGUN_B200_TC_ATTENTION=0 sends them to the mma.sync kernel instead.
USE_TC_ATTENTION = os.environ.get("RAILGUN_B200_TC_ATTENTION", "1") != "0"


class PagedAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``window`` (0: none), ``scale`` (None: head_dim^-0.5), ``position``
    (a PartSpec or None)."""

    @classmethod
    def tensor_specs(cls, p, prefix):
        H, nh, nkv, d = p["hidden_size"], p["num_heads"], p["num_kv_heads"], p["head_dim"]
        return {
            prefix + "self_attn.q_proj.weight": TensorSpec((nh * d, H)),
            prefix + "self_attn.k_proj.weight": TensorSpec((nkv * d, H)),
            prefix + "self_attn.v_proj.weight": TensorSpec((nkv * d, H)),
            prefix + "self_attn.o_proj.weight": TensorSpec((H, nh * d)),
        }

    @classmethod
    def cache_need(cls, p):
        return PagedKVNeed(p["num_kv_heads"], p["head_dim"], int(p.get("window") or 0))

    def __init__(self, p, prefix, env, tensors):
        super().__init__(p, prefix, env, tensors)
        self.nh, self.nkv, self.d = p["num_heads"], p["num_kv_heads"], p["head_dim"]
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} heads cannot share {self.nkv} key/value heads")
        if self.d > 256:
            raise ValueError(f"head size {self.d} is above the attention kernels' limit of 256")
        self.window = int(p.get("window") or 0)
        self.scale = float(p["scale"]) if p.get("scale") is not None else float(self.d) ** -0.5
        a = prefix + "self_attn."
        pos = p.get("position")
        self.position = None
        if pos is not None:
            self.position = tensors.shared_part(("position", pos), lambda: POSITION_ENCODINGS.get(pos.kind)(
                pos.params, prefix, env, tensors))
        wq, wk = tensors.get(a + "q_proj.weight", env.dtype), tensors.get(a + "k_proj.weight", env.dtype)
        # With a rotary table and a head size in steps of 16, q and k rows are kept in the order in which every
        # 16 rows hold 8 whole rotation pairs (q . k does not notice; the cache then holds k in that order): the
        # projection of a few single tokens can then rotate and write the cache in its own kernel.
        self.paired8 = getattr(self.position, "rotary_table", None) is not None and self.d % 16 == 0
        if self.paired8:
            wq, wk = ops.reorder_rope_rows(wq, self.nh, self.d), ops.reorder_rope_rows(wk, self.nkv, self.d)
        self.w_qkv = torch.cat([wq, wk, tensors.get(a + "v_proj.weight", env.dtype)], dim=0).contiguous()
        tensors.drop(a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight")
        self.w_o = tensors.get(a + "o_proj.weight", env.dtype)

    takes_normed_rows = True
    defers_output = True

    def forward(self, x, batch, cache, writes=True, defer=False):
        nh, nkv, d = self.nh, self.nkv, self.d
        slots = batch.slot_mapping[cache.group]
        if self.paired8 and self.env.dtype == torch.bfloat16 and ops.skinny_rope_ok(x, self.w_qkv, d):
            # a few single tokens: projection, rotation and cache write in one kernel
            qkv = ops.skinny_gemm_rope_cache(x, self.w_qkv, self.position.rotary_table, batch.positions,
                                             slots if writes else None, cache.kv, nh, nkv, d, batch.err_flag)
        elif (self.paired8 and self.env.dtype == torch.bfloat16 and batch.decode_only
              and ops.tc_stream_rope_ok(x, self.w_qkv, d)):
            # 17 to 64 single tokens: the same in the streaming tcgen05 product
            qkv = ops.tc_stream_gemm_rope_cache(x, self.w_qkv, self.position.rotary_table, batch.positions,
                                                slots if writes else None, cache.kv, nh, nkv, d, batch.err_flag)
        else:
            qkv = ops.linear(x, self.w_qkv)
            kv_dest = (cache.kv, slots) if writes else None
            wrote = False
            if self.position is not None:
                if self.paired8:
                    wrote = self.position.apply(qkv, batch, nh, nkv, d, kv_dest, paired8=True)
                else:
                    wrote = self.position.apply(qkv, batch, nh, nkv, d, kv_dest)
            if writes and not wrote:
                ops.rope_cache_write(qkv, None, batch.positions, slots, cache.kv, nh, nkv, d, cache.page_size,
                                     batch.err_flag)
        out = self.attend(qkv, batch, cache)
        return ops.PendingLinear(out, self.w_o) if defer else ops.linear(out, self.w_o)

    def attend(self, qkv, batch, cache):
        """Pick the attention kernels for this step's shape and precision:
        bfloat16 with a head size in steps of 16 runs on the tensor cores
        (requests with several tokens through the flash-style kernel, single
        tokens through the split kernel); everything else, and all of the
        32-bit path, through the general kernel."""
        nh, nkv, d = self.nh, self.nkv, self.d
        table = batch.block_table[cache.group]
        if qkv.dtype != torch.bfloat16 or d % 16:
            return ops.paged_attention_general(qkv, qkv.shape[1], cache.kv, table, batch.req_of_token,
                                               batch.positions, nh, nkv, d, self.window, self.scale)
        out = torch.empty((qkv.shape[0], nh * d), dtype=qkv.dtype, device=qkv.device)
        kv_tiles = nkv * (-(-(nh // nkv) // 8))
        if batch.decode_only:
            n = batch.num_tokens
            ops.decode_attention(qkv, qkv.shape[1], out, cache.kv, table, None, n, batch.req_of_token,
                                 batch.positions, nh, nkv, d, self.window, self.scale,
                                 ops.decode_splits(n, kv_tiles, batch.max_context_len))
            return out
        if batch.num_prefill_tiles:
            if USE_TC_ATTENTION and batch.num_prefill_tiles128 and ops.prefill_attention_tc_ok(
                    qkv, cache.kv, d, cache.page_size):
                ops.prefill_attention_tc(qkv, out, cache.kv, table, batch.prefill_tiles128, batch.positions,
                                         nh, nkv, d, self.window, self.scale)
            else:
                ops.prefill_attention(qkv, qkv.shape[1], out, cache.kv, table, batch.prefill_tiles, batch.positions,
                                      nh, nkv, d, self.window, self.scale)
        if batch.num_decode_rows:
            n = batch.num_decode_rows
            ops.decode_attention(qkv, qkv.shape[1], out, cache.kv, table, batch.decode_rows, n, batch.req_of_token,
                                 batch.positions, nh, nkv, d, self.window, self.scale,
                                 ops.decode_splits(n, kv_tiles, batch.max_context_len))
        return out


register_mixer("paged_attention", PagedAttention)
