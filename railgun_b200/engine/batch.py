"""One step's batch: requests with their next tokens, packed.

An entry is (request, its next tokens, the places among them whose logits are
wanted).  Portions of prompts and single decoded tokens are the same thing
here: tokens that continue at the request's position in the cache.  The
reference packs prefill chunks first and then one token per decode slot, with
a slot mapping, context lengths and a zero-padded block table
(crates/vllm-engine/src/engine.rs:185-227, crates/vllm-scheduler/src/batch.rs:41-51);
the same fields are built here, plus the per-token request index and absolute
positions that let one attention call serve every cut of the work.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


ATTENTION_TILE_ROWS = 64      # query rows per tile of the prefill attention kernel


class BatchError(ValueError):
    """A step that cannot run: bad token ids, positions or requests."""


@dataclass
class StepEntry:
    request_id: int
    tokens: list
    want: list = field(default_factory=list)     # indices into ``tokens``


@dataclass
class StepBatch:
    """Device-side description of a step (int32 tensors unless noted)."""
    num_tokens: int
    num_requests: int
    num_wanted: int
    max_query_len: int
    max_context_len: int
    token_ids: torch.Tensor          # [T]
    positions: torch.Tensor          # [T] absolute position of each token in its request
    req_of_token: torch.Tensor       # [T] index into the step's requests
    want_rows: torch.Tensor          # [W] rows whose logits are wanted
    cu_seqlens: torch.Tensor         # [R+1] offsets of each request's tokens
    context_lens: torch.Tensor       # [R] tokens in the cache after this step
    start_pos: torch.Tensor          # [R] tokens in the cache before this step
    state_slots: torch.Tensor        # [R] state slot of each request
    slot_mapping: list               # per page group: [T] page * page_size + offset
    block_table: list                # per page group: [R, max_blocks]
    err_flag: torch.Tensor | None = None
    # host copies, for parts that plan on the host
    host_cu_seqlens: np.ndarray | None = None
    host_start_pos: np.ndarray | None = None
    host_state_slots: np.ndarray | None = None
    request_ids: list = field(default_factory=list)
    h2d_bytes: int = 0
    host_buffer: torch.Tensor | None = None      # the pinned buffer the step was packed in (alive until the copy ran)
    layout: tuple = ()               # (token counts, wanted places, block-table widths): equal layouts, equal offsets
    decode_only: bool = False        # every request brings exactly one token
    # how attention splits the step: requests with several tokens in tiles of up to 64 consecutive
    # positions, [n, 3] = first row, rows, request; requests with one token as a list of rows
    prefill_tiles: torch.Tensor | None = None
    num_prefill_tiles: int = 0
    decode_rows: torch.Tensor | None = None
    num_decode_rows: int = 0
    prefill_tiles128: torch.Tensor | None = None     # the same requests in tiles of up to 128 positions
    num_prefill_tiles128: int = 0


def build_step_batch(entries, alloc, page_sizes, vocab_size: int, max_position: int, device,
                     err_flag=None, into=None) -> StepBatch:
    """Validate the entries against the cache's bookkeeping, reserve pages and
    pack everything into one host buffer that goes to the device in one copy.

    ``alloc`` is the PageAllocator; a request it does not know yet is added.
    Nothing is launched and nothing is reserved if any entry is invalid.
    Block tables are as wide as the longest one rounded up to a power of two,
    so that steps of the same token counts have the same layout.  ``into``:
    called with the layout (token counts, wanted places, block-table widths)
    once it is known; if it returns a device int32 buffer (of exactly the
    layout's size) the step is copied into that buffer, whose address is what a
    captured graph reads, and the batch's tensors are views of it."""
    if not entries:
        raise BatchError("a step needs at least one entry")
    seen = set()
    starts = []
    token_arrays = []
    for e in entries:
        if e.request_id in seen:
            raise BatchError(f"request {e.request_id} appears twice in one step")
        seen.add(e.request_id)
        n = len(e.tokens)
        if n < 1:
            raise BatchError(f"request {e.request_id}: an entry needs at least one token")
        toks = np.asarray(e.tokens)
        token_arrays.append(toks)
        if toks.min() < 0 or toks.max() >= vocab_size:
            raise BatchError(f"request {e.request_id}: token ids must be in [0, {vocab_size})")
        start = alloc.num_computed(e.request_id) if alloc.has(e.request_id) else 0
        if start + n > max_position:
            raise BatchError(f"request {e.request_id}: position {start + n - 1} is beyond the model's "
                             f"max_position_embeddings {max_position}")
        for w in e.want:
            if not 0 <= w < n:
                raise BatchError(f"request {e.request_id}: wanted place {w} is outside its {n} tokens")
        starts.append(start)
    # reserve (atomic per request; on failure give back what this call added)
    added = []
    try:
        for e, start in zip(entries, starts):
            if not alloc.has(e.request_id):
                alloc.add_request(e.request_id)
                added.append(e.request_id)
            alloc.reserve(e.request_id, start + len(e.tokens))
    except Exception:
        for rid in added:
            alloc.release(rid)
        raise

    R = len(entries)
    counts = np.array([len(e.tokens) for e in entries], dtype=np.int64)
    T = int(counts.sum())
    W = sum(len(e.want) for e in entries)
    G = len(page_sizes)
    tables = [[alloc.block_table(e.request_id, g) for e in entries] for g in range(G)]
    max_blocks = [1 << (max(1, max(len(t) for t in tables[g])) - 1).bit_length() for g in range(G)]

    tiles, tiles128, dec_rows = [], [], []
    off = 0
    for i, c in enumerate(counts):
        c = int(c)
        if c == 1:
            dec_rows.append(off)
        else:
            tiles += [(off + k, min(ATTENTION_TILE_ROWS, c - k), i) for k in range(0, c, ATTENTION_TILE_ROWS)]
            tiles128 += [(off + k, min(128, c - k), i) for k in range(0, c, 128)]
        off += c
    sizes = [T, T, T, W, R + 1, R, R, R]
    for g in range(G):
        sizes += [T, R * max_blocks[g]]
    sizes += [3 * len(tiles), len(dec_rows), 3 * len(tiles128)]
    offs = np.concatenate([[0], np.cumsum(sizes)])
    buf = torch.empty(int(offs[-1]), dtype=torch.int32, pin_memory=torch.cuda.is_available())
    host = buf.numpy()
    seg = lambda i: host[offs[i]:offs[i + 1]]
    cu = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    start_arr = np.array(starts, dtype=np.int32)
    seg(0)[:] = np.concatenate(token_arrays)
    pos = np.concatenate([np.arange(s, s + c, dtype=np.int32) for s, c in zip(starts, counts)])
    seg(1)[:] = pos
    req = np.repeat(np.arange(R, dtype=np.int32), counts)
    seg(2)[:] = req
    if W:
        seg(3)[:] = np.concatenate([cu[i] + np.asarray(e.want, dtype=np.int32)
                                    for i, e in enumerate(entries) if len(e.want)])
    seg(4)[:] = cu
    seg(5)[:] = start_arr + counts.astype(np.int32)
    seg(6)[:] = start_arr
    slots = np.array([alloc.slot(e.request_id) for e in entries], dtype=np.int32)
    seg(7)[:] = slots
    for g in range(G):
        ps = page_sizes[g]
        bt = np.zeros((R, max_blocks[g]), dtype=np.int32)
        for i, t in enumerate(tables[g]):
            bt[i, :len(t)] = np.maximum(t, 0)          # released pages are never read
        page_of = bt[req, pos // ps]
        seg(8 + 2 * g)[:] = page_of * ps + pos % ps
        seg(9 + 2 * g)[:] = bt.reshape(-1)
    if tiles:
        seg(8 + 2 * G)[:] = np.asarray(tiles, dtype=np.int32).reshape(-1)
    if dec_rows:
        seg(9 + 2 * G)[:] = np.asarray(dec_rows, dtype=np.int32)
    if tiles128:
        seg(10 + 2 * G)[:] = np.asarray(tiles128, dtype=np.int32).reshape(-1)
    layout = (tuple(int(c) for c in counts), W, tuple(max_blocks))
    static = into(layout) if into is not None else None
    if static is not None:
        if static.numel() != buf.numel():
            raise BatchError(f"the step packs {buf.numel()} ints, the buffer to copy into holds {static.numel()}")
        static.copy_(buf, non_blocking=True)
        dev = static
    else:
        dev = buf.to(device, non_blocking=True)
    d = lambda i: dev[int(offs[i]):int(offs[i + 1])]
    return StepBatch(
        num_tokens=T, num_requests=R, num_wanted=W,
        max_query_len=int(counts.max()), max_context_len=int((start_arr + counts).max()),
        token_ids=d(0), positions=d(1), req_of_token=d(2), want_rows=d(3), cu_seqlens=d(4),
        context_lens=d(5), start_pos=d(6), state_slots=d(7),
        slot_mapping=[d(8 + 2 * g) for g in range(G)],
        block_table=[d(9 + 2 * g).view(R, max_blocks[g]) for g in range(G)],
        err_flag=err_flag, host_cu_seqlens=cu, host_start_pos=start_arr, host_state_slots=slots,
        request_ids=[e.request_id for e in entries], h2d_bytes=int(offs[-1]) * 4, host_buffer=buf,
        layout=layout,
        decode_only=bool(counts.max() == 1),
        prefill_tiles=d(8 + 2 * G).view(-1, 3) if tiles else None, num_prefill_tiles=len(tiles),
        decode_rows=d(9 + 2 * G) if dec_rows else None, num_decode_rows=len(dec_rows),
        prefill_tiles128=d(10 + 2 * G).view(-1, 3) if tiles128 else None, num_prefill_tiles128=len(tiles128),
    )
