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

import array
from dataclasses import dataclass, field
from itertools import accumulate, chain

import numpy as np
import torch


ATTENTION_TILE_ROWS = 64      # query rows per tile of the prefill attention kernel


class BatchError(ValueError):
    """A step that cannot run: bad token ids, positions or requests."""


_PINNED = None


def _pinned() -> bool:
    """Whether host buffers are page-locked (asked once: the answer costs 20 us each time)."""
    global _PINNED
    if _PINNED is None:
        _PINNED = torch.cuda.is_available()
    return _PINNED


def _token_array(tokens) -> np.ndarray:
    """A request's tokens as an integer array; a list of Python ints goes through ``array``, which
    converts several times faster than numpy's type discovery."""
    if isinstance(tokens, np.ndarray):
        return tokens
    try:
        return np.frombuffer(array.array("q", tokens), dtype=np.int64)
    except (TypeError, OverflowError):
        return np.asarray(tokens)


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
    host_request_ids: np.ndarray | None = None   # int64
    host_context_lens: np.ndarray | None = None  # int32: tokens each request holds once the step has run
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
    R = len(entries)
    G = len(page_sizes)
    token_arrays = [_token_array(e.tokens) for e in entries]
    for e, toks in zip(entries, token_arrays):
        if toks.size < 1:
            raise BatchError(f"request {e.request_id}: an entry needs at least one token")
        if toks.dtype.kind not in "iu" or toks.min() < 0 or toks.max() >= vocab_size:
            raise BatchError(f"request {e.request_id}: token ids must be in [0, {vocab_size})")
    # small counts are Python numbers: every numpy call on an array of a few entries costs microseconds
    count_list = [t.size for t in token_arrays]
    want_ends = list(accumulate(len(e.want) for e in entries))
    W = want_ends[-1]
    ids = np.fromiter((e.request_id for e in entries), dtype=np.int64, count=R)
    counts = np.array(count_list, dtype=np.int32)
    want_offsets = np.array([0, *want_ends], dtype=np.int32)
    want = np.fromiter(chain.from_iterable(e.want for e in entries), dtype=np.int32, count=W)
    # checked, then reserved (all or nothing new) by the cache manager
    code, bad, value, starts, max_blocks = alloc.plan_step(ids, counts, want, want_offsets, max_position)
    if code:
        rid, n = entries[bad].request_id, int(counts[bad])
        if code == -2:
            raise BatchError(f"request {rid} appears twice in one step")
        if code == -7:
            raise BatchError(f"request {rid}: position {int(starts[bad]) + n - 1} is beyond the model's "
                             f"max_position_embeddings {max_position}")
        if code == -8:
            raise BatchError(f"request {rid}: wanted place {value} is outside its {n} tokens")
        alloc._raise(code, f"reserve({rid}, {int(starts[bad]) + n})")
    T = sum(count_list)
    several = [c for c in count_list if c > 1]
    n_tiles = sum(-(-c // ATTENTION_TILE_ROWS) for c in several)
    n_tiles128 = sum(-(-c // (2 * ATTENTION_TILE_ROWS)) for c in several)
    n_dec = R - len(several)
    max_blocks_t = tuple(max_blocks.tolist())
    start_list = starts.tolist()
    sizes = [T, T, T, W, R + 1, R, R, R]
    for g in range(G):
        sizes += [T, R * max_blocks_t[g]]
    sizes += [3 * n_tiles, n_dec, 3 * n_tiles128]
    offs = [0, *accumulate(sizes)]
    buf = torch.empty(offs[-1], dtype=torch.int32, pin_memory=_pinned())
    tokens = token_arrays[0] if R == 1 else np.concatenate(token_arrays)
    if tokens.dtype != np.int64:
        tokens = tokens.astype(np.int64)
    alloc.fill_step(ids, counts, starts, np.ascontiguousarray(tokens), want, want_offsets, max_blocks,
                    ATTENTION_TILE_ROWS, np.asarray(offs, dtype=np.int64), buf.data_ptr())
    host = buf.numpy()
    cu = host[offs[4]:offs[5]].copy()
    slots = host[offs[7]:offs[8]].copy()
    layout = (tuple(count_list), W, max_blocks_t)
    static = into(layout) if into is not None else None
    if static is not None:
        if static.numel() != buf.numel():
            raise BatchError(f"the step packs {buf.numel()} ints, the buffer to copy into holds {static.numel()}")
        static.copy_(buf, non_blocking=True)
        dev = static
    else:
        dev = buf.to(device, non_blocking=True)
    d = dev.split(sizes).__getitem__                       # views, cut in one call
    return StepBatch(
        num_tokens=T, num_requests=R, num_wanted=W,
        max_query_len=max(count_list), max_context_len=max(a + b for a, b in zip(start_list, count_list)),
        token_ids=d(0), positions=d(1), req_of_token=d(2), want_rows=d(3), cu_seqlens=d(4),
        context_lens=d(5), start_pos=d(6), state_slots=d(7),
        slot_mapping=[d(8 + 2 * g) for g in range(G)],
        block_table=[d(9 + 2 * g).view(R, max_blocks_t[g]) for g in range(G)],
        err_flag=err_flag, host_cu_seqlens=cu, host_start_pos=starts, host_state_slots=slots,
        host_request_ids=ids, host_context_lens=starts + counts,
        request_ids=[e.request_id for e in entries], h2d_bytes=offs[-1] * 4, host_buffer=buf,
        layout=layout,
        decode_only=max(count_list) == 1,
        prefill_tiles=d(8 + 2 * G).view(-1, 3) if n_tiles else None, num_prefill_tiles=n_tiles,
        decode_rows=d(9 + 2 * G) if n_dec else None, num_decode_rows=n_dec,
        prefill_tiles128=d(10 + 2 * G).view(-1, 3) if n_tiles128 else None, num_prefill_tiles128=n_tiles128,
    )
