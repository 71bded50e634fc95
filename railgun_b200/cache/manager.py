"""The cache manager: pages, block tables and state slots.

The bookkeeping lives in C++ (``csrc/host/cache_manager.hpp``); this module is
its Python face and also owns the device memory the pages stand for.

A model's mixers state what they need (``PagedKVNeed``: key/value pages of a
given geometry, maybe windowed; ``StateNeed``: a fixed-size buffer per
request).  Needs with the same geometry share a group: one set of page ids and
one block table per request, with one page tensor for every cache id in the
group.  The reference keeps one pool and one block table per request
(crates/vllm-paged-attention/src/block.rs:49-59, kv_cache.rs:10-25); its single
pool is shared by all layers, which overwrites keys; here each cache id has
its own tensor ``[pages, 2, kv_heads, page_size, head_dim]``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p, POINTER
from dataclasses import dataclass

import numpy as np

from .. import native


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


@dataclass(frozen=True)
class PagedKVNeed:
    """Pages that grow with the request: what an attention-like mixer asks for.  By default a page holds keys and
    values, ``[2, num_kv_heads, page_size, head_dim]`` in the model's precision, with the page size and the pool
    the engine was given.  A mixer that wants something else says so: ``page_size`` and ``pool_tokens`` (tokens
    the group's pool holds; a windowed group can do with fewer), ``dtype`` (a torch dtype name) and
    ``page_shape`` (what one page is, as a tuple in which the string "page" stands for the page size, for
    instance ``("page", 96)`` for one compressed vector per token)."""
    num_kv_heads: int
    head_dim: int
    window: int = 0            # 0: all keys are kept
    page_size: int = 0         # 0: the engine's
    pool_tokens: int = 0       # 0: the engine's
    dtype: str | None = None   # None: the model's
    page_shape: tuple | None = None

    def shape_of_page(self, page_size: int) -> tuple:
        if self.page_shape is None:
            return (2, self.num_kv_heads, page_size, self.head_dim)
        return tuple(page_size if x == "page" else int(x) for x in self.page_shape)


@dataclass(frozen=True)
class StateNeed:
    """A buffer of fixed size per request, indexed by the request's state slot."""
    shape: tuple
    dtype: str = "float32"


@dataclass
class GroupInfo:
    need: PagedKVNeed
    page_size: int
    num_pages: int
    cache_ids: list


_STATUS = {-1: "out of pages", -2: "duplicate request", -3: "unknown request", -4: "out of state slots",
           -5: "bad argument", -6: "cache bookkeeping is corrupt (a page freed twice or lost)"}


def _lib():
    lib = native.load("runtime", kind="host")
    if not getattr(lib, "_rg_typed", False):
        lib.rg_cache_create.restype = c_void_p
        lib.rg_cache_create.argtypes = [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int]
        lib.rg_cache_destroy.argtypes = [c_void_p]
        lib.rg_cache_destroy.restype = None
        for name in ("add_request", "release", "has", "num_computed", "slot"):
            getattr(lib, f"rg_cache_{name}").argtypes = [c_void_p, c_longlong]
        for name in ("reserve", "commit"):
            getattr(lib, f"rg_cache_{name}").argtypes = [c_void_p, c_longlong, c_int]
        lib.rg_cache_can_reserve.argtypes = [c_void_p, c_longlong, c_int, c_int]
        lib.rg_cache_table.argtypes = [c_void_p, c_longlong, c_int, c_void_p, c_int]
        lib.rg_cache_free_pages.argtypes = [c_void_p, c_int]
        lib.rg_cache_pack_decode.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_int,
                                             c_void_p]
        lib.rg_cache_records.argtypes = [c_void_p]
        lib.rg_cache_records.restype = c_void_p
        lib.rg_cache_set_request.argtypes = [c_void_p, c_longlong, c_int, c_int, c_int, c_float, c_int, c_float,
                                             c_ulonglong]
        lib.rg_cache_advance.argtypes = [c_void_p, c_void_p, c_int, c_int]
        lib.rg_cache_commit_many.argtypes = [c_void_p, c_void_p, c_void_p, c_int]
        lib.rg_cache_plan_step.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                           c_void_p, c_void_p, c_void_p]
        lib.rg_cache_fill_step.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                           c_void_p, c_int, c_void_p, c_void_p]
        for name in ("free_slots", "num_requests", "check"):
            getattr(lib, f"rg_cache_{name}").argtypes = [c_void_p]
        lib.rg_sched_create.restype = c_void_p
        lib.rg_sched_create.argtypes = [c_void_p, c_int, c_int, c_int, c_int]
        lib.rg_sched_destroy.argtypes = [c_void_p]
        lib.rg_sched_destroy.restype = None
        lib.rg_sched_add_request.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_int, c_float,
                                             c_int, c_float, c_ulonglong]
        lib.rg_sched_sampling_many.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                               c_void_p]
        for name in ("schedule", "fetch"):
            getattr(lib, f"rg_sched_{name}").argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                                         c_void_p, c_int]
        lib.rg_sched_preempted.argtypes = [c_void_p, c_void_p, c_int]
        lib.rg_sched_finished.argtypes = [c_void_p, c_void_p, c_int]
        lib.rg_sched_update.argtypes = [c_void_p, c_void_p, c_void_p, c_int]
        for name in ("abort", "finish_reason", "num_generated", "num_preemptions"):
            getattr(lib, f"rg_sched_{name}").argtypes = [c_void_p, c_longlong]
        lib.rg_sched_num_generated_many.argtypes = [c_void_p, c_void_p, c_int, c_void_p]
        lib.rg_sched_outputs.argtypes = [c_void_p, c_longlong, c_void_p, c_int]
        lib.rg_sched_error.argtypes = [c_void_p, c_longlong, c_void_p, c_int]
        lib.rg_sched_forget.argtypes = [c_void_p, c_longlong]
        lib.rg_sched_forget.restype = None
        for name in ("num_waiting", "num_running", "next_step_predictable"):
            getattr(lib, f"rg_sched_{name}").argtypes = [c_void_p]
        lib._rg_typed = True
    return lib


# A live request's record, one per state slot (csrc/host/cache_manager.hpp, RequestRecord): 64 bytes.
REQUEST_RECORD = np.dtype([
    ("request_id", "<i8"), ("num_computed", "<i4"), ("prompt_len", "<i4"), ("num_generated", "<i4"),
    ("max_new_tokens", "<i4"), ("last_token", "<i4"), ("top_k", "<i4"), ("temperature", "<f4"), ("top_p", "<f4"),
    ("seed", "<u8"), ("flags", "<i4"), ("reserved", "<i4", (3,))])


class PageAllocator:
    """The C++ cache manager: page groups, block tables, state slots and the slots' request records.  No
    device memory."""

    def __init__(self, page_sizes, num_pages, windows, max_requests: int):
        self._lib = _lib()
        n = len(page_sizes)
        if not (len(num_pages) == len(windows) == n):
            raise CacheError("page_sizes, num_pages and windows must have one entry per group")
        arr = lambda v: (c_int * n)(*[int(x) for x in v])
        self._h = self._lib.rg_cache_create(n, arr(page_sizes), arr(num_pages), arr(windows), int(max_requests))
        if not self._h:
            raise CacheError(f"cannot create a cache manager with page sizes {list(page_sizes)}, "
                             f"pages {list(num_pages)}, windows {list(windows)}, {max_requests} slots")
        self.page_sizes = [int(x) for x in page_sizes]
        self.num_pages = [int(x) for x in num_pages]
        self.windows = [int(x) for x in windows]
        self.max_requests = int(max_requests)
        self._buf = np.empty(64, dtype=np.int32)
        self._any_sampled = c_int(0)
        if self._lib.rg_cache_record_bytes() != REQUEST_RECORD.itemsize:
            raise CacheError("the request record of the native library is not the one this module describes")

    @property
    def records(self) -> np.ndarray:
        """The request records of all state slots, in place (a view of the C++ array, valid while this object
        lives): record s describes the request in slot s; ``request_id`` -1 marks a free slot."""
        n = max(1, self.max_requests)
        raw = (ctypes.c_char * (n * REQUEST_RECORD.itemsize)).from_address(self._lib.rg_cache_records(self._h))
        return np.frombuffer(raw, dtype=REQUEST_RECORD, count=n)

    def record(self, req_id: int):
        """A copy of a live request's record."""
        return self.records[self.slot(req_id)].copy()

    def set_request(self, req_id: int, prompt_len: int = 0, num_generated: int = 0, max_new_tokens: int = 0,
                    temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        """Fill in what the cache manager does not work out itself in a live request's record (the scheduler does
        this in C++ when it admits a request)."""
        code = self._lib.rg_cache_set_request(self._h, req_id, int(prompt_len), int(num_generated), int(max_new_tokens),
                                              float(temperature), int(top_k), float(top_p), int(seed) & ((1 << 64) - 1))
        if code:
            self._raise(code, f"set_request({req_id})")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rg_cache_destroy(h)

    @property
    def handle(self):
        return self._h

    def _raise(self, code: int, what: str):
        if code == -1:
            raise OutOfPages(f"{what}: out of pages")
        raise CacheError(f"{what}: {_STATUS.get(code, code)}")

    def add_request(self, req_id: int) -> int:
        slot = self._lib.rg_cache_add_request(self._h, req_id)
        if slot < 0:
            self._raise(slot, f"add_request({req_id})")
        return slot

    def has(self, req_id: int) -> bool:
        return bool(self._lib.rg_cache_has(self._h, req_id))

    def reserve(self, req_id: int, new_len: int) -> None:
        code = self._lib.rg_cache_reserve(self._h, req_id, int(new_len))
        if code:
            self._raise(code, f"reserve({req_id}, {new_len})")

    def can_reserve(self, req_id: int, new_len: int, spare: int = 0) -> bool:
        return bool(self._lib.rg_cache_can_reserve(self._h, req_id, int(new_len), int(spare)))

    def commit(self, req_id: int, new_len: int) -> None:
        code = self._lib.rg_cache_commit(self._h, req_id, int(new_len))
        if code:
            self._raise(code, f"commit({req_id}, {new_len})")

    def release(self, req_id: int) -> None:
        code = self._lib.rg_cache_release(self._h, req_id)
        if code:
            self._raise(code, f"release({req_id})")

    def num_computed(self, req_id: int) -> int:
        n = self._lib.rg_cache_num_computed(self._h, req_id)
        if n < 0:
            self._raise(n, f"num_computed({req_id})")
        return n

    def slot(self, req_id: int) -> int:
        s = self._lib.rg_cache_slot(self._h, req_id)
        if s < 0:
            self._raise(s, f"slot({req_id})")
        return s

    def block_table(self, req_id: int, group: int = 0) -> np.ndarray:
        """Logical page -> page id of one group; -1 where a window has passed."""
        n = self._lib.rg_cache_table(self._h, req_id, group, self._buf.ctypes.data, self._buf.size)
        if n < 0:
            self._raise(n, f"block_table({req_id}, {group})")
        if n > self._buf.size:
            self._buf = np.empty(max(n, 2 * self._buf.size), dtype=np.int32)
            n = self._lib.rg_cache_table(self._h, req_id, group, self._buf.ctypes.data, self._buf.size)
        return self._buf[:n].copy()

    def pack_decode(self, ids: np.ndarray, B: int, MB: int, out: np.ndarray, ahead: int = 0,
                    sampling: np.ndarray | None = None, draw_ahead: int = 0) -> bool:
        """Reserve one more token for each request in ``ids`` (int64) and write
        the decode step's positions, slots and block tables into ``out``
        (int32; layout in csrc/host/runtime.cpp, rg_cache_pack_decode).
        ``ahead`` = 1 packs the step after a step that is launched but not yet
        committed.  ``sampling`` (int32 [7 B]) receives the rows' sampling
        parameters from the requests' records, the draw numbered
        num_generated + ``draw_ahead``; returns whether any row samples."""
        code = self._lib.rg_cache_pack_decode(self._h, ids.ctypes.data, ids.size, B, MB, out.ctypes.data, int(ahead),
                                              sampling.ctypes.data if sampling is not None else None, int(draw_ahead),
                                              ctypes.byref(self._any_sampled))
        if code:
            self._raise(code, "pack_decode")
        return bool(self._any_sampled.value)

    def plan_step(self, ids: np.ndarray, counts: np.ndarray, want: np.ndarray, want_offsets: np.ndarray,
                  max_position: int):
        """Check a step of any shape (``ids`` int64, the others int32), add the requests that are new and
        reserve pages for all.  Returns (status, entry, value, starts, max_blocks): status 0, or a
        negative code about entry ``entry`` (-7: beyond ``max_position``; -8: wanted place ``value``
        is outside the entry's tokens; others as ``_STATUS``), with nothing added that was not there."""
        R = ids.size
        starts = np.empty(R, dtype=np.int32)
        max_blocks = np.empty(len(self.page_sizes), dtype=np.int32)
        bad = np.zeros(2, dtype=np.int32)
        code = self._lib.rg_cache_plan_step(self._h, ids.ctypes.data, counts.ctypes.data, R, want.ctypes.data,
                                            want_offsets.ctypes.data, int(max_position), starts.ctypes.data,
                                            max_blocks.ctypes.data, bad.ctypes.data, bad[1:].ctypes.data)
        return code, int(bad[0]), int(bad[1]), starts, max_blocks

    def fill_step(self, ids, counts, starts, tokens, want, want_offsets, max_blocks, tile_rows: int,
                  segments: np.ndarray, out_ptr: int) -> None:
        """Write a planned step into its packed buffer (layout in csrc/host/runtime.cpp,
        rg_cache_fill_step); ``tokens`` int64, ``segments`` int64 offsets of the buffer's parts."""
        code = self._lib.rg_cache_fill_step(self._h, ids.ctypes.data, counts.ctypes.data, starts.ctypes.data, ids.size,
                                            tokens.ctypes.data, want.ctypes.data, want_offsets.ctypes.data,
                                            max_blocks.ctypes.data, int(tile_rows), segments.ctypes.data, out_ptr)
        if code:
            self._raise(code, "fill_step")

    def commit_many(self, ids: np.ndarray, new_lens: np.ndarray) -> None:
        """``commit`` for several requests: ``ids`` int64, ``new_lens`` int32."""
        code = self._lib.rg_cache_commit_many(self._h, ids.ctypes.data, new_lens.ctypes.data, ids.size)
        if code:
            self._raise(code, "commit_many")

    def advance(self, ids: np.ndarray, n: int = 1) -> None:
        code = self._lib.rg_cache_advance(self._h, ids.ctypes.data, ids.size, n)
        if code:
            self._raise(code, "advance")

    def free_pages(self, group: int = 0) -> int:
        return self._lib.rg_cache_free_pages(self._h, group)

    def free_slots(self) -> int:
        return self._lib.rg_cache_free_slots(self._h)

    def num_requests(self) -> int:
        return self._lib.rg_cache_num_requests(self._h)

    def check(self) -> None:
        """Raise unless every page and slot is free exactly once or held exactly once."""
        code = self._lib.rg_cache_check(self._h)
        if code:
            self._raise(code, "check")


def group_needs(needs: dict) -> tuple[list, dict, dict]:
    """Sort the mixers' needs into page groups and state buffers.

    ``needs``: cache id -> PagedKVNeed | StateNeed | None.  Returns
    (paged groups as lists of (need, [cache ids]), cache id -> group index,
    cache id -> StateNeed)."""
    groups: list = []
    group_of: dict = {}
    states: dict = {}
    for cid, need in needs.items():
        if need is None:
            continue
        if isinstance(need, StateNeed):
            states[cid] = need
            continue
        if not isinstance(need, PagedKVNeed):
            raise CacheError(f"cache id {cid}: unknown kind of need {need!r}")
        for gi, (gneed, cids) in enumerate(groups):
            if gneed == need:
                cids.append(cid)
                group_of[cid] = gi
                break
        else:
            groups.append((need, [cid]))
            group_of[cid] = len(groups) - 1
    return groups, group_of, states


class CacheManager:
    """Pages and state slots of one model on one device.

    ``page_size`` and ``max_tokens`` (tokens a group's pool holds, rounded up
    to whole pages) are what a group gets whose need does not ask for its own;
    ``dtype`` likewise.  ``max_requests``: state slots, the most requests live
    at a time."""

    def __init__(self, needs: dict, page_size: int, max_tokens: int, max_requests: int, dtype, device):
        import torch
        groups, self.group_of, self.state_needs = group_needs(needs)
        self.groups = []
        for need, cids in groups:
            ps = int(need.page_size or page_size)
            if ps < 1:
                raise CacheError(f"a page must hold at least one token, not {ps}")
            self.groups.append(GroupInfo(need, ps, (int(need.pool_tokens or max_tokens) + ps - 1) // ps, cids))
        self.alloc = PageAllocator([g.page_size for g in self.groups], [g.num_pages for g in self.groups],
                                   [g.need.window for g in self.groups], max_requests)
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = device
        self.kv: dict = {}
        for g in self.groups:
            page_dtype = getattr(torch, g.need.dtype) if g.need.dtype else dtype
            for cid in g.cache_ids:
                self.kv[cid] = torch.zeros((g.num_pages, *g.need.shape_of_page(g.page_size)), dtype=page_dtype,
                                           device=device)
        self.state: dict = {}
        for cid, need in self.state_needs.items():
            self.state[cid] = torch.zeros((self.max_requests, *need.shape), dtype=getattr(torch, need.dtype),
                                          device=device)

    def page_size_of(self, cache_id) -> int:
        return self.groups[self.group_of[cache_id]].page_size

    def bytes_per_token(self) -> int:
        return sum(t.element_size() * t[0].numel() // self.page_size_of(cid) for cid, t in self.kv.items())
