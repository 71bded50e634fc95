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
from ctypes import c_int, c_longlong, c_void_p, POINTER
from dataclasses import dataclass

import numpy as np

from .. import native


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


@dataclass(frozen=True)
class PagedKVNeed:
    """Keys and values in pages: what an attention-like mixer asks for."""
    num_kv_heads: int
    head_dim: int
    window: int = 0            # 0: all keys are kept


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
        lib.rg_cache_pack_decode.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int]
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
        lib.rg_sched_add_request.argtypes = [c_void_p, c_longlong, c_void_p, c_int, c_int, c_void_p, c_int]
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


class PageAllocator:
    """The C++ cache manager: page groups, block tables, state slots.  No device memory."""

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

    def pack_decode(self, ids: np.ndarray, B: int, MB: int, out: np.ndarray, ahead: int = 0) -> None:
        """Reserve one more token for each request in ``ids`` (int64) and write
        the decode step's positions, slots and block tables into ``out``
        (int32; layout in csrc/host/runtime.cpp, rg_cache_pack_decode).
        ``ahead`` = 1 packs the step after a step that is launched but not yet
        committed."""
        code = self._lib.rg_cache_pack_decode(self._h, ids.ctypes.data, ids.size, B, MB, out.ctypes.data, int(ahead))
        if code:
            self._raise(code, "pack_decode")

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

    ``max_tokens``: tokens the pool of every group holds (rounded up to whole
    pages); ``max_requests``: state slots, the most requests live at a time."""

    def __init__(self, needs: dict, page_size: int, max_tokens: int, max_requests: int, dtype, device):
        import torch
        groups, self.group_of, self.state_needs = group_needs(needs)
        self.page_size = int(page_size)
        num_pages = (int(max_tokens) + self.page_size - 1) // self.page_size
        self.groups = [GroupInfo(need, self.page_size, num_pages, cids) for need, cids in groups]
        self.alloc = PageAllocator([self.page_size] * len(groups), [num_pages] * len(groups),
                                   [g.need.window for g in self.groups], max_requests)
        self.max_requests = int(max_requests)
        self.dtype = dtype
        self.device = device
        self.kv: dict = {}
        for g in self.groups:
            for cid in g.cache_ids:
                self.kv[cid] = torch.zeros((num_pages, 2, g.need.num_kv_heads, self.page_size, g.need.head_dim),
                                           dtype=dtype, device=device)
        self.state: dict = {}
        for cid, need in self.state_needs.items():
            self.state[cid] = torch.zeros((self.max_requests, *need.shape), dtype=getattr(torch, need.dtype),
                                          device=device)

    def bytes_per_token(self) -> int:
        return sum(t.element_size() * t[0].numel() // self.page_size for t in self.kv.values())
