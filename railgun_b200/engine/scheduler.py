"""Python face of the C++ scheduler (``csrc/host/scheduler.hpp``).

Names follow the reference's SchedulerConfig
(crates/vllm-scheduler/src/scheduler.rs:31-58): max_num_batched_tokens 4096,
max_num_seqs 256, max_model_len 4096; ``max_prefill_chunk`` is added (0: a
portion of a prompt is bounded by the token budget alone).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from ..cache.manager import _lib
from .request import FINISH_REASONS


class SchedulerError(ValueError):
    pass


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 4096
    max_num_seqs: int = 256
    max_prefill_chunk: int = 0
    max_model_len: int = 4096


@dataclass
class ScheduledEntry:
    request_id: int
    start: int
    tokens: np.ndarray
    want_last: bool


_ADD_ERRORS = {-1: "the prompt is empty", -2: "prompt + max_new_tokens exceeds max_model_len",
               -3: "a request with this id exists",
               -5: "max_new_tokens must be >= 1, temperature >= 0, top_k >= 0 and top_p in (0, 1]"}


class Scheduler:
    def __init__(self, allocator, config: SchedulerConfig | None = None):
        self.config = config or SchedulerConfig()
        self._lib = _lib()
        self._alloc = allocator            # keeps the C++ cache manager alive
        c = self.config
        self._h = self._lib.rg_sched_create(allocator.handle, c.max_num_batched_tokens, c.max_num_seqs,
                                            c.max_prefill_chunk, c.max_model_len)
        if not self._h:
            raise SchedulerError(f"invalid scheduler configuration {c}")
        cap_e = max(8, c.max_num_seqs)
        self._ids = np.empty(cap_e, dtype=np.int64)
        self._start = np.empty(cap_e, dtype=np.int32)
        self._count = np.empty(cap_e, dtype=np.int32)
        self._want = np.empty(cap_e, dtype=np.int32)
        self._tokens = np.empty(max(8, c.max_num_batched_tokens), dtype=np.int32)
        self._scratch = np.empty(1024, dtype=np.int64)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.rg_sched_destroy(h)

    def add_request(self, request_id: int, prompt, max_new_tokens: int, stop_token_ids=(), temperature: float = 0.0,
                    top_k: int = 0, top_p: float = 1.0, seed: int = 0) -> None:
        """The request with its sampling parameters (the reference's SamplingParams,
        crates/vllm-scheduler/src/request.rs:37-76, and a seed): the scheduler keeps them and writes them
        into the request's slot record whenever it gives the request a slot."""
        p = np.ascontiguousarray(prompt, dtype=np.int32)
        s = np.ascontiguousarray(list(stop_token_ids), dtype=np.int32)
        code = self._lib.rg_sched_add_request(self._h, int(request_id), p.ctypes.data, p.size,
                                              int(max_new_tokens), s.ctypes.data, s.size, float(temperature),
                                              int(top_k), float(top_p), int(seed) & ((1 << 64) - 1))
        if code:
            raise SchedulerError(f"request {request_id}: {_ADD_ERRORS.get(code, code)}")

    def schedule_flat(self):
        """Decide the next step and return it as arrays (views, valid until the
        next call): request ids [n], start positions [n], token counts [n],
        wants-logits flags [n], and all tokens one after the other."""
        n = self._schedule_raw()
        total = int(self._count[:n].sum()) if n else 0
        return self._ids[:n], self._start[:n], self._count[:n], self._want[:n], self._tokens[:total]

    def schedule(self) -> list:
        """Decide the next step: a list of ScheduledEntry (maybe empty)."""
        n = self._schedule_raw()
        out, off = [], 0
        for i in range(n):
            c = int(self._count[i])
            out.append(ScheduledEntry(int(self._ids[i]), int(self._start[i]), self._tokens[off:off + c].copy(),
                                      bool(self._want[i])))
            off += c
        return out

    def _schedule_raw(self) -> int:
        n = self._lib.rg_sched_schedule(self._h, self._ids.ctypes.data, self._start.ctypes.data,
                                        self._count.ctypes.data, self._want.ctypes.data, self._ids.size,
                                        self._tokens.ctypes.data, self._tokens.size)
        if n <= -1000000:
            need = -(n + 1000000)
            self._tokens = np.empty(max(need, 2 * self._tokens.size), dtype=np.int32)
            for name in ("_ids", "_start", "_count", "_want"):
                a = getattr(self, name)
                setattr(self, name, np.empty(2 * a.size + need, dtype=a.dtype))
            n = self._lib.rg_sched_fetch(self._h, self._ids.ctypes.data, self._start.ctypes.data,
                                         self._count.ctypes.data, self._want.ctypes.data, self._ids.size,
                                         self._tokens.ctypes.data, self._tokens.size)
        if n < 0:
            raise SchedulerError(f"schedule failed with status {n}")
        return n

    def preempted(self) -> list:
        n = self._lib.rg_sched_preempted(self._h, self._scratch.ctypes.data, self._scratch.size)
        return [int(x) for x in self._scratch[:min(n, self._scratch.size)]]

    def update(self, request_ids, tokens) -> int:
        """The step ran; ``tokens[i]`` was sampled for ``request_ids[i]``.  Returns how many finished."""
        ids = np.ascontiguousarray(request_ids, dtype=np.int64)
        tk = np.ascontiguousarray(tokens, dtype=np.int32)
        n = self._lib.rg_sched_update(self._h, ids.ctypes.data, tk.ctypes.data, ids.size)
        if n < 0:
            raise SchedulerError(f"update failed with status {n}")
        return n

    def next_step_predictable(self) -> bool:
        """Whether the decision after the one just made is known already, unless
        a stop token ends a request or a request arrives: all running requests
        decode, none can end by length at this step and nothing was preempted
        (a request that waits was refused in this decision and stays refused
        until a request ends)."""
        return bool(self._lib.rg_sched_next_step_predictable(self._h))

    def abort(self, request_id: int) -> None:
        if self._lib.rg_sched_abort(self._h, int(request_id)) != 0:
            raise SchedulerError(f"abort: unknown request {request_id}")

    def finished(self) -> list:
        n = self._lib.rg_sched_finished(self._h, self._scratch.ctypes.data, self._scratch.size)
        if n > self._scratch.size:
            self._scratch = np.empty(2 * n, dtype=np.int64)
            n = self._lib.rg_sched_finished(self._h, self._scratch.ctypes.data, self._scratch.size)
        return [int(x) for x in self._scratch[:n]]

    def finish_reason(self, request_id: int):
        code = self._lib.rg_sched_finish_reason(self._h, int(request_id))
        if code < 0:
            raise SchedulerError(f"unknown request {request_id}")
        return FINISH_REASONS[code]

    def num_generated(self, request_id: int) -> int:
        n = self._lib.rg_sched_num_generated(self._h, int(request_id))
        if n < 0:
            raise SchedulerError(f"unknown request {request_id}")
        return n

    def num_generated_many(self, request_ids: np.ndarray) -> np.ndarray:
        """The count of generated tokens of every request in ``request_ids`` (int64), as int64."""
        ids = np.ascontiguousarray(request_ids, dtype=np.int64)
        out = np.empty(ids.size, dtype=np.int64)
        if self._lib.rg_sched_num_generated_many(self._h, ids.ctypes.data, ids.size, out.ctypes.data) != 0:
            raise SchedulerError("num_generated_many: an unknown request")
        return out

    def sampling_many(self, request_ids) -> dict:
        """The sampling parameters of the requests as arrays (``temperature``, ``top_k``, ``top_p``, ``seed``) and
        the number of each one's next draw (``counter`` = tokens generated so far)."""
        ids = np.ascontiguousarray(request_ids, dtype=np.int64)
        n = ids.size
        out = dict(temperature=np.empty(n, np.float32), top_k=np.empty(n, np.int32), top_p=np.empty(n, np.float32),
                   seed=np.empty(n, np.int64), counter=np.empty(n, np.int64))
        if self._lib.rg_sched_sampling_many(self._h, ids.ctypes.data, n, out["temperature"].ctypes.data,
                                            out["top_k"].ctypes.data, out["top_p"].ctypes.data, out["seed"].ctypes.data,
                                            out["counter"].ctypes.data) != 0:
            raise SchedulerError("sampling_many: an unknown request")
        return out

    def num_preemptions(self, request_id: int) -> int:
        return self._lib.rg_sched_num_preemptions(self._h, int(request_id))

    def outputs(self, request_id: int) -> list:
        n = self.num_generated(request_id)
        buf = np.empty(max(1, n), dtype=np.int32)
        self._lib.rg_sched_outputs(self._h, int(request_id), buf.ctypes.data, buf.size)
        return buf[:n].tolist()

    def error(self, request_id: int):
        import ctypes
        buf = ctypes.create_string_buffer(256)
        n = self._lib.rg_sched_error(self._h, int(request_id), buf, 256)
        return buf.value.decode() if n else None

    def forget(self, request_id: int) -> None:
        self._lib.rg_sched_forget(self._h, int(request_id))

    @property
    def num_waiting(self) -> int:
        return self._lib.rg_sched_num_waiting(self._h)

    @property
    def num_running(self) -> int:
        return self._lib.rg_sched_num_running(self._h)
