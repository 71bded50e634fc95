"""The step function: model, cache and kernels behind one call.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one
batch, from the cache that earlier steps left, and returns the logits at the
wanted places.  Generation, the scheduler and trace replay all go through it.
The reference's counterpart is execute_model_step -> forward_packed
(crates/vllm-engine/src/engine.rs:175-286,
crates/vllm-models/src/llama/architecture.rs:141-156).

How a step reaches the GPU: steps of single tokens replay a CUDA graph over a
static batch (``decode_step_flat``; the graph copies its inputs in, chooses
the tokens and copies them out), and the step after such a step can be
launched before its tokens are known (``decode_follow``); large steps whose
packed layout repeats replay a graph captured for that layout
(``_step_shape_graph``); everything else launches its kernels one by one.
"""
from __future__ import annotations

import contextlib
import dataclasses
import gc
import os

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..parts.base import CacheView
from ..parts.model import DecoderModel, TensorBank, expected_tensors
from ..parts.spec import BuildEnv
from ..weights.loader import load_weights
from .. import ops
from ..cache.manager import CacheError
from .batch import BatchError, StepBatch, StepEntry, build_step_batch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


# Steps of at least this many tokens go through a graph captured for their layout once that layout repeats
# (below it the launches are few and short; single tokens have their own graphs), and so many layouts are kept.
SHAPE_GRAPH_MIN_TOKENS = 256
SHAPE_GRAPHS_KEPT = 4


@contextlib.contextmanager
def capture(graph):
    """``torch.cuda.graph(graph)`` with Python's cyclic garbage collector held off: a collection in the middle of
    a capture may free a page-locked host buffer of an earlier step, and freeing one records an event on the
    stream that used it, which is not allowed on a capturing stream and invalidates the capture."""
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
    finally:
        if was_enabled:
            gc.enable()


def raise_device_error(code: int):
    """What a kernel left in an error flag: 1 for a position outside its table."""
    if code == 1:
        raise RuntimeError("a kernel met a position outside its table")
    raise RuntimeError(f"a kernel flagged error {code}; the step's result is invalid")


# RAILGUN_B200_NVTX=1 puts a named range around every step (visible in a profiler's timeline).
NVTX = os.environ.get("RAILGUN_B200_NVTX", "0") == "1"


def parse_dtype(name):
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype {name} is not supported: bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is not supported: bfloat16 or float32") from None


class _CacheViews:
    def __init__(self, cache: CacheManager):
        self._views = {}
        for cid, t in cache.kv.items():
            self._views[cid] = CacheView(cid, group=cache.group_of[cid], kv=t, page_size=cache.page_size_of(cid))
        for cid, t in cache.state.items():
            self._views[cid] = CacheView(cid, state=t)
        self._none = {}

    def view(self, cid):
        v = self._views.get(cid)
        if v is None:
            v = self._none.setdefault(cid, CacheView(cid))
        return v


def build_model(model_dir, dtype, device, spec_override=None):
    """Read config.json, pick the architecture from the registry, load the
    weights by name and build the model.  Returns (architecture, config, model)."""
    arch, cfg = load_config(model_dir)
    spec = spec_override(cfg) if spec_override else arch.model_spec(cfg)
    expected = expected_tensors(spec)
    tensors = load_weights(model_dir, expected, device="cpu", allow_unexpected=arch.allow_unexpected(cfg))
    env = BuildEnv(device=device, dtype=dtype, hidden_size=spec.hidden_size, max_position=spec.max_position)
    model = DecoderModel(spec, env, TensorBank(tensors, device))
    return arch, cfg, model


_BATCH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256, 384, 512)


def _bucket(n: int, buckets) -> int:
    for b in buckets:
        if n <= b:
            return b
    return n


class StaticDecodeBatch:
    """Device buffers of fixed address for decode steps of up to ``B`` requests
    whose contexts stay within ``MB`` pages, with the pinned host buffer that
    is copied into them in one transfer.  A graph captured over these buffers
    can be replayed for any such step.  Layout (int32): token ids | positions |
    context lengths | start positions | state slots | per group slot mapping |
    per group block table [B, MB] | the rows' sampling parameters (seed and
    draw counter as 64-bit, temperature, top-k, top-p)."""

    def __init__(self, runner, B: int, MB: int):
        dev = runner.device
        G = len(runner.page_sizes)
        self.B, self.MB, self.G = B, MB, G
        self.sampling_off = -(-((5 + G) * B + G * B * MB) // 2) * 2          # even: 64-bit values start there
        n_ints = self.sampling_off + 7 * B
        self.host = torch.zeros(n_ints, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        # the step's tokens and, behind them, the flag that a kernel raises for a position outside its table:
        # one copy by the graph brings both to the host
        self.host_out = torch.zeros(B + 1, dtype=torch.int32, pin_memory=True)
        self.host_out_np = self.host_out.numpy()
        self.out_dev = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        self.dev = torch.zeros(n_ints, dtype=torch.int32, device=dev)
        seg = lambda i: self.dev[i * B:(i + 1) * B]
        ar = torch.arange(B + 1, dtype=torch.int32, device=dev)
        tables_off = (5 + G) * B
        self.batch = StepBatch(
            num_tokens=B, num_requests=B, num_wanted=B, max_query_len=1,
            max_context_len=MB * (min(runner.page_sizes) if G else 1),
            token_ids=seg(0), positions=seg(1), req_of_token=ar[:B], want_rows=ar[:B], cu_seqlens=ar,
            context_lens=seg(2), start_pos=seg(3), state_slots=seg(4),
            slot_mapping=[seg(5 + g) for g in range(G)],
            block_table=[self.dev[tables_off + g * B * MB:tables_off + (g + 1) * B * MB].view(B, MB)
                         for g in range(G)],
            err_flag=self.out_dev[B:], decode_only=True)
        self.sampling = sampling_views(self.dev, self.sampling_off, B)        # device views of the sampling parameters
        self.sampled = self.out_dev[:B]                                         # the tokens the last step chose
        self.step_graphs = {}          # with sampling parameters or greedy -> CapturedStep
        self.follow = [None, None]     # FollowStep: the same step fed with ``sampled`` instead of host tokens
        self.in_flight = None          # an event after the last replay that reads ``host`` and writes ``host_out``

    def raise_if_flagged(self, host_out_np) -> None:
        code = int(host_out_np[self.B])
        if code:
            self.out_dev[self.B:].zero_()
            host_out_np[self.B] = 0
            raise_device_error(code)

    def wait_until_reusable(self) -> None:
        """The pinned buffers may be written again once the last replay that copies them has run."""
        if self.in_flight is not None and not self.in_flight.query():
            self.in_flight.synchronize()

    def upload(self) -> int:
        self.dev.copy_(self.host, non_blocking=True)
        return self.host.numel() * 4


def sampling_views(buf, off: int, B: int) -> dict:
    """The sampling parameters inside a packed decode buffer (a torch tensor or a numpy array of int32)."""
    f32, i64 = (torch.float32, torch.int64) if isinstance(buf, torch.Tensor) else (np.float32, np.int64)
    return dict(seed=buf[off:off + 2 * B].view(i64), counter=buf[off + 2 * B:off + 4 * B].view(i64),
                temperature=buf[off + 4 * B:off + 5 * B].view(f32), top_k=buf[off + 5 * B:off + 6 * B],
                top_p=buf[off + 6 * B:off + 7 * B].view(f32))


class FollowStep:
    """A decode step launched before the tokens of the step before it are on the
    host: its graph takes positions, slots and block tables from this object's
    own pinned buffer, the token ids from the static batch's ``sampled``, and
    copies its greedy tokens into this object's pinned ``host_out``.  Two of
    them alternate per static batch, so that a step in flight never shares a
    pinned buffer with the step that is being read."""

    def __init__(self, static: StaticDecodeBatch):
        self.static = static
        self.host_in = torch.zeros(static.host.numel(), dtype=torch.int32, pin_memory=True)
        self.host_in_np = self.host_in.numpy()
        self.host_out = torch.zeros(static.B + 1, dtype=torch.int32, pin_memory=True)
        self.host_out_np = self.host_out.numpy()
        self.done = torch.cuda.Event()
        self.captured = {}             # with sampling parameters or greedy -> CapturedStep
        self.ids = None                # the requests of the launched step, in row order

    def tokens(self) -> np.ndarray:
        """The launched step's tokens, one per row (waits for the step; raises if a kernel of it flagged an error)."""
        self.done.synchronize()
        self.static.raise_if_flagged(self.host_out_np)
        return self.host_out_np[:self.static.B]


class ShapeGraph:
    """A captured step for one packed layout: the static device buffer the step's
    data is copied into, the batch whose tensors are views of it, the graph and
    its output."""

    def __init__(self, dev, batch, graph, logits, launches):
        self.dev, self.batch, self.graph, self.logits, self.launches = dev, batch, graph, logits, launches
        self.hold = None               # the last packed step (keeps its pinned buffer alive until the copy has run)


class CapturedStep:
    def __init__(self, graph, logits, sampled, launches):
        self.graph, self.logits, self.sampled, self.launches = graph, logits, sampled, launches


class ModelRunner:
    """A model on one GPU with its cache.

    ``max_tokens``: tokens the cache pool holds; ``max_requests``: requests
    live at a time; ``page_size``: tokens per page (the reference's
    ``--block-size``, default 16, crates/vllm-scheduler/src/scheduler.rs:53).
    ``use_graphs``: steps in which every request brings exactly one token and
    wants its logits are replayed from a captured CUDA graph."""

    def __init__(self, model_dir, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 max_tokens: int = 16384, max_requests: int = 64, spec_override=None, use_graphs: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("railgun_b200 runs on a CUDA device only; none is available")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        # 32-bit means 32-bit: no reduced-precision matrix mode, no reduced-precision accumulation
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
        self.arch, self.config, self.model = build_model(model_dir, self.dtype, self.device, spec_override)
        self.cache = CacheManager(self.model.cache_needs(), page_size, max_tokens, max_requests,
                                  self.dtype, self.device)
        self.views = _CacheViews(self.cache)
        self.page_sizes = [g.page_size for g in self.cache.groups]
        self.err_flag = torch.zeros(1, dtype=torch.int32, device=self.device)
        # graphs need every part to work from device-side descriptions only; a part that says it plans on the
        # host (none of the built-in ones) switches them off.  Per-request state is no obstacle: its buffers are
        # static and the rows' slots are data of the step (-1 in a padding row).
        self.use_graphs = bool(use_graphs) and self.model.graph_safe
        self._static: dict = {}
        self._shape_steps: dict = {}       # layout -> ShapeGraph: steps of a layout seen before replay a captured graph
        self._shape_seen: dict = {}
        self.shape_graph_min_tokens = SHAPE_GRAPH_MIN_TOKENS
        self._graph_pool = None
        self._ctx_hint = 0
        self.last_h2d_bytes = 0
        self.last_greedy = None
        self._greedy_host = None

    @property
    def alloc(self):
        return self.cache.alloc

    # ---- the step function -----------------------------------------------------------------------
    def step(self, entries) -> torch.Tensor | None:
        """Run one batch; float32 logits [wanted, vocab] in the order of the
        entries and of each entry's ``want``, or None if nothing is wanted.
        The result may be a view of a buffer the next step overwrites."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if NVTX:
            torch.cuda.nvtx.range_push(f"step {len(entries)} requests {sum(len(e.tokens) for e in entries)} tokens")
            try:
                return self._step(entries)
            finally:
                torch.cuda.nvtx.range_pop()
        return self._step(entries)

    def _step(self, entries):
        self.last_greedy = None
        if self.use_graphs and entries and all(
                len(e.tokens) == 1 and list(e.want) == [0] and self.alloc.has(e.request_id) for e in entries):
            return self._step_decode_graph(entries)
        if self.use_graphs and sum(len(e.tokens) for e in entries) >= self.shape_graph_min_tokens:
            return self._step_shape_graph(entries)
        batch = build_step_batch(entries, self.alloc, self.page_sizes, self.model.vocab_size,
                                 self.model.spec.max_position, self.device, self.err_flag)
        self.last_h2d_bytes = batch.h2d_bytes
        logits = self.model.forward(batch, self.views)
        self._commit(entries, batch)
        return logits

    def _commit(self, entries, batch) -> None:
        self.alloc.commit_many(batch.host_request_ids, batch.host_context_lens)

    def _step_shape_graph(self, entries):
        """Large steps (portions of prompts) whose packed layout was seen before
        replay a CUDA graph captured for that layout: token counts, wanted places
        and block-table widths fix every shape, everything else is data in the
        step's one device buffer.  The first step of a layout runs eagerly, the
        second is captured while it runs, later ones replay; a few layouts
        (the portions a scheduler cuts are mostly of one size) are kept."""
        build = lambda into: build_step_batch(entries, self.alloc, self.page_sizes, self.model.vocab_size,
                                              self.model.spec.max_position, self.device, self.err_flag, into=into)
        known = lambda layout: self._shape_steps[layout].dev if layout in self._shape_steps else None
        batch = build(known)
        self.last_h2d_bytes = batch.h2d_bytes
        key = batch.layout
        shape = self._shape_steps.get(key)
        if shape is not None:
            # the step was packed straight into the graph's buffer: launch
            shape.hold = batch
            shape.graph.replay()
            ops.launch_counter().value += shape.launches
            ops.mark_tc_unchecked()
            self._commit(entries, batch)
            return shape.logits
        seen = self._shape_seen.get(key, 0) + 1
        if len(self._shape_seen) > 64:
            self._shape_seen.clear()
        self._shape_seen[key] = seen
        if seen < 2:
            logits = self.model.forward(batch, self.views)
            self._commit(entries, batch)
            return logits
        # the layout repeats: a static copy of the packed buffer, one eager run over it (this step), the capture
        if len(self._shape_steps) >= SHAPE_GRAPHS_KEPT:
            self._shape_steps.pop(next(iter(self._shape_steps)))
        dev = torch.empty(batch.host_buffer.numel(), dtype=torch.int32, device=self.device)
        batch = build(lambda layout: dev)
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            eager = self.model.forward(batch, self.views)
            eager = eager.clone() if eager is not None else None
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        counter = ops.launch_counter()
        n0 = counter.value
        graph = torch.cuda.CUDAGraph()
        with capture(graph):
            logits = self.model.forward(batch, self.views)
        launches = counter.value - n0
        counter.value = n0
        self._shape_steps[key] = ShapeGraph(dev, batch, graph, logits, launches)
        self._commit(entries, batch)
        return eager

    def end(self, request_ids) -> None:
        """The requests are finished: their pages and slots come back."""
        for rid in request_ids:
            if self.alloc.has(rid):
                self.alloc.release(rid)

    def check_device_errors(self) -> None:
        """Raise if a kernel gave up a bounded wait or met a position outside its table since the last check
        (synchronises).  Steps replayed from decode graphs carry their own flag, which also travels to the host
        with their tokens."""
        ops.tc_gemm_check()
        flags = [self.err_flag] + [st.out_dev[st.B:] for st in self._static.values()]
        code = int(torch.cat(flags).max().item())
        if code:
            for f in flags:
                f.zero_()
            raise_device_error(code)

    # ---- decode steps from captured graphs -----------------------------------------------------------
    def _static_for(self, n_requests: int, max_context: int) -> StaticDecodeBatch:
        B = _bucket(n_requests, _BATCH_BUCKETS)
        # block tables are as wide as the group with the smallest pages needs
        page = min(self.page_sizes) if self.page_sizes else 16
        ctx_bucket = 1024
        while ctx_bucket < max_context:
            ctx_bucket *= 2
        key = (B, -(-ctx_bucket // page))
        if key not in self._static:
            self._static[key] = StaticDecodeBatch(self, *key)
        return self._static[key]

    def _capture(self, static: StaticDecodeBatch, follow: FollowStep | None = None,
                 sampling: bool = False) -> CapturedStep:
        """Capture one decode step over the static buffers: the copy of its
        packed inputs from pinned memory, the forward pass, the choice of the
        tokens and their copy to pinned memory, so that one graph launch and one
        wait are all the host does.  With ``follow`` the step takes its token
        ids from the step before it on the device and everything else from
        ``follow``'s pinned buffer.  With ``sampling`` the tokens are drawn with
        the rows' parameters in the static buffer (temperature 0: greedy)
        instead of the plain argmax.

        The step whose arrival makes the capture necessary runs here, once,
        outside the capture (libraries set themselves up in that run); the
        graph serves the steps after it.  So a step is executed exactly once,
        which a part with state of its own needs (rewriting a cache entry is
        harmless, advancing a state twice is not).  Returns the captured step
        and that first run's logits."""
        counter = ops.launch_counter()
        B = static.B

        def body():
            if follow is not None:
                static.dev[B:].copy_(follow.host_in[B:], non_blocking=True)
            else:
                static.dev.copy_(static.host, non_blocking=True)
            # a following step reads its token ids where the step before left its greedy tokens
            batch = static.batch if follow is None else dataclasses.replace(static.batch, token_ids=static.sampled)
            logits = self.model.forward(batch, self.views)
            if sampling:
                sp = static.sampling
                sampled = ops.sample(logits, sp["temperature"], sp["top_k"], sp["top_p"], sp["seed"],
                                     sp["counter"], out=static.sampled)
            else:
                sampled = ops.argmax(logits, out=static.sampled)
            (follow or static).host_out.copy_(static.out_dev, non_blocking=True)
            return logits, sampled

        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            first_logits, _ = body()                        # this step itself
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = counter.value
        with capture(graph):
            logits, sampled = body()
        launches = counter.value - n0
        counter.value = n0
        return CapturedStep(graph, logits, sampled, launches), first_logits

    def _step_decode_graph(self, entries) -> torch.Tensor:
        R = len(entries)
        ids = np.fromiter((e.request_id for e in entries), dtype=np.int64, count=R)
        tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=R)
        if len(set(ids.tolist())) != R:
            raise BatchError("a request appears twice in one step")
        return self.decode_step_flat(ids, tokens)

    def decode_step_flat(self, ids: np.ndarray, tokens: np.ndarray) -> torch.Tensor:
        """One decode step for requests already in the cache: ``ids`` int64
        (distinct), ``tokens`` int32, one token each, logits wanted for all.
        Returns the logits [R, V] (a view of a static buffer); the tokens the
        graph chose are in ``last_greedy``: for a request whose slot record has
        a temperature above zero a draw with the record's parameters (numbered
        by its count of generated tokens), else the argmax."""
        R = len(ids)
        self.last_greedy = None
        if tokens.min() < 0 or tokens.max() >= self.model.vocab_size:
            raise BatchError(f"token ids must be in [0, {self.model.vocab_size})")
        ctx = max(self._ctx_hint + 1, 1)
        while True:
            static = self._static_for(R, ctx)
            static.wait_until_reusable()
            try:
                sampled = self.alloc.pack_decode(ids, static.B, static.MB, static.host_np[static.B:],
                                                 sampling=static.host_np[static.sampling_off:])
                break
            except CacheError as e:
                if "bad argument" in str(e) and ctx < self.model.spec.max_position:
                    ctx = min(2 * max(ctx, 1024), self.model.spec.max_position)
                    continue
                raise
        B = static.B
        self._ctx_hint = int(static.host_np[2 * B:2 * B + R].max())
        if self._ctx_hint > self.model.spec.max_position:
            raise BatchError(f"position {self._ctx_hint - 1} is beyond the model's max_position_embeddings "
                             f"{self.model.spec.max_position}")
        static.host_np[:R] = tokens
        static.host_np[R:B] = 0
        self.last_h2d_bytes = static.host.numel() * 4
        key = sampled
        logits = None
        if key not in static.step_graphs:
            static.step_graphs[key], logits = self._capture(static, sampling=key)   # runs this step and captures it
        cap = static.step_graphs[key]
        if logits is None:
            cap.graph.replay()                              # upload, the step, greedy tokens back to pinned memory
            ops.launch_counter().value += cap.launches
            logits = cap.logits
        if static.in_flight is None:
            static.in_flight = torch.cuda.Event()
        static.in_flight.record()
        self.alloc.advance(ids, 1)
        self.last_greedy = cap.sampled[:R]
        self._greedy_host = (static, R)
        return logits[:R]

    def greedy_tokens_host(self):
        """The tokens that the last graph-replayed decode step chose (its argmax,
        or its draws if it was given sampling parameters) as a numpy array; waits
        for the step, whose graph copied them to pinned memory itself.  None if
        the last step was not such a step."""
        if self.last_greedy is None or self._greedy_host is None:
            return None
        static, R = self._greedy_host
        static.in_flight.synchronize()
        static.raise_if_flagged(static.host_out_np)
        return static.host_out_np[:R].copy()

    def decode_follow(self, ids: np.ndarray, after) -> FollowStep | None:
        """Launch the decode step that follows a launched one for the same
        requests (``ids`` int64, in its row order) before that one's tokens are
        on the host: the token ids stay on the device.  ``after`` is what that
        step ran on: the FollowStep it was, or None for the step that
        ``decode_step_flat`` launched last.  Its draws are numbered one after
        those of that step.  Nothing is committed: the caller
        commits the step once it knows that the requests went on.  Returns None
        if the step cannot be launched this way (no pages, a context beyond the
        static batch's tables or the model's positions)."""
        if after is None:
            if self._greedy_host is None:
                return None
            static, R = self._greedy_host
            k = 0
        else:
            static, R = after.static, len(after.ids)
            k = 1 - static.follow.index(after)
        if R != len(ids):
            return None
        if static.follow[k] is None:
            static.follow[k] = FollowStep(static)
        f = static.follow[k]
        if not f.done.query():                              # only after a launch that was dropped: its copies may be pending
            f.done.synchronize()
        B = static.B
        ahead = 0 if after is None else 1                   # decode_step_flat has advanced its requests already
        try:
            key = self.alloc.pack_decode(ids, B, static.MB, f.host_in_np[B:], ahead=ahead,
                                         sampling=f.host_in_np[static.sampling_off:], draw_ahead=1)
        except CacheError:
            return None
        if int(f.host_in_np[2 * B:2 * B + R].max()) > self.model.spec.max_position:
            return None
        if key not in f.captured:
            f.captured[key], _ = self._capture(static, follow=f, sampling=key)       # runs this step and captures it
        else:
            f.captured[key].graph.replay()
            ops.launch_counter().value += f.captured[key].launches
        f.done.record()
        self.last_h2d_bytes = (static.host.numel() - B) * 4
        f.ids = ids.copy()
        return f
