"""The step function: model, cache and kernels behind one call.

``ModelRunner.step(entries)`` runs exactly the tokens it is given, as one
batch, from the cache that earlier steps left, and returns the logits at the
wanted places.  Generation, the scheduler and trace replay all go through it.
The reference's counterpart is execute_model_step -> forward_packed
(crates/vllm-engine/src/engine.rs:175-286,
crates/vllm-models/src/llama/architecture.rs:141-156).
"""
from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from ..config.registry import load_config
from ..parts.base import CacheView
from ..parts.model import DecoderModel, TensorBank, expected_tensors
from ..parts.spec import BuildEnv
from ..weights.loader import load_weights
from .batch import StepEntry, build_step_batch

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


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
            self._views[cid] = CacheView(cid, group=cache.group_of[cid], kv=t, page_size=cache.page_size)
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


class ModelRunner:
    """A model on one GPU with its cache.

    ``max_tokens``: tokens the cache pool holds; ``max_requests``: requests
    live at a time; ``page_size``: tokens per page (the reference's
    ``--block-size``, default 16, crates/vllm-scheduler/src/scheduler.rs:53)."""

    def __init__(self, model_dir, dtype="bfloat16", device="cuda:0", page_size: int = 16,
                 max_tokens: int = 16384, max_requests: int = 64, spec_override=None):
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

    @property
    def alloc(self):
        return self.cache.alloc

    def step(self, entries) -> torch.Tensor | None:
        """Run one batch; float32 logits [wanted, vocab] in the order of the
        entries and of each entry's ``want``, or None if nothing is wanted."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        batch = build_step_batch(entries, self.alloc, self.page_sizes, self.model.vocab_size,
                                 self.model.spec.max_position, self.device, self.err_flag)
        logits = self.model.forward(batch, self.views)
        for e, start in zip(entries, batch.host_start_pos):
            self.alloc.commit(e.request_id, int(start) + len(e.tokens))
        return logits

    def end(self, request_ids) -> None:
        """The requests are finished: their pages and slots come back."""
        for rid in request_ids:
            if self.alloc.has(rid):
                self.alloc.release(rid)

    def check_device_errors(self) -> None:
        if int(self.err_flag.item()):
            self.err_flag.zero_()
            raise RuntimeError("a kernel met a position outside its table")
