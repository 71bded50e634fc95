"""The Python entry point: ``Engine(model_dir, ...).generate(prompt_ids, params)``.

The loop is the reference's engine loop without the async plumbing
(crates/vllm-engine/src/engine.rs:82-163): schedule -> one model step on the
packed batch -> sample at each request's last position -> update the
scheduler -> collect finished requests.  Option names are the reference's
(crates/vllm-cli/src/serve.rs:44-77, docs/cli-configuration.md:7-27):
``dtype``, ``max_num_seqs``, ``max_num_batched_tokens``, ``block_size``,
``num_gpu_blocks``, ``max_model_len``.
"""
from __future__ import annotations

import numpy as np

from .. import ops
from ..sampling.sampler import Sampler
from .batch import StepEntry, _token_array
from .request import RequestOutput, SamplingParams, StepResponse
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerConfig


class Engine:
    def __init__(self, model_dir, dtype="bfloat16", cuda_device: int = 0, block_size: int = 16,
                 num_gpu_blocks: int = 1000, max_num_seqs: int = 256, max_num_batched_tokens: int = 4096,
                 max_model_len: int = 4096, max_prefill_chunk: int = 0):
        self.runner = ModelRunner(model_dir, dtype=dtype, device=f"cuda:{cuda_device}", page_size=block_size,
                                  max_tokens=num_gpu_blocks * block_size, max_requests=max_num_seqs)
        max_model_len = min(max_model_len, self.runner.model.spec.max_position)
        self.scheduler = Scheduler(self.runner.alloc, SchedulerConfig(
            max_num_batched_tokens=max_num_batched_tokens, max_num_seqs=max_num_seqs,
            max_prefill_chunk=max_prefill_chunk, max_model_len=max_model_len))
        self.sampler = Sampler(self.runner.device)
        self._next_id = 1
        self.steps_run = 0
        # launch the next decode step before this one's tokens are on the host; not for a model whose parts keep
        # state of their own: a launched step that is then dropped would have advanced it
        self.run_ahead = not self.runner.cache.state
        self._ahead = None             # the step launched that way, if any (runner.FollowStep)
        self.steps_ahead = 0           # how many steps were taken from a launch made ahead

    # ---- low level --------------------------------------------------------------------------
    def add_request(self, prompt_ids, params: SamplingParams | None = None) -> int:
        params = params or SamplingParams()
        params.validate()
        vocab = self.runner.model.vocab_size
        prompt = _token_array(prompt_ids)
        if prompt.size and (prompt.dtype.kind not in "iu" or prompt.min() < 0 or prompt.max() >= vocab):
            raise ValueError(f"prompt token ids must be integers in [0, {vocab})")
        rid = self._next_id
        self._next_id += 1
        # the scheduler keeps the parameters and writes them into the request's slot record, from which decode
        # steps are packed: the request has no second home here
        self.scheduler.add_request(rid, prompt, params.max_new_tokens, params.stop_token_ids, params.temperature,
                                   params.top_k, params.top_p, params.seed)
        return rid

    def step(self) -> list:
        """One scheduler decision and one model step.  Returns the (request id,
        sampled token) pairs of this step, or None if nothing could be scheduled.

        While every running request decodes and none can end by length, the
        step after this one is launched before this one's tokens are read: its
        token ids stay on the device, and its positions and pages are known.
        The next call checks the guess against the scheduler's decision: the
        same requests, or some of them (a stop token ended the others; rows
        are independent), take the launched step's results; anything else
        drops them and runs the decision as usual, which recomputes the same
        cache entries."""
        ids, starts, counts, wants, tokens = self.scheduler.schedule_flat()
        ahead, self._ahead = self._ahead, None
        if len(ids) == 0:
            return None
        self.steps_run += 1
        if self.runner.use_graphs and len(tokens) == len(ids) and bool(wants.all()):
            wanted, sampled = self._decode_step(ids, tokens, ahead)
        else:
            wanted, sampled = self._mixed_step(ids, counts, wants, tokens)
        if sampled is None:
            self.scheduler.update([], [])
            return []
        # the tokens are on the host, so the step has finished: did a kernel give up a wait or meet a bad position?
        # (decode graphs bring their flag back with the tokens, see _decode_step)
        ops.tc_gemm_check()
        self.scheduler.update(wanted, sampled)
        return list(zip(wanted, sampled.tolist()))

    def _decode_step(self, ids, tokens, ahead):
        """Every request brings one token and wants its logits: the step is a graph replay that chooses the
        tokens itself, or the step launched ahead in the call before if it answers this decision."""
        wanted = ids.tolist()
        rows = self._rows_of_launched(ahead, ids) if ahead is not None else None
        launched = ahead if rows is not None else None
        if launched is not None:
            self.steps_ahead += 1
        else:
            self.runner.decode_step_flat(ids, tokens)   # draws or takes the argmax as the requests' records say
        if (self.run_ahead and (launched is None or len(launched.ids) == len(ids))
                and self.scheduler.next_step_predictable()):
            self._ahead = self.runner.decode_follow(ids, launched)
        # only now wait for this step's tokens
        return wanted, (launched.tokens()[rows] if launched is not None else self.runner.greedy_tokens_host())

    def _mixed_step(self, ids, counts, wants, tokens):
        """Portions of prompts, maybe beside decoded tokens: one packed step; the tokens are chosen afterwards
        at the rows that asked for logits."""
        batch, off, wanted = [], 0, []
        for i in range(len(ids)):
            c = int(counts[i])
            rid = int(ids[i])
            batch.append(StepEntry(rid, tokens[off:off + c], [c - 1] if wants[i] else []))
            if wants[i]:
                wanted.append(rid)
            off += c
        logits = self.runner.step(batch)
        if logits is None:
            return wanted, None
        sampled = self.sampler.sample_arrays(logits, self.scheduler.sampling_many(wanted))
        self.runner.check_device_errors()
        return wanted, sampled

    @staticmethod
    def _rows_of_launched(launched, ids):
        """The rows of the step launched ahead that answer the decision ``ids``, or None if it does not cover it."""
        if len(ids) == len(launched.ids) and (ids == launched.ids).all():
            return slice(0, len(ids))
        row = {int(r): i for i, r in enumerate(launched.ids)}
        rows = [row.get(int(r), -1) for r in ids]
        return None if min(rows) < 0 else np.asarray(rows)

    def abort(self, request_id: int) -> None:
        self.scheduler.abort(request_id)

    def collect(self, request_id: int) -> RequestOutput:
        """The outcome of a finished request; the engine forgets it."""
        out = RequestOutput(request_id, self.scheduler.outputs(request_id),
                            self.scheduler.finish_reason(request_id), self.scheduler.error(request_id),
                            self.scheduler.num_preemptions(request_id))
        self.scheduler.forget(request_id)
        return out

    def has_unfinished(self) -> bool:
        return self.scheduler.num_waiting + self.scheduler.num_running > 0

    def stats(self) -> dict:
        return dict(num_waiting=self.scheduler.num_waiting, num_running=self.scheduler.num_running,
                    num_free_blocks=self.runner.alloc.free_pages(0), steps=self.steps_run)

    def stream(self, prompt_ids, params=None):
        """Generate for every prompt and yield a StepResponse for every token as
        the step that made it ends (the reference's receiver of
        EngineStepResponse, crates/vllm-engine/src/engine.rs:64-76); the last
        response of a request has ``is_finished`` and its finish reason.  A
        request that ends without a token (an error, an abort) gets one
        response without a token.  The engine forgets a request once its last
        response has been made."""
        if prompt_ids and isinstance(prompt_ids[0], (int, np.integer)):
            prompt_ids = [prompt_ids]
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompt_ids)
        if len(params) != len(prompt_ids):
            raise ValueError(f"{len(prompt_ids)} prompts but {len(params)} parameter sets")
        open_ids = {self.add_request(list(p), sp) for p, sp in zip(prompt_ids, params)}
        while open_ids:
            made = self.step()
            done = [r for r in self.scheduler.finished() if r in open_ids]
            if made is None and not done and not self.scheduler.preempted():
                raise RuntimeError("the scheduler can make no progress: no request fits the cache")
            out = []
            for rid, token in made or ():
                if rid in open_ids:
                    ended = rid in done
                    out.append(StepResponse(rid, token, ended, self.scheduler.finish_reason(rid) if ended else None))
                    if ended:
                        open_ids.discard(rid)
            for rid in done:
                if rid in open_ids:                                  # ended in this step without a token
                    open_ids.discard(rid)
                    out.append(StepResponse(rid, None, True, self.scheduler.finish_reason(rid)))
            for r in out:
                if r.is_finished:
                    self.scheduler.forget(r.request_id)
            yield from out

    # ---- the call a user makes --------------------------------------------------------------
    def generate(self, prompt_ids, params=None) -> list:
        """Generate for every prompt (lists of token ids); ``params`` is one
        SamplingParams for all or a list with one per prompt.  Returns a
        RequestOutput per prompt, in order."""
        if prompt_ids and isinstance(prompt_ids[0], (int, np.integer)):
            prompt_ids = [prompt_ids]
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompt_ids)
        if len(params) != len(prompt_ids):
            raise ValueError(f"{len(prompt_ids)} prompts but {len(params)} parameter sets")
        rids = [self.add_request(list(p), sp) for p, sp in zip(prompt_ids, params)]
        while self.has_unfinished():
            finished_before = len(self.scheduler.finished())
            if (self.step() is None and len(self.scheduler.finished()) == finished_before
                    and not self.scheduler.preempted()):
                raise RuntimeError("the scheduler can make no progress: no request fits the cache")
        return [self.collect(r) for r in rids]
