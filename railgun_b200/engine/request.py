"""Requests' parameters and outcomes.

SamplingParams has the reference's fields and defaults
(crates/vllm-scheduler/src/request.rs:37-76): max_new_tokens 128, temperature
0.0 (greedy), top_p 1.0, top_k 0 (off), stop_token_ids []; plus ``seed``, which
the reference lacks (it seeds from the wall clock,
crates/vllm-engine/src/sampling.rs:21-24).  Finish reasons are the reference's
(crates/vllm-scheduler/src/request.rs:80-89).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    max_new_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    stop_token_ids: list = field(default_factory=list)
    seed: int = 0

    def validate(self) -> None:
        if self.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        if self.temperature < 0.0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")


FINISH_REASONS = {0: None, 1: "max_tokens", 2: "stop_token", 3: "cancelled", 4: "error"}


@dataclass
class RequestOutput:
    request_id: int
    token_ids: list
    finish_reason: str | None
    error: str | None = None
    num_preemptions: int = 0


@dataclass
class StepResponse:
    """One generated token of one request, as the reference sends one
    EngineStepResponse per token to the request's receiver
    (crates/vllm-engine/src/engine.rs:27-33); ``token_id`` stands where the
    reference has the decoded text (tokenizers are outside this engine)."""
    request_id: int
    token_id: int | None
    is_finished: bool
    finish_reason: str | None = None
