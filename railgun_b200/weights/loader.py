"""Loading weights by tensor name.

A model lists the tensors it expects (name -> shape); the loader opens the
folder's safetensors files, checks every name and shape, and raises ONE
``WeightError`` that lists what is missing, what is unexpected and what has the
wrong shape.  Stored precision is kept: 16-bit floats become bfloat16, a tensor
stored in 32-bit stays 32-bit, integer tables become int32.  Each part then
casts what it computes with (crates/vllm-models/src/llama/model.rs:115-119
casts everything to the model dtype at load).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .safetensors_io import open_model_files, SafetensorsError


class WeightError(ValueError):
    """The model folder's tensors do not match what the model expects."""

    def __init__(self, message, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple
    init: str = "normal"        # how random-weights mode fills it: "normal" | "norm" | "zeros"
    optional: bool = False


def stored_precision(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.to(torch.bfloat16)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8):
        return t.to(torch.int32)
    return t


def load_weights(model_dir, expected: dict[str, TensorSpec], device="cpu",
                 allow_unexpected=()) -> dict[str, torch.Tensor]:
    """name -> tensor on ``device`` for every expected tensor present.

    ``allow_unexpected``: names that may be in the files without being used
    (for instance ``lm_head.weight`` beside tied embeddings)."""
    try:
        entries = open_model_files(model_dir)
    except SafetensorsError as e:
        raise WeightError(str(e)) from e
    missing = [n for n, s in expected.items() if n not in entries and not s.optional]
    unexpected = [n for n in entries if n not in expected and n not in allow_unexpected]
    wrong = [(n, tuple(expected[n].shape), entries[n].shape)
             for n in expected if n in entries and tuple(expected[n].shape) != entries[n].shape]
    if missing or unexpected or wrong:
        lines = [f"weights in {model_dir} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(g)}" for n, e, g in sorted(wrong)))
        raise WeightError("\n".join(lines), missing, unexpected, wrong)
    out = {}
    for name in expected:
        if name in entries:
            out[name] = stored_precision(entries[name].read()).to(device)
    return out
