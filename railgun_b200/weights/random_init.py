"""Random-weights mode: a model folder from a configuration and a seed.

Every tensor is drawn from its own generator, seeded by the seed and a hash of
the tensor's name, so the values do not depend on the order tensors are made
in.  Matrices and embeddings ~ N(0, 0.02); norm weights 1 + U(-0.1, 0.1).
The reference has no such mode; its loader only reads files
(crates/vllm-models/src/llama/model.rs:92-137).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .loader import TensorSpec
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: TensorSpec, seed: int, dtype=torch.bfloat16, std: float = 0.02) -> torch.Tensor:
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, name))
    if spec.init == "normal":
        t = torch.empty(spec.shape, dtype=torch.float32).normal_(0.0, std, generator=g)
    elif spec.init == "norm":
        t = 1.0 + (torch.rand(spec.shape, dtype=torch.float32, generator=g) * 0.2 - 0.1)
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, dtype=torch.float32)
    else:
        raise ValueError(f"unknown init {spec.init!r} for {name}")
    return t.to(dtype)


def write_random_model(config, seed: int, out_dir, dtype=torch.bfloat16, std: float = 0.02) -> Path:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a typed
    configuration of a registered architecture) into ``out_dir``."""
    from ..config.registry import architecture_of
    arch = architecture_of(config.architecture)
    spec = arch.model_spec(config)
    from ..parts.model import expected_tensors
    expected = expected_tensors(spec)
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    tensors = {name: random_tensor(name, ts, seed, dtype, std)
               for name, ts in expected.items() if not ts.optional}
    (out_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    write_safetensors(out_dir / "model.safetensors", tensors)
    return out_dir
