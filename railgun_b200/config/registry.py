"""The registry from architecture name to model.

``config.json``'s ``architectures[0]`` selects an entry; the entry parses the
typed configuration and turns it into a ``ModelSpec``.  The reference's
ModelRegistry maps the same string to a factory with metadata
(crates/vllm-models/src/registry.rs:13-182; Llama registers as
"LlamaForCausalLM", crates/vllm-models/src/llama/model.rs:256-267) but its
command line never fills it; here every entry point goes through it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

from .base import ConfigError, read_json


@dataclass
class Architecture:
    name: str
    config_from_dict: Callable            # dict -> typed config
    model_spec: Callable                  # typed config -> ModelSpec
    description: str = ""
    family: str = ""
    allow_unexpected: Callable = field(default=lambda cfg: ())   # tensor names that may be present unused


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(arch: Architecture, replace: bool = False) -> Architecture:
    if arch.name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture {arch.name!r} is already registered")
    _ARCHITECTURES[arch.name] = arch
    return arch


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def architecture_of(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture: {name}; known: {known_architectures()}") from None


def load_config(model_dir):
    """(Architecture, typed config) of a model folder, chosen by config.json."""
    path = Path(model_dir) / "config.json"
    data = read_json(path)
    archs = data.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError(f"{path}: 'architectures' must be a non-empty list of names; "
                          f"known: {known_architectures()}")
    arch = architecture_of(archs[0])
    return arch, arch.config_from_dict(data, str(path))


def _ensure_builtin():
    if "LlamaForCausalLM" not in _ARCHITECTURES:
        from ..models import llama  # noqa: F401  (registers itself)
