"""Typed reading of config.json keys.

Every size and constant of a model comes from its config.json through a typed
configuration class; nothing in the parts or kernels holds a model's numbers.
The reference's ``ModelConfig`` (crates/vllm-models/src/config.rs:11-58) is a
serde struct with required keys and defaults; this module gives the same
behaviour (required keys, defaults, unknown keys ignored) with explicit errors.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot be turned into a typed configuration."""


_MISSING = object()


class KeyReader:
    """Reads keys of one JSON object with a type check and a clear error."""

    def __init__(self, data: dict, where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected a JSON object, got {type(data).__name__}")
        self.data = data
        self.where = where

    def _get(self, key: str, default: Any):
        v = self.data.get(key, _MISSING)
        if v is _MISSING or v is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return _MISSING
        return v

    def integer(self, key: str, default: Any = _MISSING, minimum: int | None = None):
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default: Any = _MISSING, positive: bool = False):
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0.0:
            raise ConfigError(f"{self.where}: '{key}' must be > 0, got {v}")
        return v

    def boolean(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default: Any = _MISSING):
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: '{key}' must be a string, got {v!r}")
        return v

    def int_list(self, key: str, default: Any = _MISSING):
        """An integer or a list of integers, returned as a tuple."""
        v = self._get(key, default)
        if v is _MISSING:
            return default
        if isinstance(v, int) and not isinstance(v, bool):
            return (v,)
        if isinstance(v, list) and all(isinstance(t, int) and not isinstance(t, bool) for t in v):
            return tuple(v)
        raise ConfigError(f"{self.where}: '{key}' must be an integer or a list of integers, got {v!r}")

    def obj(self, key: str):
        """A nested object as a KeyReader, or None when absent or null."""
        v = self.data.get(key)
        if v is None:
            return None
        return KeyReader(v, f"{self.where}:{key}")


def read_json(path) -> dict:
    path = Path(path)
    try:
        text = path.read_text()
    except OSError as e:
        raise ConfigError(f"cannot read {path}: {e}") from e
    try:
        data = json.loads(text)
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: invalid JSON: {e}") from e
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected a JSON object")
    return data
