"""Reading and writing safetensors files without a library.

Format: an unsigned 64-bit little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}}`` and the tensors'
bytes.  The reference memory-maps every ``*.safetensors`` file of the model
folder, sorted by name (crates/vllm-models/src/llama/model.rs:66-74,115-119);
so does ``open_model_files``.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple
    begin: int
    end: int
    file: "SafetensorsFile"

    def read(self) -> torch.Tensor:
        """A tensor over the mapped bytes (no copy; read-only memory)."""
        n = 1
        for s in self.shape:
            n *= s
        if n == 0:
            return torch.empty(self.shape, dtype=self.dtype)
        buf = memoryview(self.file.map)[self.file.data_start + self.begin:self.file.data_start + self.end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only on purpose
            return torch.frombuffer(buf, dtype=self.dtype, count=n).reshape(self.shape)


class SafetensorsFile:
    def __init__(self, path):
        self.path = Path(path)
        try:
            self._fh = open(self.path, "rb")
        except OSError as e:
            raise SafetensorsError(f"cannot open {self.path}: {e}") from e
        size = self.path.stat().st_size
        if size < 8:
            raise SafetensorsError(f"{self.path}: truncated (no header length)")
        self.map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        (hlen,) = struct.unpack("<Q", self.map[:8])
        if 8 + hlen > size:
            raise SafetensorsError(f"{self.path}: truncated header ({hlen} bytes announced, file has {size})")
        try:
            header = json.loads(bytes(self.map[8:8 + hlen]))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{self.path}: header is not JSON: {e}") from e
        self.data_start = 8 + hlen
        self.entries: dict[str, TensorEntry] = {}
        for name, meta in header.items():
            if name == "__metadata__":
                continue
            dt = _DTYPES.get(meta.get("dtype"))
            if dt is None:
                raise SafetensorsError(f"{self.path}: tensor {name} has unknown dtype {meta.get('dtype')!r}")
            begin, end = meta["data_offsets"]
            shape = tuple(int(s) for s in meta["shape"])
            n = 1
            for s in shape:
                n *= s
            if end - begin != n * torch.empty((), dtype=dt).element_size():
                raise SafetensorsError(f"{self.path}: tensor {name}: {end - begin} bytes do not match shape {shape}")
            if self.data_start + end > size:
                raise SafetensorsError(f"{self.path}: truncated: tensor {name} ends beyond the file")
            self.entries[name] = TensorEntry(name, dt, shape, begin, end, self)


def open_model_files(model_dir) -> dict[str, TensorEntry]:
    """All tensors of every ``*.safetensors`` file in the folder, by name."""
    model_dir = Path(model_dir)
    files = sorted(model_dir.glob("*.safetensors"))
    if not files:
        raise SafetensorsError(f"no .safetensors file in {model_dir}")
    merged: dict[str, TensorEntry] = {}
    for f in files:
        for name, e in SafetensorsFile(f).entries.items():
            if name in merged:
                raise SafetensorsError(f"tensor {name} appears in both {merged[name].file.path.name} and {f.name}")
            merged[name] = e
    return merged


def write_safetensors(path, tensors: dict[str, torch.Tensor]) -> None:
    """Write tensors (on the CPU) in name order; data begins 8-byte aligned."""
    header = {}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of {name}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((-len(blob)) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
