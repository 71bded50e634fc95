"""Building and loading the native libraries.

Each ``.cu`` file under ``csrc/kernels`` becomes one shared library of
``extern "C"`` launchers, compiled for sm_100a only, and each ``.cpp`` under
``csrc/host`` one host library.  A library is compiled the first time something
asks for it, so a model compiles what it uses.  Nothing here falls back to
another implementation: if a library cannot be built or loaded, the call
raises ``NativeBuildError``.

The reference builds its kernels to PTX at cargo build time and loads them at
start (crates/vllm-cuda/build.rs:11-30, crates/vllm-cuda/src/kernels/mod.rs:89-123);
here nvcc produces sm_100a machine code directly and ctypes loads it.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
KERNEL_DIR = CSRC / "kernels"
HOST_DIR = CSRC / "host"

# No fast-math: softmax, norms and rotation must be IEEE 32-bit.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC",
]
GXX_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-Wall"]


class NativeBuildError(RuntimeError):
    """A native library could not be compiled or loaded."""


_lock = threading.Lock()
_loaded: dict[str, ctypes.CDLL] = {}


def _say(msg: str) -> None:
    from . import log
    log.info(msg)
    for h in log.handlers:
        h.flush()


def _find(tool: str, extra: list[str]) -> str:
    path = shutil.which(tool)
    if path:
        return path
    for p in extra:
        if os.path.exists(p):
            return p
    raise NativeBuildError(f"{tool} not found; it is needed to build the native libraries")


_build_dir_cache: list = []


def _build_dir() -> Path:
    """In-tree ``_native/`` when writable, else a per-user folder under the
    system's temporary directory."""
    if _build_dir_cache:
        return _build_dir_cache[0]
    env = os.environ.get("RAILGUN_B200_BUILD_DIR")
    candidates = [Path(env)] if env else []
    candidates.append(Path(__file__).resolve().parent / "_native")
    candidates.append(Path(tempfile.gettempdir()) / f"railgun_b200_native_{os.getuid()}")
    for c in candidates:
        try:
            c.mkdir(parents=True, exist_ok=True)
            probe = c / f".w{os.getpid()}_{threading.get_ident()}"
            probe.write_text("")
            probe.unlink()
            _build_dir_cache.append(c)
            return c
        except OSError:
            continue
    raise NativeBuildError("no writable folder for the native libraries: tried " + ", ".join(map(str, candidates)))


def _source_digest(src: Path, flags: list[str]) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(src.parent.glob("*.cuh")) + sorted(src.parent.glob("*.h")) + sorted(src.parent.glob("*.hpp")):
        h.update(hdr.name.encode())
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _run_with_progress(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    _say(f"compiling {what} ...")
    while True:
        try:
            out, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {what} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        raise NativeBuildError(f"building {what} failed (exit {proc.returncode}):\n{' '.join(cmd)}\n{out}")
    _say(f"compiled {what} in {time.time() - t0:.1f} s")


def library_path(name: str, kind: str) -> tuple[Path, Path, list[str], str]:
    if kind == "kernel":
        src = KERNEL_DIR / f"{name}.cu"
        flags = list(NVCC_FLAGS)
        compiler = "nvcc"
    else:
        src = HOST_DIR / f"{name}.cpp"
        flags = list(GXX_FLAGS)
        compiler = "g++"
    if not src.exists():
        raise NativeBuildError(f"no source file {src}")
    digest = _source_digest(src, flags)
    out = _build_dir() / f"librailgun_{name}.{digest}.so"
    return src, out, flags, compiler


def build(name: str, kind: str = "kernel") -> Path:
    """Compile one library if its built file is missing or stale; return its path."""
    src, out, flags, compiler = library_path(name, kind)
    if out.exists():
        return out
    if compiler == "nvcc":
        exe = _find("nvcc", ["/usr/local/cuda/bin/nvcc"])
    else:
        exe = _find("g++", ["/usr/bin/g++"])
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [exe, *flags, "-o", str(tmp), str(src)]
    _run_with_progress(cmd, f"{src.name} ({'sm_100a' if compiler == 'nvcc' else 'host'})")
    os.replace(tmp, out)
    for old in out.parent.glob(f"librailgun_{name}.*.so"):
        if old != out and ".tmp" not in old.name:
            try:
                old.unlink()
            except OSError:
                pass
    return out


def load(name: str, kind: str = "kernel") -> ctypes.CDLL:
    """The loaded library, built first if need be.  Raises, never falls back."""
    key = f"{kind}:{name}"
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = build(name, kind)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise NativeBuildError(f"cannot load {path}: {e}") from e
            _loaded[key] = lib
        return lib


def kernel_sources() -> list[str]:
    return sorted(p.stem for p in KERNEL_DIR.glob("*.cu"))


def host_sources() -> list[str]:
    return sorted(p.stem for p in HOST_DIR.glob("*.cpp"))


def build_all() -> list[Path]:
    """Compile every library (the check that everything builds for sm_100a)."""
    from concurrent.futures import ThreadPoolExecutor
    jobs = [(n, "kernel") for n in kernel_sources()] + [(n, "host") for n in host_sources()]
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        return list(ex.map(lambda j: build(*j), jobs))
