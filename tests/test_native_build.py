"""The builder of the native libraries (railgun_b200/native.py), on the CPU with
the host library: names carry a digest of the source and its headers, a missing
source or a failing compiler is one clear error, the build folder can be moved."""
import ctypes

import pytest

from railgun_b200 import native


def test_library_names_carry_the_digest_of_source_and_flags():
    src, out, flags, compiler = native.library_path("runtime", "host")
    assert src.name == "runtime.cpp" and compiler == "g++"
    digest = native._source_digest(src, flags)
    assert out.name == f"librailgun_runtime.{digest}.so" and len(digest) == 16
    assert native._source_digest(src, flags + ["-DX"]) != digest          # other flags, another library
    ksrc, kout, kflags, kcompiler = native.library_path("norm", "kernel")
    assert kcompiler == "nvcc" and "arch=compute_100a,code=sm_100a" in kflags
    assert "norm" in native.kernel_sources() and "runtime" in native.host_sources()


def test_a_missing_source_is_a_clear_error():
    with pytest.raises(native.NativeBuildError, match="no source file .*no_such_kernel.cu"):
        native.load("no_such_kernel")


def test_the_build_folder_can_be_moved(tmp_path, monkeypatch):
    monkeypatch.setenv("RAILGUN_B200_BUILD_DIR", str(tmp_path / "built"))
    monkeypatch.setattr(native, "_build_dir_cache", [])
    path = native.build("runtime", "host")
    assert path.parent == tmp_path / "built" and path.is_file()
    lib = ctypes.CDLL(str(path))
    assert hasattr(lib, "rg_cache_create") and hasattr(lib, "rg_sched_schedule")
    assert native.build("runtime", "host") == path                       # built once
