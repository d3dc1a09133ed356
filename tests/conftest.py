"""Shared pytest configuration: the ``gpu`` marker, import paths, and the native library."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
PKG = REPO / "nki-autotune_b200"
for p in (str(PKG), str(REPO)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def native_lib():
    """The shared library, brought up to date with the sources whenever nvcc is present (the build
    recompiles only what is stale, so this is a no-op for current objects); without nvcc the
    existing library is used, and a missing one fails the test."""
    import importlib.util
    import shutil

    from autotune import native

    have_nvcc = shutil.which("nvcc") is not None or Path("/usr/local/cuda/bin/nvcc").is_file()
    if have_nvcc:
        spec = importlib.util.spec_from_file_location("b200_build", PKG / "build.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return native.load()


@pytest.fixture(scope="session")
def checked_lib_path(native_lib):
    """Path of the checked variant of the library (``-DB200_CHECKED_BUILD``), built like the normal one."""
    import importlib.util
    import shutil

    have_nvcc = shutil.which("nvcc") is not None or Path("/usr/local/cuda/bin/nvcc").is_file()
    spec = importlib.util.spec_from_file_location("b200_build", PKG / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if have_nvcc:
        mod.build(checked=True)
    assert mod.CHECKED_LIB_PATH.exists(), "build it with: python nki-autotune_b200/build.py --checked"
    return mod.CHECKED_LIB_PATH


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(REPO / "tests" / "golden" / "reference_outputs.npz")
