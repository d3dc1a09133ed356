"""Builds libb200_autotune.so in-tree with nvcc for sm_100a.

Usage: ``python build.py [--force] [--verbose] [--checked]``.  The library lands in ``lib/`` next
to this file; objects go to ``build/``.  Sources are recompiled only when they (or a header) are
newer than their object.  ``--checked`` builds ``lib/libb200_autotune_checked.so`` instead: the same
sources with ``-DB200_CHECKED_BUILD`` (device-side validation of every address and index, for
debugging; objects in ``build/checked/``).
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "build"
LIB_DIR = HERE / "lib"
LIB_PATH = LIB_DIR / "libb200_autotune.so"
CHECKED_LIB_PATH = LIB_DIR / "libb200_autotune_checked.so"
INCLUDE = HERE.parent / "include"

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    """Locate nvcc: $CUDA_HOME, PATH, then /usr/local/cuda."""
    candidates = []
    if os.environ.get("CUDA_HOME"):
        candidates.append(os.path.join(os.environ["CUDA_HOME"], "bin", "nvcc"))
    which = shutil.which("nvcc")
    if which:
        candidates.append(which)
    candidates.append("/usr/local/cuda/bin/nvcc")
    for c in candidates:
        if os.path.isfile(c):
            return c
    raise RuntimeError("nvcc not found (set CUDA_HOME)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hdrs)


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool, defines: tuple[str, ...] = ()) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> Path:
    """Compile every csrc/*.cu and link the shared library (or its checked variant); returns its path."""
    nvcc = find_nvcc()
    obj_dir = BUILD / "checked" if checked else BUILD
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    defines = ("-DB200_CHECKED_BUILD",) if checked else ()
    obj_dir.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    hdr_time = _headers_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_time)
        if stale:
            jobs.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        logs = list(pool.map(lambda so: _compile(nvcc, so[0], so[1], verbose, defines), jobs))
    if verbose:
        for (src, _), log in zip(jobs, logs):
            print(f"== {src.name}\n{log}")
    if jobs or not lib_path.exists():
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
               "-o", str(lib_path), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    return lib_path


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--checked", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, checked=a.checked))
    sys.exit(0)
