"""The checked build of the library (``-DB200_CHECKED_BUILD``): every kernel family runs a matrix of
shapes with device-side validation of its shared-memory, tensor-memory and barrier addresses, TMA
coordinates and global indices; no check may fire, the results must still match the oracle, and
the library's self-test (out-of-range arguments that the checks refuse and skip) must be recorded.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]


def test_checked_build_runs_every_family_without_a_failed_check(checked_lib_path):
    env = dict(os.environ, B200_AUTOTUNE_LIB=str(checked_lib_path))
    proc = subprocess.run([sys.executable, str(ROOT / "tests" / "checked_build_cases.py")], env=env, capture_output=True,
                          text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    assert res["cases"] == 14
    assert res["after_cases"] is not None, "the child loaded the normal library"
    assert res["after_cases"]["failures"] == 0, res["after_cases"]
    assert res["worst_err"] <= 1e-2
    # the self-test: 32 lanes x 3 refused accesses, first one recorded with its code and line
    st = res["after_selftest"]
    assert st["failures"] == 96 and st["code"] in (1, 4, 5) and st["line"] > 0, st
    assert res["after_clear"]["failures"] == 0


def test_normal_library_has_no_check_record(native_lib):
    from autotune import native

    assert native.checked_build_report() is None
