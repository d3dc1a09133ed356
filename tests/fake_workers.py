"""Host-only stand-ins for the GPU worker body, used to exercise the process pool on CPU.
Failures are made on the host: an exception, a process that exits, one that never answers."""

import os
import time

from autotune.runner.types import ProfileResult


def _row(item):
    return ProfileResult(item["kernel_name"], "[8, 8] float32",
                         {"total_time": 0.001 * (1 + item.get("i", 0)), "mfu_estimated_percent": 0.5,
                          "device_env": os.environ.get("CUDA_VISIBLE_DEVICES")})


def well_behaved(items, opts, emit):
    for it in items:
        emit(_row(it))


def faulty(items, opts, emit):
    """Per-item behaviour chosen by the item's "inject" field."""
    for it in items:
        kind = it.get("inject")
        if kind == "raise":
            raise RuntimeError("injected failure in " + it["kernel_name"])
        if kind == "exit":
            os._exit(3)
        if kind == "hang":
            time.sleep(3600)
        emit(_row(it))
