"""Host-only stand-ins for the GPU worker body, used to exercise the process pool on CPU.
Failures are made on the host: an exception, a process that exits, one that never answers."""

import os
import time

from autotune.runner.types import ProfileResult


def _row(item):
    return ProfileResult(item["kernel_name"], "[8, 8] float32",
                         {"total_time": 0.001 * (1 + item.get("i", 0)), "mfu_estimated_percent": 0.5,
                          "device_env": os.environ.get("CUDA_VISIBLE_DEVICES"), "pid": os.getpid()})


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


def reads_shared_inputs(items, opts, emit):
    """Attaches to the input tensors the parent published and reports a checksum per item."""
    from autotune.runner.driver import SharedInputs

    for it in items:
        arrays, handles = SharedInputs.attach(opts["shared_inputs"][it["batch"]])
        sums = {name: float(a.astype("float64").sum()) for name, a in arrays.items()}
        shapes = {name: list(a.shape) for name, a in arrays.items()}
        del arrays
        for h in handles:
            h.close()
        emit(ProfileResult(it["kernel_name"], "[8, 8] float32",
                           {"total_time": 0.001, "mfu_estimated_percent": 0.5, "sums": sums, "shapes": shapes}))
