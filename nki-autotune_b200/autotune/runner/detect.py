"""Hardware detection (reference: ``autotune/src/autotune/runner/detect.py:7-20``)."""

from __future__ import annotations

from autotune import native


def detect_gpus() -> int:
    """Number of CUDA devices visible to this process.

    Raises:
        RuntimeError: if the native library cannot be loaded or no device is visible
            (the reference raises when ``neuron-ls`` reports 0 cores).
    """
    count = native.device_count()
    if count == 0:
        raise RuntimeError("no CUDA device is visible (0 GPUs)")
    return count


# the reference's name for the same question
detect_neuron_cores = detect_gpus
