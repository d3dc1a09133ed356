"""Vendor-library baseline row.

Upstream ``profile_numpy_baseline`` (``autotune/src/autotune/runner/baseline.py:75-144``) compiles
a numpy function with the vendor compiler and profiles it the same way as the tuned kernels,
so every report carries a "what the stock toolchain gives" row.  The B200 analogue runs the
same function on device tensors through PyTorch (cuBLAS for ``@``), timed with CUDA events
and summarised with the same keys.  It is a yard-stick only: nothing in the product path
calls it.
"""

from __future__ import annotations

import os
import shutil
import statistics
from typing import Any, Callable

from autotune.peaks import load_peaks
from autotune.runner.benchmark import generate_tensors
from autotune.runner.types import ProfileResult, capture_error


def profile_numpy_baseline(
    func: Callable[..., Any],
    input_specs: dict[str, tuple],
    output_dir: str,
    kernel_name: str = "baseline",
    additional_compiler_args: str = "",
    collect_detailed_profile: bool = False,
    flops: float | None = None,
    warmup: int = 3,
    iters: int = 10,
) -> tuple[ProfileResult, str]:
    """Time ``func`` (array-API style, e.g. ``lambda a, b: a.T @ b``) on the GPU via PyTorch.

    ``input_specs`` order must match ``func``'s positional parameters; inputs come from
    ``generate_tensors(..., seed=42)`` as upstream.  ``flops`` (optional) fills the MFU field.
    Returns ``(ProfileResult, description)``; failures are captured into ``hardware_output``.
    """
    del additional_compiler_args
    shutil.rmtree(output_dir, ignore_errors=True)
    os.makedirs(output_dir, exist_ok=True)
    summary: dict[str, Any] | None = None
    detailed: dict[str, Any] | None = None
    hardware_output = "baseline"
    description = "torch eager on device tensors (cuBLAS for matmul)"
    try:
        import torch

        from autotune import kernels

        specs = {}
        for name, spec in input_specs.items():
            entry = {"shape": list(spec[0]), "dtype": spec[1]}
            if len(spec) > 2 and spec[2]:
                entry["dist"] = dict(spec[2])
            specs[name] = entry
        tensors = [kernels.to_device(v) for v in generate_tensors(specs, seed=42).values()]
        for _ in range(warmup):
            out = func(*tensors)
        ms = []
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = func(*tensors)
            e1.record()
            e1.synchronize()
            ms.append(e0.elapsed_time(e1))
        t = statistics.median(ms) * 1e-3
        peaks = load_peaks()
        nbytes = sum(x.numel() * x.element_size() for x in tensors) + out.numel() * out.element_size()
        summary = {
            "total_time": t,
            "mfu_estimated_percent": (flops / (t * peaks["bf16_tflops"] * 1e12)) if flops else 0.0,
            "mbu_estimated_percent": nbytes / (t * peaks["hbm_gbs"] * 1e9),
            "time_ms_each": [float(x) for x in ms],
            "peaks": peaks,
        }
        hardware_output = f"{list(out.shape)} {str(out.dtype).replace('torch.', '')}"
        if collect_detailed_profile:
            detailed = {"launches_ms": [float(x) for x in ms]}
    except Exception as exc:  # noqa: BLE001
        hardware_output = capture_error(exc)
    return ProfileResult(kernel_name, hardware_output, summary, detailed), description
