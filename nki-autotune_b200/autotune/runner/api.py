"""Public entry point of the profiling path.

``profile()`` keeps the signature, return type and cache layout of the reference
(``autotune/src/autotune/runner/api.py:24-75``): write the candidate sources, run the
validate-and-time pipeline, write logs and ``results.json``, return a ``ProfileOutput``.
"""

from __future__ import annotations

import logging
import os
import time

from autotune.runner.driver import run_pipeline
from autotune.runner.output import ProfileOutput, write_compiler_logs, write_kernel_sources, write_results_json
from autotune.runner.types import KernelJob

logger = logging.getLogger(__name__)

SUPPORTED_TARGETS = ("b200", "sm_100a", "sm100a", "blackwell")


def profile(
    kernels: dict[str, KernelJob],
    cache_dir: str,
    seed: int,
    neuron_platform_target: str,
    collect_detailed_profile: bool,
    n_gpus: int | None = None,
    warmup: int = 10,
    iters: int = 50,
    shard: tuple[int, int] | None = None,
    retime_top: int = 0,
    inputs: dict | None = None,
    keep_workers: bool = False,
) -> ProfileOutput:
    """Validate and time a set of candidates on the GPUs of this box.

    Args:
        kernels: Candidate file name -> ``KernelJob``.
        cache_dir: Directory for sources, logs, per-candidate JSON and ``results.json``; the
            empty string skips all disk output.
        seed: Seed of the input tensors (one ``numpy.random.default_rng(seed)`` per batch).
        neuron_platform_target: Kept from the reference signature.  ``"b200"`` / ``"sm_100a"``
            name this backend; the reference's ``"trn2"`` is accepted and ignored so existing
            drivers run unchanged.
        collect_detailed_profile: Attach the per-launch timing list as ``profile.json``.
        n_gpus: Optional cap on the number of GPUs the sweep is sharded over (extension).
        warmup, iters: Untimed and timed launches per candidate; the reported time is the median
            of the timed ones (extension).
        shard: ``(rank, world)`` when the caller already runs one process per GPU; this
            process then times only its share of the candidates (extension).
        retime_top: After a sweep sharded over several GPUs, time the fastest ``retime_top``
            candidates again on one GPU so that the leaders are ranked on one device (extension).
        inputs: Input arrays by tensor name, if the caller already holds what ``seed`` and the
            specs would generate; nothing is generated then (extension).
        keep_workers: The per-GPU worker processes of a multi-GPU sweep stay alive, pinned to their
            GPUs with their CUDA contexts, for the next ``profile()`` call of this process;
            ``autotune.runner.driver.shutdown_workers()`` (or the end of the process) ends them
            (extension).

    Returns:
        ``ProfileOutput`` with every candidate present, as a success or as a failure row.
    """
    os.environ["B200_AUTOTUNE_TARGET"] = neuron_platform_target
    if neuron_platform_target.lower() not in SUPPORTED_TARGETS:
        logger.info("platform target %r is not a B200 name; running on the local GPUs anyway", neuron_platform_target)
    keep_logs = bool(cache_dir)
    if cache_dir:
        os.makedirs(cache_dir, exist_ok=True)
        write_kernel_sources(cache_dir, kernels)

    start = time.monotonic()
    results, compiler_logs = run_pipeline(
        kernels,
        seed=seed,
        collect_compiler_logs=keep_logs,
        collect_detailed_profile=collect_detailed_profile,
        n_gpus=n_gpus,
        warmup=warmup,
        iters=iters,
        shard=shard,
        retime_top=retime_top,
        inputs=inputs,
        keep_workers=keep_workers,
    )
    elapsed_s = time.monotonic() - start
    logger.info("Profile complete: %d results in %.1fs", len(results), elapsed_s)

    if cache_dir:
        write_compiler_logs(cache_dir, compiler_logs)
        write_results_json(cache_dir, len(kernels), results, elapsed_s, _run_metadata(results, seed, warmup, iters, n_gpus, shard))
        logger.info("Cache saved to %s", cache_dir)

    return ProfileOutput(results=results, compiler_logs=compiler_logs, elapsed_s=elapsed_s, cache_dir=cache_dir)


def _run_metadata(results, seed: int, warmup: int, iters: int, n_gpus, shard) -> dict:
    """What ``results.json`` needs beyond the reference's two metadata keys to be read on its own."""
    from autotune.peaks import load_peaks
    from autotune.runner.benchmark import TOL_BF16, TOL_FP32

    devices = sorted({(r.profiler_summary or {}).get("device") for r in results} - {None})
    indices = sorted({(r.profiler_summary or {}).get("device_index") for r in results} - {None})
    return {
        "gpu_name": devices[0] if devices else None,
        "n_gpus": (shard[1] if shard else None) or n_gpus or max(1, len(indices)),
        "peaks": load_peaks(),
        "seed": seed,
        "tolerance": {"bf16_max_abs_rel_err": TOL_BF16, "fp32_max_abs_rel_err": TOL_FP32},
        "timing": {"warmup": warmup, "iters": iters, "statistic": "median"},
    }
