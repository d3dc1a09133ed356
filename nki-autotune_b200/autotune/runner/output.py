"""Result table, ``results.json`` and the on-disk cache layout.

Behaviour follows ``autotune/src/autotune/runner/output.py`` upstream: same file names
(``<cache>/<stem>/<stem>.py``, ``log-neuron-cc.txt``, ``profile_summary.json``, optional
``profile.json`` / ``file.neff`` / ``profile.ntff``, and ``<cache>/results.json``), same JSON
keys, same text table.  Two counters are added next to the Trainium ones: ``smem_oom`` and
``tmem_oom`` (shared-memory / tensor-memory over-subscription); ``sbuf_oom`` and ``psum_oom``
stay present so existing readers keep working.
"""

from __future__ import annotations

import base64
import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import NamedTuple

from autotune.runner.types import KernelJob, ProfileResult, profiler_percent

SUMMARY_FILE = "profile_summary.json"
DETAILED_FILE = "profile.json"
BINARY_FILE = "file.neff"
TRACE_FILE = "profile.ntff"
LOG_FILE = "log-neuron-cc.txt"

_MFU = "mfu_estimated_percent"
_MBU = "mbu_estimated_percent"
_CEILING = "mfu_max_achievable_estimated_percent"


class SuccessRow(NamedTuple):
    """A result that ran and was timed (reference: output.py:18-25)."""

    kernel_name: str
    total_time_s: float
    mfu: float
    mbu: float | None
    roofline_ceiling: float | None


def _ran(result: ProfileResult) -> bool:
    """Success sentinel: the output description starts with ``[`` (reference: output.py:32,76)."""
    return result.hardware_output.startswith("[")


def _total_time(result: ProfileResult) -> float | None:
    total = (result.profiler_summary or {}).get("total_time")
    return float(total) if isinstance(total, (int, float)) else None


def _collect_successes(results: list[ProfileResult]) -> list[SuccessRow]:
    """Results that ran, have a numeric ``total_time`` and a usable MFU (reference: output.py:28-49)."""
    rows = []
    for r in results:
        total = _total_time(r)
        mfu = profiler_percent(r.profiler_summary, _MFU)
        if not _ran(r) or total is None or mfu is None:
            continue
        rows.append(
            SuccessRow(
                r.kernel_name,
                total,
                mfu,
                profiler_percent(r.profiler_summary, _MBU),
                profiler_percent(r.profiler_summary, _CEILING),
            )
        )
    return rows


@dataclass
class ProfileOutput:
    """What :func:`autotune.runner.api.profile` returns (reference: output.py:52-85)."""

    results: list[ProfileResult]
    compiler_logs: dict[str, str]
    elapsed_s: float
    cache_dir: str = ""

    @property
    def successes(self) -> list[SuccessRow]:
        return _collect_successes(self.results)

    @property
    def failures(self) -> list[ProfileResult]:
        return [r for r in self.results if r.profiler_summary is None or not _ran(r)]

    def __str__(self) -> str:
        ok = self.successes
        parts = _table_lines(ok) + _failure_lines(self.failures) + _footer_lines(ok, self)
        return "\n".join(parts)


def _pct(value: float | None) -> str:
    return "-" if value is None else f"{value:.2f}%"


def _table_lines(rows: list[SuccessRow]) -> list[str]:
    """Fastest-first table; MFU and roofline columns appear only when some row has them."""
    if not rows:
        return []
    with_mfu = any(r.mfu > 0 for r in rows)
    with_roof = any(r.mbu is not None or r.roofline_ceiling is not None for r in rows)
    head = f"{'Kernel':<30} {'total_s':>10}"
    if with_mfu:
        head += f" {'mfu':>8}"
    if with_roof:
        head += f" {'mbu':>8} {'ceiling':>8}"
    out = [head, "-" * len(head)]
    for r in sorted(rows, key=lambda x: x.total_time_s):
        line = f"{r.kernel_name:<30} {r.total_time_s:>10.6f}"
        if with_mfu:
            line += f" {r.mfu:>7.2f}%"
        if with_roof:
            line += f" {_pct(r.mbu):>8} {_pct(r.roofline_ceiling):>8}"
        out.append(line)
    return out


def _failure_lines(failed: list[ProfileResult]) -> list[str]:
    if not failed:
        return []
    return [f"\n{len(failed)} failures:"] + [f"  {r.kernel_name}: {r.hardware_output}" for r in failed]


def _footer_lines(rows: list[SuccessRow], out: ProfileOutput) -> list[str]:
    lines = ["\nSummary:", f"  Succeeded:  {len(rows)}/{len(out.results)}", f"  Wallclock:  {out.elapsed_s:.1f}s"]
    if rows:
        times = [r.total_time_s for r in rows]
        # upstream prints the first row's name next to the minimum (output.py:136); the name
        # printed here is the one the minimum belongs to
        best = min(rows, key=lambda r: r.total_time_s)
        lines.append(f"  Best:       {best.total_time_s:.6f} s ({best.kernel_name})")
        lines.append(f"  Worst:      {max(times):.6f} s")
    if out.cache_dir:
        lines.append(f"  Cache:      {out.cache_dir}")
    return lines


def _variant_dir(cache_dir: str, kernel_name: str) -> tuple[str, str]:
    stem = Path(kernel_name).stem
    path = os.path.join(cache_dir, stem)
    os.makedirs(path, exist_ok=True)
    return stem, path


def write_kernel_sources(cache_dir: str, kernels: dict[str, KernelJob]) -> None:
    """``<cache>/<stem>/<stem>.py`` for every job (reference: output.py:143-150)."""
    for name, job in kernels.items():
        stem, path = _variant_dir(cache_dir, name)
        with open(os.path.join(path, f"{stem}.py"), "w") as fh:
            fh.write(job.source)


def write_compiler_logs(cache_dir: str, compiler_logs: dict[str, str]) -> None:
    """``<cache>/<stem>/log-neuron-cc.txt`` (reference: output.py:153-160)."""
    for name, text in compiler_logs.items():
        _, path = _variant_dir(cache_dir, name)
        with open(os.path.join(path, LOG_FILE), "w") as fh:
            fh.write(text)


def _kernel_sort_key(kernel_name: str) -> tuple[int, int, str]:
    """``<prefix>_<N>.py`` sorts by N; other names follow alphabetically (reference: output.py:163-173)."""
    stem = Path(kernel_name).stem
    suffix = stem.rsplit("_", 1)[-1]
    if suffix.isdigit():
        return (0, int(suffix), stem)
    return (1, 0, stem)


def _write_per_kernel_profiles(cache_dir: str, results: list[ProfileResult]) -> None:
    """Per-candidate JSON and binary artefacts (reference: output.py:176-199)."""
    for r in results:
        _, path = _variant_dir(cache_dir, r.kernel_name)
        if r.profiler_summary is not None:
            with open(os.path.join(path, SUMMARY_FILE), "w") as fh:
                json.dump(r.profiler_summary, fh, indent=2)
        if r.profile_detailed is not None:
            with open(os.path.join(path, DETAILED_FILE), "w") as fh:
                json.dump(r.profile_detailed, fh)
        for blob, fname in ((r.neff_b64, BINARY_FILE), (r.ntff_b64, TRACE_FILE)):
            if blob is not None:
                with open(os.path.join(path, fname), "wb") as fh:
                    fh.write(base64.b64decode(blob))


def write_results_json(cache_dir: str, num_kernels: int, results: list[ProfileResult], wallclock_s: float,
                       extra_metadata: dict | None = None) -> None:
    """Write ``results.json`` and the per-candidate files (reference: output.py:218-271).

    ``extra_metadata`` follows the two upstream metadata keys: what a reader needs to interpret the
    numbers (GPU name, GPUs used, the peaks behind the MFU / MBU percentages, seed, tolerance)."""
    _write_per_kernel_profiles(cache_dir, results)

    rows = []
    counters = {"success": 0, "sbuf_oom": 0, "psum_oom": 0, "smem_oom": 0, "tmem_oom": 0}
    needles = {
        "sbuf_oom": "Out of memory in sbuf",
        "psum_oom": "Out of memory in psum",
        "smem_oom": "Out of memory in smem",
        "tmem_oom": "Out of memory in tmem",
    }
    for r in results:
        total = _total_time(r)
        rows.append(
            {
                "result": r,
                "total": total,
                "mfu": profiler_percent(r.profiler_summary, _MFU),
                "mbu": profiler_percent(r.profiler_summary, _MBU),
                "ceiling": profiler_percent(r.profiler_summary, _CEILING),
            }
        )
        if total is not None:
            counters["success"] += 1
        else:
            for key, needle in needles.items():
                if needle in r.hardware_output:
                    counters[key] += 1

    timed = [row for row in rows if row["total"] is not None]
    times = [row["total"] for row in timed]
    mfus = [row["mfu"] for row in timed if row["mfu"] is not None]
    mbus = [row["mbu"] for row in timed if row["mbu"] is not None]

    def _name_at(pick):
        return pick(timed, key=lambda row: row["total"])["result"].kernel_name if timed else None

    index = []
    for row in sorted(rows, key=lambda row: _kernel_sort_key(row["result"].kernel_name)):
        r = row["result"]
        stem = Path(r.kernel_name).stem
        index.append(
            {
                "kernel_name": r.kernel_name,
                "kernel_path": f"{stem}/{stem}.py",
                "hardware_output": r.hardware_output,
                "total_time_s": row["total"],
                _MFU: row["mfu"],
                _MBU: row["mbu"],
                _CEILING: row["ceiling"],
            }
        )

    metrics = {
        "best_total_time_s": min(times) if times else None,
        "worst_total_time_s": max(times) if times else None,
        "best_kernel": _name_at(min),
        "worst_kernel": _name_at(max),
        "best_mfu": max(mfus) if mfus else None,
        "worst_mfu": min(mfus) if mfus else None,
        "best_mbu": max(mbus) if mbus else None,
        "worst_mbu": min(mbus) if mbus else None,
        "success": counters["success"],
        "sbuf_oom": counters["sbuf_oom"],
        "psum_oom": counters["psum_oom"],
        "smem_oom": counters["smem_oom"],
        "tmem_oom": counters["tmem_oom"],
    }
    doc = {
        "metadata": {"num_kernels": num_kernels, "wallclock_s": wallclock_s, **(extra_metadata or {})},
        "metrics": metrics,
        "kernels": index,
    }
    with open(os.path.join(cache_dir, "results.json"), "w") as fh:
        json.dump(doc, fh, indent=2)
