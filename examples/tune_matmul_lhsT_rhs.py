"""Sweep the meta-parameter grid of ``matmul_lhsT_rhs`` on the GPUs of this box.

    python examples/tune_matmul_lhsT_rhs.py --cache DIR [--detailed] [--size 8192] [--gpus N] [--extended]

Counterpart of ``examples/tune_matmul_lhsT_rhs.py`` upstream: build the jobs, profile them
(every candidate is checked against the fp32 device kernel before it is accepted), print the
table, then print the vendor-library baseline next to the best candidate.
"""

import argparse
import os
import shutil
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "nki-autotune_b200"))

from autotune.runner.api import profile  # noqa: E402
from autotune.runner.baseline import profile_numpy_baseline  # noqa: E402
from autotune.runner.candidate import enumerate_grid, extended_grid, jobs_from_candidates  # noqa: E402
from autotune.runner.types import profiler_percent  # noqa: E402

SEED = 1


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cache", required=True)
    ap.add_argument("--detailed", action="store_true", help="keep the per-launch timings of every candidate")
    ap.add_argument("--size", type=int, default=8192, help="K = M = N")
    ap.add_argument("--gpus", type=int, default=None, help="shard the candidates over this many GPUs")
    ap.add_argument("--retime-top", type=int, default=5,
                    help="after a multi-GPU sweep, time the fastest N candidates again on one GPU")
    ap.add_argument("--split-k", default="0", help="comma-separated split-K factors to sweep as a further dimension, e.g. 0,2,4,8")
    ap.add_argument("--extended", action="store_true", help="add the 24 large-tile points (512-row / 512-column tiles)")
    args = ap.parse_args()

    n = args.size
    dist = {"kind": "normal", "scale": n ** -0.5}
    specs = {"lhs_T": ((n, n), "bfloat16", dist), "rhs": ((n, n), "bfloat16", dist)}
    cache_dir = os.path.join(args.cache, "tune_matmul_lhsT_rhs")
    shutil.rmtree(cache_dir, ignore_errors=True)

    splits = tuple(int(v) for v in args.split_k.split(","))
    grid = extended_grid("matmul_lhsT_rhs") if args.extended else enumerate_grid("matmul_lhsT_rhs", split_k=splits)
    jobs = jobs_from_candidates(grid, (n, n), specs)
    print(f"[tune] profiling {len(jobs)} candidates at {n}^3 ...\n")
    output = profile(jobs, cache_dir=cache_dir, seed=SEED, neuron_platform_target="b200",
                     collect_detailed_profile=args.detailed, n_gpus=args.gpus, retime_top=args.retime_top)
    print(output)

    baseline, how = profile_numpy_baseline(lambda lhs_T, rhs: lhs_T.T @ rhs, specs,
                                           os.path.join(cache_dir, "compiler_baseline"),
                                           kernel_name="compiler_baseline", flops=2.0 * n ** 3)
    base_t = (baseline.profiler_summary or {}).get("total_time")
    print("\n[tune] reference comparison:")
    if output.successes:
        best = min(output.successes, key=lambda s: s.total_time_s)
        print(f"  tuned ({best.kernel_name}): {best.total_time_s:.6f} s   {best.mfu:.2f}% of bf16 peak")
    if isinstance(base_t, float):
        print(f"  vendor baseline ({how}): {base_t:.6f} s   "
              f"{profiler_percent(baseline.profiler_summary, 'mfu_estimated_percent'):.2f}% of bf16 peak")
    else:
        print(f"  vendor baseline unavailable: {baseline.hardware_output.splitlines()[-1]}")


if __name__ == "__main__":
    main()
