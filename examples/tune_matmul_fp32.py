"""The fp32 configuration: ``matmul_lhsT_rhs`` at 512^3 in float32, four tile candidates.

    python examples/tune_matmul_fp32.py --cache DIR

Counterpart of the reference's CPU-simulator case (``examples/tune_matmul_lhsT_rhs.py:156-172``:
every rendered variant is simulated in fp32 and compared with ``lhs_T.T @ rhs`` before it is
profiled).  Here the four (tile_m, tile_n, tile_k) candidates from {128, 256} x {128, 512} x {128}
run on the fp32 CUDA-core kernel -- tensor-core tf32 cannot meet the 1e-5 tolerance -- so the tile
numbers only name the candidates; each is checked against the fp32 device reference at 1e-5 inside
``profile()``.  The vendor-library row follows, as upstream prints its compiler baseline.
"""

import argparse
import os
import shutil
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "nki-autotune_b200"))

from autotune.runner.api import profile  # noqa: E402
from autotune.runner.baseline import profile_numpy_baseline  # noqa: E402
from autotune.runner.candidate import Candidate, jobs_from_candidates  # noqa: E402

SEED = 0


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cache", required=True)
    ap.add_argument("--detailed", action="store_true")
    args = ap.parse_args()

    n = 512
    specs = {"lhs_T": ((n, n), "float32"), "rhs": ((n, n), "float32")}
    cands = [Candidate("matmul_lhsT_rhs", dict(tile_m=tm, tile_n=tn, tile_k=128, stages=2))
             for tm in (128, 256) for tn in (128, 512)]
    cache_dir = os.path.join(args.cache, "tune_matmul_fp32")
    shutil.rmtree(cache_dir, ignore_errors=True)
    print(f"[tune] profiling {len(cands)} fp32 candidates at {n}^3 (seed {SEED}, tolerance 1e-5) ...\n")
    output = profile(jobs_from_candidates(cands, (n, n), specs), cache_dir=cache_dir, seed=SEED,
                     neuron_platform_target="b200", collect_detailed_profile=args.detailed, n_gpus=1)
    print(output)
    baseline, how = profile_numpy_baseline(lambda lhs_T, rhs: lhs_T.T @ rhs, specs,
                                           os.path.join(cache_dir, "compiler_baseline"), kernel_name="compiler_baseline")
    t = (baseline.profiler_summary or {}).get("total_time")
    print(f"\n[tune] vendor baseline ({how}): " + (f"{t:.6f} s" if isinstance(t, float) else baseline.hardware_output.splitlines()[-1]))


if __name__ == "__main__":
    main()
