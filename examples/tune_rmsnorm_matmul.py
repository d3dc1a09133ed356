"""Sweep ``rmsnorm_matmul`` (fused RMSNorm + matmul) candidates.

    python examples/tune_rmsnorm_matmul.py --cache DIR [--skinny] [--gpus N]

Default shape is x[4096,4096] . w[4096,11008] (eps 1e-6); ``--skinny`` is the decode shape
x[16,8192] . w[8192,28672] (eps 1e-5), which runs the weight-streaming kernel.
"""

import argparse
import os
import shutil
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "nki-autotune_b200"))

from autotune.runner.api import profile  # noqa: E402
from autotune.runner.candidate import Candidate, enumerate_grid, extended_grid, jobs_from_candidates  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cache", required=True)
    ap.add_argument("--skinny", action="store_true")
    ap.add_argument("--gpus", type=int, default=None)
    args = ap.parse_args()

    if args.skinny:
        m, k, n, eps, seed = 16, 8192, 28672, 1e-5, 3
        cands = [Candidate("rmsnorm_matmul", dict(tile_m=16, tile_n=256, tile_k=tk, stages=st), {"eps": eps})
                 for tk in (64, 128) for st in (2, 3, 4, 5, 6)]
    else:
        m, k, n, eps, seed = 4096, 4096, 11008, 1e-6, 2
        cands = []
        for mode in (2, 1):  # prologue variant, inline variant
            for c in enumerate_grid("rmsnorm_matmul", stages=(2, 3, 4, 6), scalars={"eps": eps}):
                cfg = dict(c.config, norm_mode=mode)
                cands.append(Candidate("rmsnorm_matmul", cfg, dict(c.scalars)))
        # the prologue variant runs the plain GEMM main loop, so the large pair tiles apply to it too
        for c in extended_grid("rmsnorm_matmul", scalars={"eps": eps})[64:]:
            if c.config["tile_m"] == 512:
                cands.append(Candidate("rmsnorm_matmul", dict(c.config, norm_mode=2), dict(c.scalars)))
    specs = {"x": ((m, k), "bfloat16"), "gamma": ((k,), "bfloat16", {"kind": "uniform", "low": 0.5, "high": 1.5}),
             "weight": ((k, n), "bfloat16", {"kind": "normal", "scale": k ** -0.5})}
    cache_dir = os.path.join(args.cache, "tune_rmsnorm_matmul" + ("_skinny" if args.skinny else ""))
    shutil.rmtree(cache_dir, ignore_errors=True)
    jobs = jobs_from_candidates(cands, (m, n), specs)
    print(f"[tune] profiling {len(jobs)} candidates for x[{m},{k}] . w[{k},{n}] ...\n")
    print(profile(jobs, cache_dir=cache_dir, seed=seed, neuron_platform_target="b200",
                  collect_detailed_profile=False, n_gpus=args.gpus))


if __name__ == "__main__":
    main()
