"""Sweep ``rmsnorm_matmul`` (fused RMSNorm + matmul) candidates.

    python examples/tune_rmsnorm_matmul.py --cache DIR [--skinny] [--gpus N] [--detailed]

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
from autotune.runner.baseline import profile_numpy_baseline  # noqa: E402
from autotune.runner.candidate import Candidate, enumerate_grid, extended_grid, jobs_from_candidates  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cache", required=True)
    ap.add_argument("--skinny", action="store_true")
    ap.add_argument("--gpus", type=int, default=None)
    ap.add_argument("--detailed", action="store_true", help="keep launch plan, cycle counts and time series per candidate")
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
    output = profile(jobs, cache_dir=cache_dir, seed=seed, neuron_platform_target="b200",
                     collect_detailed_profile=args.detailed, n_gpus=args.gpus)
    print(output)

    # the row the reference prints next to its tuned kernel: the stock toolchain on the same maths,
    # here the unfused form through the vendor library (an rmsnorm pass, then a cuBLAS matmul)
    def unfused(x, gamma, weight):
        xf = x.float()
        xn = xf * (xf.pow(2).mean(dim=1, keepdim=True) + eps).rsqrt() * gamma.float()
        return xn.to(x.dtype) @ weight

    baseline, how = profile_numpy_baseline(unfused, specs, os.path.join(cache_dir, "compiler_baseline"),
                                           kernel_name="compiler_baseline", flops=2.0 * m * n * k)
    base_t = (baseline.profiler_summary or {}).get("total_time")
    print("\n[tune] reference comparison:")
    if output.successes:
        best = min(output.successes, key=lambda s: s.total_time_s)
        print(f"  tuned ({best.kernel_name}): {best.total_time_s:.6f} s")
    if isinstance(base_t, float):
        print(f"  unfused vendor baseline ({how}: rmsnorm pass + matmul): {base_t:.6f} s")
    else:
        print(f"  vendor baseline unavailable: {baseline.hardware_output.splitlines()[-1]}")


if __name__ == "__main__":
    main()
