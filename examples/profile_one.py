"""Profile ONE configuration of one kernel family, with the detailed artefacts.

    python examples/profile_one.py --cache DIR [--family matmul_lhsT_rhs] [--size 8192 | --m M --k K --n N]
                                   [--tile-m 512 --tile-n 256 --tile-k 64 --stages 4 --cluster-m 2]
                                   [--warmup 10 --iters 50]

Counterpart of ``examples/profile_hand_90mfu.py:35-45`` upstream (one hand-tuned kernel through
``profile(..., collect_detailed_profile=True)``).  The cache directory then holds, beside the
descriptor and the validation log, ``profile_summary.json`` (time, MFU, MBU, error against the
fp32 device reference), ``profile.json`` (launch plan: grid, cluster, shared / tensor memory,
waves, registers; the kernel's own longest CTA lifetime in SM cycles; the estimate of how busy
the tensor pipe was), ``file.neff`` (descriptor + raw ``b200_cfg``) and ``profile.ntff`` (the
per-launch time series).
"""

import argparse
import json
import os
import shutil
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "nki-autotune_b200"))

from autotune.runner.api import profile  # noqa: E402
from autotune.runner.candidate import Candidate, jobs_from_candidates  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--cache", required=True)
    ap.add_argument("--family", default="matmul_lhsT_rhs", choices=("matmul_lhsT_rhs", "matmul_lhs_rhs", "rmsnorm_matmul"))
    ap.add_argument("--size", type=int, default=8192, help="K = M = N (rmsnorm_matmul: x[size, size] . w[size, size])")
    ap.add_argument("--m", type=int, default=0, help="rows of the result (overrides --size)")
    ap.add_argument("--k", type=int, default=0, help="contraction length (overrides --size)")
    ap.add_argument("--n", type=int, default=0, help="columns of the result (overrides --size)")
    ap.add_argument("--eps", type=float, default=1e-6)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--tile-m", type=int, default=512)
    ap.add_argument("--tile-n", type=int, default=256)
    ap.add_argument("--tile-k", type=int, default=64)
    ap.add_argument("--stages", type=int, default=4)
    ap.add_argument("--cluster-m", type=int, default=2)
    ap.add_argument("--norm-mode", type=int, default=0)
    args = ap.parse_args()

    m, k, n = args.m or args.size, args.k or args.size, args.n or args.size
    d = {"kind": "normal", "scale": k ** -0.5}
    if args.family == "matmul_lhsT_rhs":
        specs, scalars = {"lhs_T": ((k, m), "bfloat16", d), "rhs": ((k, n), "bfloat16", d)}, {}
    elif args.family == "matmul_lhs_rhs":
        specs, scalars = {"lhs": ((m, k), "bfloat16", d), "rhs": ((k, n), "bfloat16", d)}, {}
    else:
        specs = {"x": ((m, k), "bfloat16"), "gamma": ((k,), "bfloat16", {"kind": "uniform", "low": 0.5, "high": 1.5}),
                 "weight": ((k, n), "bfloat16", d)}
        scalars = {"eps": args.eps}
    cfg = dict(tile_m=args.tile_m, tile_n=args.tile_n, tile_k=args.tile_k, stages=args.stages, cluster_m=args.cluster_m,
               norm_mode=args.norm_mode)
    cache_dir = os.path.join(args.cache, "profile_one")
    shutil.rmtree(cache_dir, ignore_errors=True)
    jobs = jobs_from_candidates([Candidate(args.family, cfg, scalars)], (m, n), specs)
    out = profile(jobs, cache_dir=cache_dir, seed=1, neuron_platform_target="b200", collect_detailed_profile=True, n_gpus=1,
                  warmup=args.warmup, iters=args.iters)
    print(out)
    stem = next(iter(jobs))[:-3]
    detail = Path(cache_dir) / stem / "profile.json"
    if detail.exists():
        doc = json.loads(detail.read_text())
        doc.pop("launches_ms", None)
        print("\n[profile] " + json.dumps(doc, indent=2))
    print("\n[profile] artefacts:", sorted(p.name for p in (Path(cache_dir) / stem).iterdir()))


if __name__ == "__main__":
    main()
