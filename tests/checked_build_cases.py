"""Runs a matrix of shapes and candidates through whichever library ``B200_AUTOTUNE_LIB`` names and
prints one JSON object: the worst error against the CPU oracle, the device-side check record after
the cases, the record after the library's self-test, and the record after clearing.

Started as a child process by ``test_gpu_checked_build.py`` with the checked library selected, so
the parent's own process keeps the normal one.
"""

import json
import sys
from pathlib import Path

import ml_dtypes
import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path[:0] = [str(ROOT), str(ROOT / "nki-autotune_b200")]

from autotune import kernels, native  # noqa: E402
from oracle import oracle as O  # noqa: E402

BF = ml_dtypes.bfloat16


def cfg(tm, tn, tk, st, cm=1, sw=0, nm=0, sk=0):
    return dict(tile_m=tm, tile_n=tn, tile_k=tk, stages=st, cluster_m=cm, swizzle=sw, norm_mode=nm, split_k=sk)


def n_(k):
    return {"kind": "normal", "scale": k ** -0.5}


MATMUL = [
    # k, m, n, candidate
    (256, 256, 256, cfg(128, 128, 64, 4)),
    (192, 200, 136, cfg(128, 64, 64, 3)),                  # ragged in every dimension
    (512, 1024, 768, cfg(256, 256, 64, 4, cm=2)),          # CTA pair
    (512, 1024, 1024, cfg(512, 256, 64, 4, cm=2)),         # two row blocks, accumulator handed over in halves
    (512, 1024, 1024, cfg(256, 512, 64, 4, cm=2, sw=2)),   # two column blocks
    (2048, 256, 256, cfg(128, 128, 64, 4, sk=4)),          # split-K and its second kernel
    (640, 392, 520, cfg(256, 128, 128, 3, cm=2)),          # ragged with a pair
]
FUSED = [
    # m, k, n, gamma, candidate
    (512, 512, 768, True, cfg(256, 256, 64, 4, cm=2, nm=2)),   # norm pass inside the launch
    (304, 256, 264, True, cfg(128, 128, 64, 4, nm=2)),         # ragged rows and columns
    (512, 512, 512, False, cfg(256, 256, 64, 4, cm=2, nm=2)),  # without gamma: the main loop reads x itself
    (256, 512, 512, True, cfg(128, 128, 64, 3, nm=1)),         # inline variant (x scaled on its way through tensor memory)
    (16, 1024, 4096, True, cfg(16, 256, 128, 3)),              # weight-streaming kernel, donors and owners
    (5, 512, 1288, True, cfg(16, 256, 64, 4)),                 # fewer rows than 16, last tile 8 columns wide
    (16, 8192, 256, False, cfg(16, 256, 128, 3)),              # one tile shared by every CTA
]


def main() -> None:
    try:
        run()
    except native.NativeError as exc:   # a refused access leaves its consumer to the bounded wait: say which check fired
        print(json.dumps({"error": str(exc), "record": native.checked_build_report(clear=True)}))
        raise SystemExit(1)


def run() -> None:
    worst = 0.0
    for seed, (k, m, n, c) in enumerate(MATMUL):
        t = O.generate_inputs(seed, [("lhs_T", (k, m), n_(k)), ("rhs", (k, n), n_(k))], bf16=True)
        got = kernels.matmul_lhsT_rhs_host(t["lhs_T"].astype(BF), t["rhs"].astype(BF), c).astype(np.float32)
        worst = max(worst, O.max_abs_rel_err(got, O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])))
    for seed, (m, k, n, with_gamma, c) in enumerate(FUSED):
        specs = [("x", (m, k), None)] + ([("gamma", (k,), {"kind": "uniform", "low": 0.5, "high": 1.5})] if with_gamma else [])
        specs.append(("w", (k, n), n_(k)))
        t = O.generate_inputs(100 + seed, specs, bf16=True)
        gamma = t["gamma"].astype(BF) if with_gamma else None
        got = kernels.rmsnorm_matmul_host(t["x"].astype(BF), gamma, t["w"].astype(BF), 1e-6, c).astype(np.float32)
        want = O.rmsnorm_matmul(t["x"], t["gamma"] if with_gamma else None, t["w"], 1e-6)
        worst = max(worst, O.max_abs_rel_err(got, want))
    after_cases = native.checked_build_report(clear=True)
    after_selftest = native.checked_build_report(clear=True, selftest=True)
    after_clear = native.checked_build_report(clear=False)
    print(json.dumps({"cases": len(MATMUL) + len(FUSED), "worst_err": worst, "after_cases": after_cases,
                      "after_selftest": after_selftest, "after_clear": after_clear}))


if __name__ == "__main__":
    main()
