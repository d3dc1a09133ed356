"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own code.

Run from a checkout that has the reference tree available:

    python tests/golden/make_golden.py --reference /path/to/nki-autotune

What runs (all reference-owned code, imported read-only; ``nki`` itself comes from nki_shim):
  * the ``@nkigym_kernel`` op-level numpy simulator (``nkigym/src/nkigym/ops``): the SSA matmul
    of ``test/ops/test_direct_numpy_call.py`` / ``examples/tune_matmul_lhsT_rhs.py:111-119`` and a
    gamma-extended RMSNorm+matmul DAG built from the reference's ops;
  * ``simulate_fp32`` (``nkigym/src/nkigym/synthesis/simulate_nki.py``) on the two hand kernels of
    ``kernel_library`` at their only legal shape, 2048^3.
Outputs are stored whole for the small cases and as a strided sample (plus checksums) for the
2048^3 cases.  Inputs are not stored: the tests regenerate them from the recorded seeds with the
reference's recipe (one ``default_rng(seed)``, tensors drawn in order).
"""

from __future__ import annotations

import argparse
import os
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def _load_file(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def draw(seed: int, specs: list[tuple[str, tuple[int, ...], dict]]) -> dict[str, np.ndarray]:
    """Reference input recipe (autotune/src/autotune/runner/benchmark.py:163-168) + distributions."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape, dist in specs:
        if dist["kind"] == "normal":
            v = rng.standard_normal(shape) * dist.get("scale", 1.0)
        else:
            v = rng.uniform(dist["low"], dist["high"], shape)
        out[name] = v.astype(np.float32)
    return out


def bf16_round(a: np.ndarray) -> np.ndarray:
    import ml_dtypes

    return a.astype(ml_dtypes.bfloat16).astype(np.float32)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("NKI_AUTOTUNE_REFERENCE"), required="NKI_AUTOTUNE_REFERENCE" not in os.environ,
                    help="checkout of awslabs/nki-autotune (or set NKI_AUTOTUNE_REFERENCE)")
    args = ap.parse_args()
    ref = Path(args.reference)
    sys.path.insert(0, str(HERE))
    import nki_shim

    nki_shim.install()
    sys.path.insert(0, str(ref / "nkigym" / "src"))

    from nkigym.ops import nkigym_kernel
    from nkigym.ops.activation import NKIActivation
    from nkigym.ops.activation_reduce import NKIActivationReduce
    from nkigym.ops.dma_transpose import NKIDMATranspose
    from nkigym.ops.load import NKILoad
    from nkigym.ops.matmul import NKIMatmul
    from nkigym.ops.store import NKIStore
    from nkigym.ops.tensor_copy import NKITensorCopy
    from nkigym.ops.tensor_scalar import NKITensorScalar
    from nkigym.synthesis.simulate_nki import simulate_fp32

    @nkigym_kernel
    def f_matmul(lhs_T, rhs):
        a = NKILoad()(src=lhs_T)
        b = NKILoad()(src=rhs)
        acc = NKIMatmul()(stationary=a, moving=b)
        return NKIStore()(src=NKITensorCopy()(src=acc))

    def make_rmsnorm(eps: float, K: int, with_gamma: bool):
        @nkigym_kernel
        def f_rms(x, gamma, weight):
            xs = NKILoad()(src=x)
            ws = NKILoad()(src=weight)
            sumsq = NKIActivationReduce()(data=xs, op="square", reduce_op="add")
            rinv = NKIActivation()(data=sumsq, op="rsqrt", scale=1.0 / K, bias=eps)
            xn = NKITensorScalar()(data=xs, op="multiply", operand0=rinv)
            xt = NKIDMATranspose()(src=xn)
            if with_gamma:
                gs = NKILoad()(src=gamma)
                xt = NKITensorScalar()(data=xt, op="multiply", operand0=gs)
            acc = NKIMatmul()(stationary=xt, moving=ws)
            return NKIStore()(src=NKITensorCopy()(src=acc))

        return f_rms

    out: dict[str, np.ndarray] = {}

    # 1. the reference's own op test case: 128^3, seed 0, standard normal, fp32
    t = draw(0, [("lhs_T", (128, 128), {"kind": "normal"}), ("rhs", (128, 128), {"kind": "normal"})])
    out["matmul_128_seed0"] = np.asarray(f_matmul(**t), dtype=np.float32)

    # 2. fp32 configuration: 512^3, seed 0
    t = draw(0, [("lhs_T", (512, 512), {"kind": "normal"}), ("rhs", (512, 512), {"kind": "normal"})])
    out["matmul_512_seed0"] = np.asarray(f_matmul(**t), dtype=np.float32)

    # 3. bf16-rounded inputs, ragged-ish small shape (K=384, M=256, N=320), seed 1
    t = draw(1, [("lhs_T", (384, 256), {"kind": "normal", "scale": 384 ** -0.5}),
                 ("rhs", (384, 320), {"kind": "normal", "scale": 384 ** -0.5})])
    t = {k: bf16_round(v) for k, v in t.items()}
    out["matmul_bf16in_384x256x320_seed1"] = np.asarray(f_matmul(**t), dtype=np.float32)

    # 4. RMSNorm+matmul with gamma: M=256, K=512, N=384, eps 1e-6, seed 2, bf16-rounded inputs
    t = draw(2, [("x", (256, 512), {"kind": "normal"}), ("gamma", (512,), {"kind": "uniform", "low": 0.5, "high": 1.5}),
                 ("weight", (512, 384), {"kind": "normal", "scale": 512 ** -0.5})])
    t = {k: bf16_round(v) for k, v in t.items()}
    out["rmsnorm_gamma_256x512x384_seed2"] = np.asarray(make_rmsnorm(1e-6, 512, True)(**t), dtype=np.float32)

    # 5. skinny RMSNorm+matmul: M=16, K=1024, N=512, eps 1e-5, seed 3
    t = draw(3, [("x", (16, 1024), {"kind": "normal"}), ("gamma", (1024,), {"kind": "uniform", "low": 0.5, "high": 1.5}),
                 ("weight", (1024, 512), {"kind": "normal", "scale": 1024 ** -0.5})])
    t = {k: bf16_round(v) for k, v in t.items()}
    out["rmsnorm_gamma_16x1024x512_seed3"] = np.asarray(make_rmsnorm(1e-5, 1024, True)(**t), dtype=np.float32)

    # 6. the hand kernels through the reference's simulate_fp32 at 2048^3, seed 0 (strided samples)
    t = draw(0, [("lhs_T", (2048, 2048), {"kind": "normal"}), ("rhs", (2048, 2048), {"kind": "normal"})])
    mm = _load_file(ref / "kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py", "ref_matmul_lhsT_rhs")
    full = np.asarray(simulate_fp32(mm.matmul_lhsT_rhs_nkigym)(t["lhs_T"], t["rhs"]), dtype=np.float32)
    out["hand_matmul_2048_seed0_sample"] = full[::127, ::131].copy()
    out["hand_matmul_2048_seed0_rowsum"] = full.sum(axis=1, dtype=np.float64)[::64].astype(np.float64)
    ssa = np.asarray(f_matmul(**t), dtype=np.float32)
    print("hand matmul kernel vs SSA op simulator, max abs diff:", float(np.abs(full - ssa).max()))

    t = draw(0, [("lhs", (2048, 2048), {"kind": "normal"}), ("rhs", (2048, 2048), {"kind": "normal"})])
    rm = _load_file(ref / "kernel_library/rmsnorm_matmul/kernel_hand_online.py", "ref_rmsnorm_matmul")
    full = np.asarray(simulate_fp32(rm.rmsnorm_matmul_online)(t["lhs"], t["rhs"]), dtype=np.float32)
    out["hand_rmsnorm_2048_seed0_sample"] = full[::127, ::131].copy()
    out["hand_rmsnorm_2048_seed0_rowsum"] = full.sum(axis=1, dtype=np.float64)[::64].astype(np.float64)
    ssa = np.asarray(make_rmsnorm(1e-6, 2048, False)(x=t["lhs"], gamma=None, weight=t["rhs"]), dtype=np.float32)
    print("hand rmsnorm kernel vs SSA op simulator (gamma absent), max abs diff:", float(np.abs(full - ssa).max()))
    out["ssa_rmsnorm_2048_seed0_sample"] = ssa[::127, ::131].copy()

    # 7. the lhs . rhs hand kernel (K-major lhs, DMA-transposed upstream) at 2048^3, seed 0
    t = draw(0, [("lhs", (2048, 2048), {"kind": "normal"}), ("rhs", (2048, 2048), {"kind": "normal"})])
    lr = _load_file(ref / "kernel_library/matmul/lhs_rhs/kernel_handtuned_89.26mfu.py", "ref_matmul_lhs_rhs")
    full = np.asarray(simulate_fp32(lr.matmul_lhs_rhs_nkigym)(t["lhs"], t["rhs"]), dtype=np.float32)
    out["hand_matmul_lhs_rhs_2048_seed0_sample"] = full[::127, ::131].copy()
    print("hand lhs.rhs kernel vs numpy, max abs diff:", float(np.abs(full - t["lhs"] @ t["rhs"]).max()))

    np.savez_compressed(HERE / "reference_outputs.npz", **out)
    for k, v in out.items():
        print(f"{k:45s} {v.shape} {v.dtype}")
    print("wrote", HERE / "reference_outputs.npz", (HERE / "reference_outputs.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
