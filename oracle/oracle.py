"""numpy restatement of the reference's CPU simulator for the hot path.  TEST INFRASTRUCTURE.

Parity status: PINNED.  ``tests/test_oracle.py`` checks every function here against
``tests/golden/reference_outputs.npz``, which ``tests/golden/make_golden.py`` produced by
running the reference's own code (its ``@nkigym_kernel`` op-level simulator and its
``simulate_fp32`` wrapper over the two ``kernel_library`` hand kernels).

Each function restates, op by op, what the reference's per-op ``_run`` methods compute:

* matmul      -- ``NKIMatmul._run``            nkigym/src/nkigym/ops/matmul.py:43-45
* square-sum  -- ``NKIActivationReduce._run``  nkigym/src/nkigym/ops/activation_reduce.py:96-100
* rsqrt       -- ``NKIActivation._run``        nkigym/src/nkigym/ops/activation.py:58-64
* row scale   -- ``NKITensorScalar._run``      nkigym/src/nkigym/ops/tensor_scalar.py:48-53
* transpose   -- ``NKIDMATranspose._run``      nkigym/src/nkigym/ops/dma_transpose.py:40-42
* inputs      -- ``generate_tensors``          autotune/src/autotune/runner/benchmark.py:156-169
"""

from __future__ import annotations

import numpy as np


def generate_inputs(seed: int, specs: list[tuple[str, tuple[int, ...], dict | None]], bf16: bool) -> dict[str, np.ndarray]:
    """One ``default_rng(seed)``; tensors drawn in list order; fp32 (optionally bf16-rounded).

    ``specs`` entries are ``(name, shape, dist)`` with ``dist`` ``None`` (standard normal),
    ``{"kind": "normal", "scale": s}`` or ``{"kind": "uniform", "low": a, "high": b}``.
    With ``bf16=True`` the values are rounded to bfloat16 and returned upcast to fp32, which
    is what ``simulate_fp32`` feeds the simulator when handed bf16 arrays
    (nkigym/src/nkigym/synthesis/simulate_nki.py:44-45).
    """
    rng = np.random.default_rng(seed)
    out: dict[str, np.ndarray] = {}
    for name, shape, dist in specs:
        dist = dist or {"kind": "normal", "scale": 1.0}
        if dist["kind"] == "normal":
            values = rng.standard_normal(shape)
            scale = float(dist.get("scale", 1.0))
            if scale != 1.0:
                values *= scale
        elif dist["kind"] == "uniform":
            values = rng.uniform(float(dist["low"]), float(dist["high"]), shape)
        else:
            raise ValueError(f"unknown distribution {dist!r}")
        values = values.astype(np.float32)
        if bf16:
            values = bf16_round(values)
        out[name] = values
    return out


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bfloat16, returned as fp32."""
    import ml_dtypes

    return np.asarray(a).astype(ml_dtypes.bfloat16).astype(np.float32)


def matmul_lhsT_rhs(lhs_T: np.ndarray, rhs: np.ndarray) -> np.ndarray:
    """``stationary.astype(f32).T @ moving.astype(f32)`` -- Load, Load, Matmul, TensorCopy, Store
    (examples/tune_matmul_lhsT_rhs.py:111-119)."""
    return lhs_T.astype(np.float32).T @ rhs.astype(np.float32)


def matmul_lhs_rhs(lhs: np.ndarray, rhs: np.ndarray) -> np.ndarray:
    """``lhs @ rhs`` as the reference computes it: DMATranspose of lhs, then the same Matmul
    (kernel_library/matmul/lhs_rhs/kernel_handtuned_89.26mfu.py:226-287; ops/dma_transpose.py:40-42)."""
    lhs_t = np.array(lhs).T
    return lhs_t.astype(np.float32).T @ rhs.astype(np.float32)


def rmsnorm_matmul(x: np.ndarray, gamma: np.ndarray | None, weight: np.ndarray, eps: float) -> np.ndarray:
    """``(x * rsqrt(mean_k x^2 + eps) * gamma) @ weight`` as the reference's op chain:

    ActivationReduce(square, add) -> Activation(rsqrt, scale=1/K, bias=eps) -> TensorScalar(multiply)
    -> DMATranspose -> TensorScalar(multiply by gamma, per partition = per k) -> Matmul.
    With ``gamma=None`` this is the maths of ``rmsnorm_matmul_online``
    (kernel_library/rmsnorm_matmul/kernel_hand_online.py:5-17; eps inside the sqrt, added to the mean).
    """
    xf = x.astype(np.float32)
    k = xf.shape[1]
    sumsq = np.sum(np.square(xf), axis=1).astype(np.float32)
    rinv = 1.0 / np.sqrt(sumsq.astype(np.float32) * (1.0 / k) + eps)
    xn = np.multiply(xf, rinv[..., np.newaxis])
    xt = np.array(xn).T
    if gamma is not None:
        xt = np.multiply(xt, gamma.astype(np.float32)[..., np.newaxis])
    return xt.astype(np.float32).T @ weight.astype(np.float32)


def max_abs_rel_err(actual: np.ndarray, expected: np.ndarray) -> float:
    """``max |a-e| / (|e| + rms(e))``: the reference's relative-error style
    (nkigym/src/nkigym/synthesis/numpy_to_nkigym.py:282-284) with rms(e) as the floor."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    floor = max(float(np.sqrt(np.mean(e * e))), 1e-30)
    return float(np.max(np.abs(a - e) / (np.abs(e) + floor)))


# The five benchmark configurations: seed, ordered tensor specs, scalars.
def config_specs(name: str) -> dict:
    n = lambda s: {"kind": "normal", "scale": s}  # noqa: E731
    u = {"kind": "uniform", "low": 0.5, "high": 1.5}
    table = {
        "cfg1_fp32_512": dict(family="matmul_lhsT_rhs", seed=0, bf16=False, eps=0.0,
                              specs=[("lhs_T", (512, 512), None), ("rhs", (512, 512), None)]),
        "cfg2_bf16_8192": dict(family="matmul_lhsT_rhs", seed=1, bf16=True, eps=0.0,
                               specs=[("lhs_T", (8192, 8192), n(8192 ** -0.5)), ("rhs", (8192, 8192), n(8192 ** -0.5))]),
        "cfg3_rmsnorm_4096": dict(family="rmsnorm_matmul", seed=2, bf16=True, eps=1e-6,
                                  specs=[("x", (4096, 4096), None), ("gamma", (4096,), u),
                                         ("weight", (4096, 11008), n(4096 ** -0.5))]),
        "cfg4_rmsnorm_skinny": dict(family="rmsnorm_matmul", seed=3, bf16=True, eps=1e-5,
                                    specs=[("x", (16, 8192), None), ("gamma", (8192,), u),
                                           ("weight", (8192, 28672), n(8192 ** -0.5))]),
        "cfg5_large_m": dict(family="matmul_lhsT_rhs", seed=4, bf16=True, eps=0.0,
                             specs=[("lhs_T", (4096, 131072), n(4096 ** -0.5)), ("rhs", (4096, 4096), n(4096 ** -0.5))]),
    }
    return table[name]
