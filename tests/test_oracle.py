"""The CPU oracle against golden vectors produced by the reference's own code (CPU only)."""

import numpy as np
import pytest

from oracle import oracle as O

U = {"kind": "uniform", "low": 0.5, "high": 1.5}


def test_matmul_128_matches_reference_op_simulator(golden):
    # the case of test/ops/test_direct_numpy_call.py:32-38 upstream (128^3, seed 0)
    t = O.generate_inputs(0, [("lhs_T", (128, 128), None), ("rhs", (128, 128), None)], bf16=False)
    got = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
    assert np.array_equal(got, golden["matmul_128_seed0"])
    assert np.allclose(got, t["lhs_T"].T @ t["rhs"], atol=1e-4, rtol=1e-4)


def test_matmul_512_fp32_config(golden):
    cfg = O.config_specs("cfg1_fp32_512")
    t = O.generate_inputs(cfg["seed"], cfg["specs"], cfg["bf16"])
    got = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
    assert O.max_abs_rel_err(got, golden["matmul_512_seed0"]) <= 1e-6
    f64 = t["lhs_T"].astype(np.float64).T @ t["rhs"].astype(np.float64)
    assert O.max_abs_rel_err(got, f64) <= 1e-5


def test_matmul_bf16_rounded_inputs(golden):
    s = 384 ** -0.5
    t = O.generate_inputs(1, [("lhs_T", (384, 256), {"kind": "normal", "scale": s}),
                              ("rhs", (384, 320), {"kind": "normal", "scale": s})], bf16=True)
    got = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
    assert O.max_abs_rel_err(got, golden["matmul_bf16in_384x256x320_seed1"]) <= 1e-6


@pytest.mark.parametrize(
    "key,seed,M,K,N,eps",
    [("rmsnorm_gamma_256x512x384_seed2", 2, 256, 512, 384, 1e-6), ("rmsnorm_gamma_16x1024x512_seed3", 3, 16, 1024, 512, 1e-5)],
)
def test_rmsnorm_with_gamma(golden, key, seed, M, K, N, eps):
    t = O.generate_inputs(seed, [("x", (M, K), None), ("gamma", (K,), U),
                                 ("weight", (K, N), {"kind": "normal", "scale": K ** -0.5})], bf16=True)
    got = O.rmsnorm_matmul(t["x"], t["gamma"], t["weight"], eps)
    assert O.max_abs_rel_err(got, golden[key]) <= 1e-6
    # independent float64 evaluation of the same formula
    x, g, w = (t[k].astype(np.float64) for k in ("x", "gamma", "weight"))
    ref = (x / np.sqrt((x * x).mean(axis=1, keepdims=True) + eps) * g) @ w
    assert O.max_abs_rel_err(got, ref) <= 1e-5


def test_hand_kernels_2048_samples(golden):
    """The oracle against the reference's two hand kernels run through its simulate_fp32.

    Tolerance 5e-3 abs/rel is the reference's own (examples/tune_matmul_lhsT_rhs.py:156,172);
    the hand kernels reduce K in two stages, so agreement is not bitwise.
    """
    t = O.generate_inputs(0, [("lhs_T", (2048, 2048), None), ("rhs", (2048, 2048), None)], bf16=False)
    mm = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
    np.testing.assert_allclose(mm[::127, ::131], golden["hand_matmul_2048_seed0_sample"], atol=5e-3, rtol=5e-3)
    np.testing.assert_allclose(mm.sum(axis=1, dtype=np.float64)[::64], golden["hand_matmul_2048_seed0_rowsum"],
                               atol=5e-2, rtol=1e-4)
    # same draws serve as (lhs, rhs) of the rmsnorm kernel: same seed, same order, same shapes
    rn = O.rmsnorm_matmul(t["lhs_T"], None, t["rhs"], 1e-6)
    np.testing.assert_allclose(rn[::127, ::131], golden["hand_rmsnorm_2048_seed0_sample"], atol=5e-3, rtol=5e-3)
    np.testing.assert_allclose(rn[::127, ::131], golden["ssa_rmsnorm_2048_seed0_sample"], atol=1e-5, rtol=1e-5)
    np.testing.assert_allclose(rn.sum(axis=1, dtype=np.float64)[::64], golden["hand_rmsnorm_2048_seed0_rowsum"],
                               atol=5e-2, rtol=1e-4)


def test_matmul_lhs_rhs_hand_kernel_sample(golden):
    t = O.generate_inputs(0, [("lhs", (2048, 2048), None), ("rhs", (2048, 2048), None)], bf16=False)
    got = O.matmul_lhs_rhs(t["lhs"], t["rhs"])
    np.testing.assert_allclose(got[::127, ::131], golden["hand_matmul_lhs_rhs_2048_seed0_sample"], atol=5e-3, rtol=5e-3)
    assert np.array_equal(got, t["lhs"] @ t["rhs"])


def test_error_metric_edge_cases():
    e = np.zeros((4, 4), dtype=np.float32)
    assert O.max_abs_rel_err(e, e) == 0.0
    a = np.ones((2, 2)); b = a * 1.01
    assert 0.004 < O.max_abs_rel_err(b, a) < 0.006


def test_generate_inputs_is_order_and_seed_stable():
    a = O.generate_inputs(5, [("p", (3, 4), None), ("q", (2,), U)], bf16=False)
    b = O.generate_inputs(5, [("p", (3, 4), None), ("q", (2,), U)], bf16=False)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    rng = np.random.default_rng(5)
    assert np.array_equal(a["p"], rng.standard_normal((3, 4)).astype(np.float32))
