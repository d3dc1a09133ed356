"""BASELINE-size configurations on the GPU: sampled rows against the CPU oracle plus properties
that do not depend on the size (scale invariance of the norm, linearity, checksums, determinism).

Inputs are seeded synthetic tensors with the shapes and distributions of the benchmark
configurations; rows compared with the oracle are a sample, so that the CPU side stays at seconds."""

import ml_dtypes
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
BF = ml_dtypes.bfloat16


@pytest.fixture(scope="module")
def K(native_lib):
    from autotune import kernels

    return kernels


def _bf16_dev(K, arr):
    return K.to_device(arr.astype(BF))


def test_fused_config_4096x11008x4096(K):
    """configs[2]: x[4096,4096], gamma U(0.5,1.5), weight N(0,1)/sqrt(K), eps 1e-6."""
    import torch

    spec = O.config_specs("cfg3_rmsnorm_4096")
    t = O.generate_inputs(spec["seed"], spec["specs"], bf16=True)
    x, g, w = _bf16_dev(K, t["x"]), _bf16_dev(K, t["gamma"]), _bf16_dev(K, t["weight"])
    out = K.rmsnorm_matmul(x, g, w, eps=1e-6)                        # default: prologue variant
    inline = K.rmsnorm_matmul(x, g, w, eps=1e-6, cfg=dict(tile_m=128, tile_n=256, tile_k=128, stages=2, cluster_m=1, norm_mode=1))
    again = K.rmsnorm_matmul(x, g, w, eps=1e-6)
    scaled = K.rmsnorm_matmul(x * 4, g, w, eps=1e-6 * 16)           # rmsnorm(4x; 16 eps) == rmsnorm(x; eps) exactly
    torch.cuda.synchronize()
    assert torch.equal(out, again)
    assert torch.equal(out, scaled)
    rows = np.arange(0, 4096, 97)                                     # 43 rows spread over every M tile
    expect = O.rmsnorm_matmul(t["x"][rows], t["gamma"], t["weight"], 1e-6)
    got = K.to_host(out).astype(np.float32)
    assert O.max_abs_rel_err(got[rows], expect) <= TOL_BF16
    assert O.max_abs_rel_err(K.to_host(inline).astype(np.float32)[rows], expect) <= TOL_BF16
    assert np.isfinite(got).all()


def test_skinny_config_16x28672x8192(K):
    """configs[3]: the decode shape, every output against the oracle, twice (scratch reuse)."""
    import torch

    spec = O.config_specs("cfg4_rmsnorm_skinny")
    t = O.generate_inputs(spec["seed"], spec["specs"], bf16=True)
    x, g, w = _bf16_dev(K, t["x"]), _bf16_dev(K, t["gamma"]), _bf16_dev(K, t["weight"])
    first = K.rmsnorm_matmul(x, g, w, eps=1e-5)
    second = K.rmsnorm_matmul(x, g, w, eps=1e-5)
    torch.cuda.synchronize()
    assert torch.equal(first, second)
    expect = O.rmsnorm_matmul(t["x"], t["gamma"], t["weight"], 1e-5)
    assert O.max_abs_rel_err(K.to_host(first).astype(np.float32), expect) <= TOL_BF16


def test_matmul_config_8192_every_output_against_the_oracle(K):
    """configs[1] on its own seeded inputs (default_rng(1), N(0,1)/sqrt(K), bf16-rounded): the
    library default and the four configurations the benchmark chooses among, EVERY output against
    the CPU oracle (one fp32 BLAS product of the same inputs)."""
    import torch

    spec = O.config_specs("cfg2_bf16_8192")
    t = O.generate_inputs(spec["seed"], spec["specs"], bf16=True)
    expect = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
    a, b = _bf16_dev(K, t["lhs_T"]), _bf16_dev(K, t["rhs"])
    configs = [None,
               dict(tile_m=512, tile_n=256, tile_k=64, stages=4, cluster_m=2),
               dict(tile_m=256, tile_n=512, tile_k=64, stages=4, cluster_m=2),
               dict(tile_m=256, tile_n=256, tile_k=128, stages=3, cluster_m=2),
               dict(tile_m=128, tile_n=256, tile_k=128, stages=2, cluster_m=1)]
    out = torch.empty(8192, 8192, dtype=torch.bfloat16, device="cuda")
    for cfg in configs:
        out.zero_()
        K.matmul_lhsT_rhs(a, b, cfg=cfg, out=out)
        torch.cuda.synchronize()
        err = O.max_abs_rel_err(K.to_host(out).astype(np.float32), expect)
        assert err <= TOL_BF16, f"{cfg}: max-abs-rel error {err:.3e}"


def test_large_m_config_131072x4096x4096(K):
    """configs[4] on one GPU, on its own seeded inputs (default_rng(4): lhsT[4096,131072] = 1 GiB in
    bf16, rhs[4096,4096]): 128 rows spread over the whole of M against the CPU oracle, the
    column-sum checksum, and a row block computed from a column slice of lhsT."""
    import torch

    spec = O.config_specs("cfg5_large_m")
    t = O.generate_inputs(spec["seed"], spec["specs"], bf16=True)
    Kd, M = t["lhs_T"].shape
    a, b = _bf16_dev(K, t["lhs_T"]), _bf16_dev(K, t["rhs"])
    c = K.matmul_lhsT_rhs(a, b)
    block = K.matmul_lhsT_rhs(a[:, 65536:65536 + 16384], b)         # one rank's share of an 8-way split
    torch.cuda.synchronize()
    assert torch.equal(block, c[65536:65536 + 16384])
    rows = np.arange(5, M, 1031)[:128]                                # 128 rows, every 512-row tile class
    expect = O.matmul_lhsT_rhs(np.ascontiguousarray(t["lhs_T"][:, rows]), t["rhs"])
    got = K.to_host(c[torch.from_numpy(rows).cuda()]).astype(np.float32)
    assert O.max_abs_rel_err(got, expect) <= TOL_BF16
    ref = a.float().sum(dim=1) @ b.float()                           # sum_m C[m, n]
    got_sum = c.float().sum(dim=0)
    assert float((got_sum - ref).abs().max() / ref.abs().max()) < 2e-2
