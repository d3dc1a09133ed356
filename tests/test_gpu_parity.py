"""Parity of the CUDA kernels with the CPU oracle, through the C ABI (GPU box only).

Tolerances: max |a-e| / (|e| + rms(e)) <= 1e-2 for bf16 inputs with fp32 accumulation and
bf16 output; <= 1e-5 for the fp32 configuration.
"""

import ml_dtypes
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_BF16 = 1e-2
TOL_FP32 = 1e-5
U = {"kind": "uniform", "low": 0.5, "high": 1.5}
BF = ml_dtypes.bfloat16


def N_(k):
    return {"kind": "normal", "scale": k ** -0.5}


def cfg(tm, tn, tk, st, cm=1, sw=0, nm=0):
    return dict(tile_m=tm, tile_n=tn, tile_k=tk, stages=st, cluster_m=cm, swizzle=sw, norm_mode=nm)


@pytest.fixture(scope="module")
def K(native_lib):
    import torch

    assert torch.cuda.is_available()
    from autotune import kernels

    return kernels


def _mm_case(K, seed, k, m, n, c):
    t = O.generate_inputs(seed, [("lhs_T", (k, m), N_(k)), ("rhs", (k, n), N_(k))], bf16=True)
    got = K.matmul_lhsT_rhs_host(t["lhs_T"].astype(BF), t["rhs"].astype(BF), c).astype(np.float32)
    return O.max_abs_rel_err(got, O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"]))


# ---- fp32 configuration ----------------------------------------------------------------------
def test_fp32_config_512_matches_golden(K, golden):
    c = O.config_specs("cfg1_fp32_512")
    t = O.generate_inputs(c["seed"], c["specs"], c["bf16"])
    got = K.matmul_lhsT_rhs_host(t["lhs_T"], t["rhs"])
    assert O.max_abs_rel_err(got, golden["matmul_512_seed0"]) <= TOL_FP32
    assert O.max_abs_rel_err(got, O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])) <= TOL_FP32


def test_fp32_reference_op_case_128(K, golden):
    t = O.generate_inputs(0, [("lhs_T", (128, 128), None), ("rhs", (128, 128), None)], bf16=False)
    got = K.matmul_lhsT_rhs_host(t["lhs_T"], t["rhs"])
    assert np.allclose(got, golden["matmul_128_seed0"], atol=1e-4, rtol=1e-4)  # the reference's own tolerance


@pytest.mark.parametrize("k,m,n", [(1, 1, 1), (7, 13, 5), (300, 200, 136), (16, 65, 129)])
def test_fp32_ragged_shapes(K, k, m, n):
    t = O.generate_inputs(11, [("lhs_T", (k, m), None), ("rhs", (k, n), None)], bf16=False)
    got = K.matmul_lhsT_rhs_host(t["lhs_T"], t["rhs"])
    assert O.max_abs_rel_err(got, O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])) <= TOL_FP32


# ---- tcgen05 GEMM ----------------------------------------------------------------------------
def test_bf16_golden_case(K, golden):
    t = O.generate_inputs(1, [("lhs_T", (384, 256), N_(384)), ("rhs", (384, 320), N_(384))], bf16=True)
    got = K.matmul_lhsT_rhs_host(t["lhs_T"].astype(BF), t["rhs"].astype(BF), cfg(128, 64, 64, 3)).astype(np.float32)
    assert O.max_abs_rel_err(got, golden["matmul_bf16in_384x256x320_seed1"]) <= TOL_BF16


GRID = [cfg(tm, tn, tk, st, cm)
        for tm in (128, 256) for tn in (128, 256) for tk in (64, 128) for st in (3, 4) for cm in (1, 2)]


@pytest.mark.parametrize("c", GRID, ids=lambda c: f"{c['tile_m']}x{c['tile_n']}x{c['tile_k']}s{c['stages']}c{c['cluster_m']}")
def test_bf16_every_tile_candidate_small(K, c):
    """256x256x512 (the reference's cheap fixture shape family) for every point of the tile grid."""
    from autotune import native

    status, msg, _, _ = native.cfg_check("matmul_lhsT_rhs", c, 512, 512, 512)
    if status != native.OK:
        assert status in (native.ERR_SMEM_OOM, native.ERR_TMEM_OOM), msg
        with pytest.raises(native.NativeError):
            _mm_case(K, 5, 512, 512, 512, c)
        return
    assert _mm_case(K, 5, 512, 512, 512, c) <= TOL_BF16


@pytest.mark.parametrize("k,m,n", [(64, 128, 64), (8, 8, 8), (72, 136, 200), (520, 1000, 1016), (2048, 2048, 2048), (1000, 264, 72)])
@pytest.mark.parametrize("c", [cfg(128, 128, 64, 4), cfg(256, 128, 64, 4, cm=2), cfg(256, 128, 64, 3)],
                         ids=["1cta", "pair", "msub2"])
def test_bf16_edges_and_sizes(K, k, m, n, c):
    assert _mm_case(K, 6, k, m, n, c) <= TOL_BF16


@pytest.mark.parametrize("k,m,n", [(64, 256, 512), (520, 1000, 1016), (1024, 512, 2048)])
@pytest.mark.parametrize("c", [cfg(256, 512, 64, 4, cm=2), cfg(128, 512, 64, 2), cfg(256, 512, 128, 2, cm=2)], ids=["pair", "1cta", "pair-k128"])
def test_bf16_wide_tiles_two_ummas_along_n(K, k, m, n, c):
    assert _mm_case(K, 9, k, m, n, c) <= TOL_BF16


@pytest.mark.parametrize("k,m,n", [(64, 512, 256), (520, 1000, 1016), (1024, 2048, 512), (2048, 2048, 2048)])
@pytest.mark.parametrize("c", [cfg(512, 256, 64, 4, cm=2), cfg(512, 256, 128, 2, cm=2), cfg(512, 128, 64, 4, cm=2)],
                         ids=["512x256", "512x256-k128", "512x128"])
def test_bf16_tall_pair_tiles_two_ummas_along_m(K, k, m, n, c):
    assert _mm_case(K, 10, k, m, n, c) <= TOL_BF16


@pytest.mark.parametrize("k,m,n", [(512, 256, 384), (4096, 256, 4096), (520, 1000, 1016), (8192, 128, 512), (192, 136, 72)])
@pytest.mark.parametrize("c", [dict(cfg(256, 256, 128, 3, cm=2), split_k=4), dict(cfg(128, 128, 64, 4), split_k=3),
                               dict(cfg(512, 256, 64, 4, cm=2), split_k=2), dict(cfg(256, 128, 64, 3), split_k=16)],
                         ids=["pair-x4", "1cta-x3", "tall-x2", "msub2-x16"])
def test_bf16_split_k(K, k, m, n, c):
    """K range of every tile dealt to several work units, fp32 partials summed by a second kernel."""
    assert _mm_case(K, 12, k, m, n, c) <= TOL_BF16
    t = O.generate_inputs(12, [("lhs", (m, k), N_(k)), ("rhs", (k, n), N_(k))], bf16=True)
    got = K.to_host(K.matmul_lhs_rhs(K.to_device(t["lhs"].astype(BF)), K.to_device(t["rhs"].astype(BF)), cfg=c)).astype(np.float32)
    assert O.max_abs_rel_err(got, O.matmul_lhs_rhs(t["lhs"], t["rhs"])) <= TOL_BF16


def test_bf16_hand_kernel_shape_2048(K, golden):
    """2048^3, the only shape the reference's hand kernel accepts, against its simulated output."""
    t = O.generate_inputs(0, [("lhs_T", (2048, 2048), None), ("rhs", (2048, 2048), None)], bf16=True)
    got = K.matmul_lhsT_rhs_host(t["lhs_T"].astype(BF), t["rhs"].astype(BF)).astype(np.float32)
    assert O.max_abs_rel_err(got, O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])) <= TOL_BF16
    # the golden was computed from unrounded fp32 inputs: bf16 input rounding adds ~2^-9 relative noise per term
    sample, ref = got[::127, ::131], golden["hand_matmul_2048_seed0_sample"]
    assert np.max(np.abs(sample - ref)) / np.sqrt(np.mean(ref * ref)) <= 3e-2


def test_strided_operands(K):
    """A column slice of lhsT (the large-M shard case) and a padded output, no copies."""
    import torch

    k, m_total, n = 256, 1024, 256
    t = O.generate_inputs(8, [("lhs_T", (k, m_total), N_(k)), ("rhs", (k, n), N_(k))], bf16=True)
    a = K.to_device(t["lhs_T"].astype(BF))
    b = K.to_device(t["rhs"].astype(BF))
    out = torch.zeros(m_total, n + 64, dtype=torch.bfloat16, device="cuda")
    for g in range(4):
        K.matmul_lhsT_rhs(a[:, g * 256:(g + 1) * 256], b, cfg=cfg(128, 128, 64, 3), out=out[g * 256:(g + 1) * 256, :n])
    torch.cuda.synchronize()
    got = K.to_host(out).astype(np.float32)
    assert O.max_abs_rel_err(got[:, :n], O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])) <= TOL_BF16
    assert not got[:, n:].any()  # padding untouched


def test_linearity_and_determinism_full_size(K):
    """Size-independent properties at 8192^3: C(a, 2b) = 2 C(a, b) exactly in bf16 (power-of-two
    scale), and two launches agree bit for bit."""
    import torch

    torch.manual_seed(1)
    a = (torch.randn(8192, 8192, device="cuda") * 8192 ** -0.5).bfloat16()
    b = (torch.randn(8192, 8192, device="cuda") * 8192 ** -0.5).bfloat16()
    c1 = K.matmul_lhsT_rhs(a, b)
    c2 = K.matmul_lhsT_rhs(a, b)
    c3 = K.matmul_lhsT_rhs(a, b * 2)
    torch.cuda.synchronize()
    assert torch.equal(c1, c2)
    assert torch.equal(c3, c1 * 2)
    # column-sum checksum against an fp32 evaluation: sum_m C[m, n] = (sum_m lhsT[:, m]) . rhs[:, n]
    ref = (a.float().sum(dim=1) @ b.float())
    got = c1.float().sum(dim=0)
    assert float((got - ref).abs().max() / ref.abs().max()) < 2e-2


def test_host_pipeline_keeps_every_step_apart(K):
    """The host-buffer pipeline (pinned staging, uploads / kernels / downloads overlapped over two
    buffer sets): five different operand pairs in a row, each result against the CPU oracle."""
    from autotune.pipeline import matmul_lhsT_rhs_pipelined

    k, m, n = 512, 384, 640
    pairs = [O.generate_inputs(40 + i, [("lhs_T", (k, m), N_(k)), ("rhs", (k, n), N_(k))], bf16=True) for i in range(5)]
    outs = matmul_lhsT_rhs_pipelined([p["lhs_T"].astype(BF) for p in pairs], [p["rhs"].astype(BF) for p in pairs],
                                     cfg=cfg(128, 128, 64, 3))
    assert len(outs) == 5
    for p, got in zip(pairs, outs):
        assert O.max_abs_rel_err(got.astype(np.float32), O.matmul_lhsT_rhs(p["lhs_T"], p["rhs"])) <= TOL_BF16


# ---- matmul_lhs_rhs (K-major lhs) --------------------------------------------------------------
@pytest.mark.parametrize("k,m,n", [(64, 128, 64), (512, 256, 384), (520, 1000, 1016), (2048, 2048, 2048), (72, 136, 200)])
@pytest.mark.parametrize("c", [cfg(128, 128, 64, 4), cfg(128, 256, 128, 2), cfg(256, 256, 64, 4, cm=2), cfg(256, 128, 64, 3), None],
                         ids=["1cta", "1cta-k128", "pair", "msub2", "default"])
def test_matmul_lhs_rhs(K, k, m, n, c):
    t = O.generate_inputs(7, [("lhs", (m, k), N_(k)), ("rhs", (k, n), N_(k))], bf16=True)
    got = K.to_host(K.matmul_lhs_rhs(K.to_device(t["lhs"].astype(BF)), K.to_device(t["rhs"].astype(BF)), cfg=c)).astype(np.float32)
    assert O.max_abs_rel_err(got, O.matmul_lhs_rhs(t["lhs"], t["rhs"])) <= TOL_BF16


def test_matmul_lhs_rhs_hand_kernel_shape_2048(K, golden):
    t = O.generate_inputs(0, [("lhs", (2048, 2048), None), ("rhs", (2048, 2048), None)], bf16=True)
    got = K.to_host(K.matmul_lhs_rhs(K.to_device(t["lhs"].astype(BF)), K.to_device(t["rhs"].astype(BF)))).astype(np.float32)
    sample, ref = got[::127, ::131], golden["hand_matmul_lhs_rhs_2048_seed0_sample"]
    assert np.max(np.abs(sample - ref)) / np.sqrt(np.mean(ref * ref)) <= 3e-2   # bf16 input rounding vs fp32 golden


# ---- fused RMSNorm + matmul ------------------------------------------------------------------
def _rms_case(K, seed, m, k, n, eps, c, gamma=True):
    t = O.generate_inputs(seed, [("x", (m, k), None), ("gamma", (k,), U), ("weight", (k, n), N_(k))], bf16=True)
    g = t["gamma"] if gamma else None
    got = K.rmsnorm_matmul_host(t["x"].astype(BF), g.astype(BF) if gamma else None, t["weight"].astype(BF), eps, c)
    return got.astype(np.float32), O.rmsnorm_matmul(t["x"], g, t["weight"], eps)


@pytest.mark.parametrize("key,seed,m,k,n,eps", [("rmsnorm_gamma_256x512x384_seed2", 2, 256, 512, 384, 1e-6),
                                                ("rmsnorm_gamma_16x1024x512_seed3", 3, 16, 1024, 512, 1e-5)])
@pytest.mark.parametrize("c", [cfg(128, 128, 64, 3), cfg(128, 128, 128, 2), cfg(256, 128, 64, 3), cfg(256, 128, 64, 3, cm=2)],
                         ids=["1cta", "tk128", "msub2", "pair"])
def test_rmsnorm_golden_cases(K, golden, key, seed, m, k, n, eps, c):
    got, expect = _rms_case(K, seed, m, k, n, eps, c)
    assert O.max_abs_rel_err(got, golden[key]) <= TOL_BF16
    assert O.max_abs_rel_err(got, expect) <= TOL_BF16


@pytest.mark.parametrize("m,k,n", [(1000, 512, 1016), (2048, 2048, 2048), (520, 64, 264)])
@pytest.mark.parametrize("c", [cfg(512, 256, 64, 4, cm=2, nm=2), cfg(512, 128, 128, 2, cm=2, nm=2), cfg(256, 512, 64, 4, cm=2, nm=2)],
                         ids=["512x256", "512x128-k128", "256x512"])
def test_rmsnorm_prologue_variant_with_large_pair_tiles(K, m, k, n, c):
    got, expect = _rms_case(K, 13, m, k, n, 1e-6, c)
    assert O.max_abs_rel_err(got, expect) <= TOL_BF16


@pytest.mark.parametrize("nm", [1, 2], ids=["inline", "prologue"])
@pytest.mark.parametrize("m,k,n", [(256, 512, 384), (1000, 512, 1016), (2048, 2048, 2048), (136, 64, 72)])
@pytest.mark.parametrize("tiles", [(128, 128, 64, 3, 1), (128, 256, 128, 2, 1), (256, 256, 64, 4, 2), (256, 256, 128, 3, 2),
                                   (256, 128, 64, 3, 1)], ids=["1cta", "1cta-k128", "pair", "pair-k128", "msub2"])
def test_rmsnorm_both_norm_placements(K, nm, m, k, n, tiles):
    """Inline (tensor-memory path) and prologue (same-launch scratch) variants, twice in a row."""
    tm, tn, tk, st, cm = tiles
    for _ in range(2):
        got, expect = _rms_case(K, 23, m, k, n, 1e-6, cfg(tm, tn, tk, st, cm=cm, nm=nm))
        assert O.max_abs_rel_err(got, expect) <= TOL_BF16


def test_rmsnorm_prologue_needs_workspace(K):
    import torch

    from autotune import native

    lib = native.load()
    x = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    c = native.Cfg.from_dict(cfg(128, 128, 64, 3, nm=2))
    import ctypes as C

    rc = lib.b200_rmsnorm_matmul(x.data_ptr(), None, w.data_ptr(), out.data_ptr(), 128, 256, 256, 1e-6, C.byref(c), None, 0,
                                 None, torch.cuda.current_stream().cuda_stream)
    assert rc == native.ERR_WORKSPACE
    c1 = native.Cfg.from_dict(cfg(128, 128, 64, 3, nm=1))
    assert lib.b200_workspace_bytes(b"rmsnorm_matmul", C.byref(c1), 128, 256, 256) == 0
    assert lib.b200_workspace_bytes(b"rmsnorm_matmul", C.byref(c), 128, 256, 256) >= 128 * 256 * 2 + 128 * 4


def test_rmsnorm_without_gamma_is_reference_kernel_maths(K, golden):
    t = O.generate_inputs(0, [("lhs", (2048, 2048), None), ("rhs", (2048, 2048), None)], bf16=True)
    got = K.rmsnorm_matmul_host(t["lhs"].astype(BF), None, t["rhs"].astype(BF), 1e-6).astype(np.float32)
    assert O.max_abs_rel_err(got, O.rmsnorm_matmul(t["lhs"], None, t["rhs"], 1e-6)) <= TOL_BF16
    sample, ref = got[::127, ::131], golden["hand_rmsnorm_2048_seed0_sample"]
    assert np.max(np.abs(sample - ref)) / np.sqrt(np.mean(ref * ref)) <= 3e-2


def test_rmsnorm_row_scale_invariance(K):
    """rmsnorm(c * x) = rmsnorm(x) for c a power of two (eps negligible): outputs agree closely."""
    g1, _ = _rms_case(K, 9, 256, 512, 256, 1e-12, cfg(128, 128, 64, 3))
    t = O.generate_inputs(9, [("x", (256, 512), None), ("gamma", (512,), U), ("weight", (512, 256), N_(512))], bf16=True)
    got4 = K.rmsnorm_matmul_host((t["x"] * 4).astype(BF), t["gamma"].astype(BF), t["weight"].astype(BF), 1e-12,
                                 cfg(128, 128, 64, 3)).astype(np.float32)
    assert O.max_abs_rel_err(got4, g1) <= 1e-2


def test_fused_matches_fp32_device_crosscheck(K):
    import torch

    t = O.generate_inputs(4, [("x", (512, 1024), None), ("gamma", (1024,), U), ("weight", (1024, 768), N_(1024))], bf16=True)
    x, g, w = (K.to_device(t[k].astype(BF)) for k in ("x", "gamma", "weight"))
    ref = K.rmsnorm_matmul_f32(x, g, w, 1e-6)
    out = K.rmsnorm_matmul(x, g, w, 1e-6, cfg(128, 256, 64, 4))
    torch.cuda.synchronize()
    assert O.max_abs_rel_err(K.to_host(ref), O.rmsnorm_matmul(t["x"], t["gamma"], t["weight"], 1e-6)) <= 1e-4
    assert O.max_abs_rel_err(K.to_host(out).astype(np.float32), K.to_host(ref)) <= TOL_BF16


# ---- skinny activations: weight-streaming kernel with scratch ----------------------------------
@pytest.mark.parametrize("m,k,n", [(16, 64, 128), (16, 1024, 512), (8, 256, 200), (1, 512, 1024), (16, 4096, 4096), (12, 2048, 3080)])
@pytest.mark.parametrize("c", [cfg(16, 128, 64, 3), cfg(16, 128, 128, 2), None], ids=["tk64", "tk128", "default"])
def test_rmsnorm_skinny_shapes(K, m, k, n, c):
    eps = 1e-5
    for _ in range(2):  # the second call runs on the scratch the first one left behind
        got, expect = _rms_case(K, 21, m, k, n, eps, c)
        assert O.max_abs_rel_err(got, expect) <= TOL_BF16


@pytest.mark.parametrize("m,k,n", [
    (16, 256, 37888),   # 148 tiles on 148 SMs: one whole tile per CTA, nothing shared
    (16, 128, 40000),   # whole tiles plus a few left-over tiles with owners and donors; ragged last tile
    (4, 192, 9472),     # K not a multiple of the 128-deep stage; fewer tiles than SMs
    (16, 8192, 512),    # two tiles, every CTA a donor or an owner of a long K range
])
def test_rmsnorm_skinny_work_splits(K, m, k, n):
    """Shapes that exercise every branch of the tile split of the weight-streaming kernel (whole
    tiles only, whole tiles + shared left-over tiles, shared tiles only), twice on one scratch."""
    for _ in range(2):
        got, expect = _rms_case(K, 23, m, k, n, 1e-5, None)
        assert O.max_abs_rel_err(got, expect) <= TOL_BF16


def test_rmsnorm_skinny_chain_of_dependent_launches(K):
    """The weight-streaming kernel is a programmatic dependent launch: in a chain it starts (and
    streams its weights) while its predecessor finishes, and waits for it before touching x, the
    scratch or out.  A chain whose launches alternate between two activations and three weight
    copies, every launch on the scratch its predecessor just used, must give each launch's own
    result; so must the same chain launched the ordinary way."""
    import torch

    m, k, n = 16, 1024, 9472
    t = O.generate_inputs(24, [("x", (m, k), None), ("gamma", (k,), U), ("weight", (k, n), N_(k))], bf16=True)
    xs = [K.to_device(t["x"].astype(BF)), K.to_device((t["x"] * 0.5).astype(BF))]
    g = K.to_device(t["gamma"].astype(BF))
    ws = [K.to_device(t["weight"].astype(BF)) for _ in range(3)]
    expect = [O.rmsnorm_matmul(t["x"] * s, t["gamma"], t["weight"], 1e-5) for s in (1.0, 0.5)]
    torch.cuda.synchronize()
    for c in (None, dict(tile_m=16, tile_n=256, tile_k=128, stages=3, _serial_launch=1)):
        outs = [K.rmsnorm_matmul(xs[i % 2], g, ws[i % 3], eps=1e-5, cfg=c) for i in range(12)]
        torch.cuda.synchronize()
        for i, o in enumerate(outs):
            assert O.max_abs_rel_err(K.to_host(o).astype(np.float32), expect[i % 2]) <= TOL_BF16, (c, i)


def test_rmsnorm_skinny_counters_are_left_zero_and_slots_need_no_clearing(K):
    """The scratch starts with one counter per 256-column tile (zero between launches); the
    partial-tile slots behind them are written before they are read, so stale contents are harmless."""
    import torch

    first, expect = _rms_case(K, 22, 16, 2048, 4096, 1e-5, None)
    ws = K.workspace_for("rmsnorm_matmul", 16, 4096, 2048, "cuda")
    torch.cuda.synchronize()
    tiles = 4096 // 256
    assert ws is not None and int((ws.view(torch.uint8)[: tiles * 4] != 0).sum()) == 0
    ws.view(torch.uint8)[256:].fill_(0x7F)                       # NaN-ish garbage in every slot
    again, _ = _rms_case(K, 22, 16, 2048, 4096, 1e-5, None)
    assert np.array_equal(again, first) and O.max_abs_rel_err(again, expect) <= TOL_BF16
    assert int((ws.view(torch.uint8)[: tiles * 4] != 0).sum()) == 0


def test_rmsnorm_skinny_without_workspace_is_an_error(K):
    """Straight through the C ABI: the skinny kernel refuses to run without its scratch."""
    import torch

    from autotune import native

    lib = native.load()
    x = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(16, 256, dtype=torch.bfloat16, device="cuda")
    rc = lib.b200_rmsnorm_matmul(x.data_ptr(), None, w.data_ptr(), out.data_ptr(), 16, 256, 256, 1e-5, None, None, 0, None,
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == native.ERR_WORKSPACE and "workspace" in native.last_error()
    assert lib.b200_workspace_bytes(b"rmsnorm_matmul", None, 16, 256, 256) >= 16 * 256 * 4
    assert lib.b200_workspace_bytes(b"matmul_lhsT_rhs", None, 4096, 256, 256) == 0


# ---- argument checking and bounded waits -------------------------------------------------------
def test_bad_arguments_raise(K):
    import torch

    from autotune.native import NativeError

    a = torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NativeError):
        K.matmul_lhsT_rhs(a, torch.zeros(32, 128, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(NativeError):
        K.matmul_lhsT_rhs(a, a, cfg=cfg(128, 128, 64, 99))
    with pytest.raises(NativeError):
        K.matmul_lhsT_rhs(torch.zeros(64, 100, dtype=torch.bfloat16, device="cuda"), a)  # M not a multiple of 8


def test_wait_that_runs_out_reports_status_and_context_survives(K):
    """A producer that issues nothing makes the consumer's bounded wait expire: the launch ends,
    the status block names the wait, and the next launch on the same context is correct."""
    import torch

    from autotune.native import NativeError

    a = torch.ones(128, 256, dtype=torch.bfloat16, device="cuda")
    st = K.new_status()
    c = cfg(128, 128, 64, 3)
    c.update(_debug_skip_producer=1, _wait_limit_us=2000)
    K.matmul_lhsT_rhs(a, a, cfg=c, status=st)
    with pytest.raises(NativeError, match="wait expired"):
        K.raise_on_status(st)
    assert st.cpu()[0].item() == 7
    assert _mm_case(K, 3, 256, 256, 256, cfg(128, 128, 64, 3)) <= TOL_BF16
