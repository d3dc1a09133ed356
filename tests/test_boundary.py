"""Drop-in boundary on CPU: result types, cache writers, candidate descriptors, budget
checks, and that the shared library exports every symbol the header declares."""

import json
import re

import numpy as np
import pytest

from autotune.runner.candidate import Candidate, enumerate_grid, extended_grid, jobs_from_candidates, parse_source
from autotune.runner.output import ProfileOutput, write_kernel_sources, write_results_json
from autotune.runner.types import KernelJob, ProfileResult, make_failure, profiler_percent, resolve_dtype, tensor_inputs

from conftest import REPO


def _ok(name, t, mfu, **extra):
    return ProfileResult(name, "[128, 512] float32", {"total_time": t, "mfu_estimated_percent": mfu, **extra})


# ---- behaviour pinned by the reference's test/runner/test_output.py ------------------------
def test_results_json_has_no_hosts_key(tmp_path):
    write_results_json(str(tmp_path), num_kernels=1, results=[_ok("k_0.py", 0.001, 0.9)], wallclock_s=1.5)
    data = json.loads((tmp_path / "results.json").read_text())
    assert "hosts" not in data["metadata"]
    assert data["metadata"] == {"num_kernels": 1, "wallclock_s": 1.5}
    assert data["metrics"]["success"] == 1
    assert data["kernels"][0]["kernel_name"] == "k_0.py"


def test_results_json_sorts_numerically(tmp_path):
    write_results_json(str(tmp_path), 2, [_ok("kernel_10.py", 0.002, 0.5), _ok("kernel_2.py", 0.001, 0.5)], 1.0)
    data = json.loads((tmp_path / "results.json").read_text())
    assert [k["kernel_name"] for k in data["kernels"]] == ["kernel_2.py", "kernel_10.py"]


def test_profile_output_str():
    out = ProfileOutput([_ok("k_0.py", 0.001, 0.9)], {}, 2.0, "")
    text = str(out)
    assert "Hosts:" not in text and "Succeeded:  1/1" in text and "90.00%" in text


# ---- further behaviour of the same module ---------------------------------------------------
def test_results_json_schema_and_counters(tmp_path):
    results = [
        _ok("m_0.py", 0.002, 0.4, mbu_estimated_percent=0.1, mfu_max_achievable_estimated_percent=1.0),
        _ok("m_1.py", 0.001, 0.8),
        make_failure("m_2.py", "Out of memory in smem: 5 stages ..."),
        make_failure("m_3.py", "Out of memory in tmem: ..."),
        make_failure("m_4.py", "Out of memory in sbuf"),
        ProfileResult("m_5.py", "[1, 1] x", {"total_time": None, "mfu_estimated_percent": -1.0}),
    ]
    write_results_json(str(tmp_path), 6, results, 3.0)
    data = json.loads((tmp_path / "results.json").read_text())
    m = data["metrics"]
    assert (m["success"], m["smem_oom"], m["tmem_oom"], m["sbuf_oom"], m["psum_oom"]) == (2, 1, 1, 1, 0)
    assert m["best_kernel"] == "m_1.py" and m["worst_kernel"] == "m_0.py"
    assert m["best_total_time_s"] == 0.001 and m["best_mfu"] == pytest.approx(80.0) and m["best_mbu"] == pytest.approx(10.0)
    row = data["kernels"][0]
    assert set(row) == {"kernel_name", "kernel_path", "hardware_output", "total_time_s", "mfu_estimated_percent",
                        "mbu_estimated_percent", "mfu_max_achievable_estimated_percent"}
    assert row["kernel_path"] == "m_0/m_0.py"
    assert json.loads((tmp_path / "m_0" / "profile_summary.json").read_text())["total_time"] == 0.002
    assert not (tmp_path / "m_2" / "profile_summary.json").exists()


def test_success_and_failure_partition():
    rs = [_ok("a_0.py", 0.1, 0.5), make_failure("a_1.py", "Traceback ..."),
          ProfileResult("a_2.py", "[1] f", {"total_time": 0.1, "mfu_estimated_percent": -0.5})]
    out = ProfileOutput(rs, {}, 1.0)
    assert [s.kernel_name for s in out.successes] == ["a_0.py"]
    assert [f.kernel_name for f in out.failures] == ["a_1.py"]
    assert "1 failures:" in str(out)


def test_types_helpers():
    assert profiler_percent({"x": 0.25}, "x") == 25.0
    assert profiler_percent({"x": -1}, "x") is None and profiler_percent(None, "x") is None
    assert resolve_dtype("bfloat16").itemsize == 2 and resolve_dtype("float32") == np.float32
    assert len(tensor_inputs({"a": np.zeros((2, 2)), "s": 3.0, "b": np.zeros(3)})) == 2
    job = KernelJob("src", "f", (1, 2), {"a": ((1, 2), "float32")})
    assert job.neuronx_cc_args == () and job.lnc == 1


def test_write_kernel_sources(tmp_path):
    jobs = jobs_from_candidates(enumerate_grid("matmul_lhsT_rhs")[:2], (256, 256),
                                {"lhs_T": ((128, 256), "bfloat16"), "rhs": ((128, 256), "bfloat16")})
    write_kernel_sources(str(tmp_path), jobs)
    text = (tmp_path / "matmul_lhsT_rhs_1" / "matmul_lhsT_rhs_1.py").read_text()
    assert parse_source(text).family == "matmul_lhsT_rhs"


# ---- candidate descriptors -------------------------------------------------------------------
def test_candidate_round_trip_and_grid():
    c = Candidate("rmsnorm_matmul", {"tile_m": 128, "tile_n": 256, "tile_k": 64, "stages": 4}, {"eps": 1e-6})
    back = parse_source(c.to_source())
    assert back.family == c.family and back.config["tile_n"] == 256 and back.scalars == {"eps": 1e-6}
    assert back.config["cluster_m"] == 1 and back.config["norm_mode"] == 0
    assert parse_source(Candidate("matmul_lhs_rhs", {"tile_m": 128, "norm_mode": 2}).to_source()).config["norm_mode"] == 2
    grid = enumerate_grid("matmul_lhsT_rhs")
    assert len(grid) == 64 and len({tuple(sorted(g.config.items())) for g in grid}) == 64
    ext = extended_grid("matmul_lhsT_rhs")
    assert len(ext) == 94 and ext[:64] == grid and len({tuple(sorted(g.config.items())) for g in ext}) == 94
    assert sorted({g.config["swizzle"] for g in ext[88:]}) == [1, 4, 8]
    with pytest.raises(ValueError):
        parse_source("FAMILY = 'nope'\n")
    with pytest.raises(ValueError):
        parse_source("def f(:\n")


# ---- native library: exports + budget checks (no GPU needed) ---------------------------------
def test_library_exports_every_declared_symbol(native_lib):
    header = (REPO / "include" / "b200_autotune.h").read_text()
    declared = set(re.findall(r"^(?:int|size_t|const char\*)\s+(b200_\w+)\s*\(", header, flags=re.M))
    from autotune import native

    assert declared == set(native.SIGNATURES), declared ^ set(native.SIGNATURES)
    for name in declared:
        assert hasattr(native_lib, name), name
    assert native_lib.b200_abi_version() == 1


def test_checked_variant_exports_the_same_symbols_and_normal_one_reports_none(native_lib, checked_lib_path):
    """The checked library is a drop-in (selected with B200_AUTOTUNE_LIB); the normal one answers
    that it has no device-side check record."""
    import ctypes as C

    from autotune import native

    checked = C.CDLL(str(checked_lib_path))
    for name in native.SIGNATURES:
        assert hasattr(checked, name), name
    assert checked.b200_abi_version() == 1
    out = (C.c_longlong * 4)(7, 7, 7, 7)
    assert native_lib.b200_checked_build_report(out, 0) == native.ERR_UNSUPPORTED and list(out) == [0, 0, 0, 0]


def test_cfg_check_budgets(native_lib):
    from autotune import native

    ok = native.cfg_check("matmul_lhsT_rhs", dict(tile_m=128, tile_n=256, tile_k=64, stages=4, cluster_m=1), 8192, 8192, 8192)
    assert ok[0] == native.OK and ok[2] <= 232448 and ok[3] == 512
    oom = native.cfg_check("matmul_lhsT_rhs", dict(tile_m=128, tile_n=256, tile_k=64, stages=5, cluster_m=1), 8192, 8192, 8192)
    assert oom[0] == native.ERR_SMEM_OOM and "Out of memory in smem" in oom[1] and oom[2] > 232448
    assert native.cfg_check("matmul_lhsT_rhs", dict(tile_m=96, tile_n=256, tile_k=64, stages=4))[0] == native.ERR_UNSUPPORTED
    # 512-row tiles exist only as a CTA pair issuing two UMMAs along M; all 512 accumulator columns are in use
    tall = native.cfg_check("matmul_lhsT_rhs", dict(tile_m=512, tile_n=256, tile_k=64, stages=4, cluster_m=2))
    assert tall[0] == native.OK and tall[3] == 512
    assert native.cfg_check("matmul_lhsT_rhs", dict(tile_m=512, tile_n=256, tile_k=64, stages=4, cluster_m=1))[0] == native.ERR_UNSUPPORTED
    assert native.cfg_check("matmul_lhsT_rhs", dict(tile_m=512, tile_n=256, tile_k=64, stages=5, cluster_m=2))[0] == native.ERR_SMEM_OOM
    assert native.cfg_check("matmul_lhsT_rhs", dict(tile_m=512, tile_n=512, tile_k=64, stages=2, cluster_m=2))[0] == native.ERR_TMEM_OOM
    assert native.cfg_check("matmul_lhsT_rhs", dict(tile_m=128, tile_n=256, tile_k=64, stages=4), 100, 64, 64)[0] == native.ERR_BAD_SHAPE
    assert native.cfg_check("nope", None)[0] == native.ERR_BAD_ARG
    assert native.cfg_check("rmsnorm_matmul", None, 4096, 11008, 4096)[0] == native.OK
    accepted = sum(native.cfg_check("matmul_lhsT_rhs", c.config, 8192, 8192, 8192)[0] == native.OK
                   for c in enumerate_grid("matmul_lhsT_rhs"))
    assert 0 < accepted < 64  # the grid holds both runnable and over-subscribed points
    big = [native.cfg_check("matmul_lhsT_rhs", c.config, 8192, 8192, 8192)[0] for c in extended_grid("matmul_lhsT_rhs")[64:]]
    assert native.OK in big and native.ERR_SMEM_OOM in big and set(big) <= {native.OK, native.ERR_SMEM_OOM}
    print("accepted of the 64-point grid:", accepted, "of the 30 extra points:", big.count(native.OK))


def test_describe_launch_reports_the_plan(native_lib):
    """The launch description a detailed profile stores: schedule arithmetic checked by hand for
    the headline shape (512 tiles over 74 CTA pairs = 6.92 waves, 7 tiles on the busiest pair,
    7 x 128 k-blocks x 4 UMMA steps x 2 row blocks x 128 cycles)."""
    from autotune import native

    d = native.describe_launch("matmul_lhsT_rhs", dict(tile_m=512, tile_n=256, tile_k=64, stages=4, cluster_m=2), 8192, 8192, 8192)
    assert d["kernel"] == "gemm_tcgen05_kernel<2,2,lhsT>" and d["cluster"] == 2 and d["tmem_cols"] == 512 and d["acc_bufs"] == 1
    if not d["sm_count_from_device"]:
        assert d["grid"] == 148 and d["cta_groups"] == 74 and d["tiles"] == 512 and d["tiles_of_busiest_group"] == 7
        assert abs(d["waves"] - 512 / 74) < 1e-3 and d["umma_bound_sm_cycles"] == 7 * 128 * 4 * 2 * 128
        assert d["registers"] is None
    assert d["smem_bytes"] <= 232448
    f = native.describe_launch("rmsnorm_matmul", None, 4096, 11008, 4096)
    assert f["kernel"].endswith("norm>") and f["tiles"] == 8 * 43
    sk = native.describe_launch("rmsnorm_matmul", None, 16, 28672, 8192)
    assert sk["kernel"] == "rmsnorm_skinny_kernel" and sk["tiles_256_columns"] == 112
    capped = native.describe_launch("matmul_lhsT_rhs", dict(tile_m=512, tile_n=256, tile_k=64, stages=4, cluster_m=2, _max_ctas=132), 8192, 8192, 8192)
    assert capped["grid"] <= 132


def test_split_k_validation_and_scratch(native_lib):
    import ctypes as C

    from autotune import native
    from autotune.native import Cfg

    pair = dict(tile_m=256, tile_n=256, tile_k=128, stages=3, cluster_m=2)
    assert native.cfg_check("matmul_lhsT_rhs", dict(pair, split_k=4), 256, 4096, 4096)[0] == native.OK
    assert native.cfg_check("matmul_lhs_rhs", dict(pair, split_k=16), 256, 4096, 4096)[0] == native.OK
    assert native.cfg_check("matmul_lhsT_rhs", dict(pair, split_k=17), 256, 4096, 4096)[0] == native.ERR_UNSUPPORTED
    assert native.cfg_check("rmsnorm_matmul", dict(pair, split_k=2, norm_mode=2), 4096, 4096, 4096)[0] == native.ERR_UNSUPPORTED
    assert native.cfg_check("rmsnorm_matmul", dict(pair, split_k=2, norm_mode=1), 4096, 4096, 4096)[0] == native.ERR_UNSUPPORTED
    lib = native.load()

    def ws(fam, c, M, N, K):
        cc = Cfg.from_dict(c)
        return lib.b200_workspace_bytes(fam, C.byref(cc), M, N, K)

    assert ws(b"matmul_lhsT_rhs", dict(pair, split_k=4), 256, 4096, 4096) == 4 * 256 * 4096 * 4
    assert ws(b"matmul_lhsT_rhs", dict(pair, split_k=4), 200, 4096, 4096) == 4 * 256 * 4096 * 4   # rows padded to the tile
    assert ws(b"matmul_lhsT_rhs", dict(pair, split_k=8), 256, 4096, 256) == 2 * 256 * 4096 * 4    # only 2 k-blocks to deal out
    assert ws(b"matmul_lhsT_rhs", dict(pair, split_k=1), 256, 4096, 4096) == 0


def test_default_candidate_follows_the_problem_size(native_lib):
    """No cfg: large problems get the 512x256 pair tile, short ones a tile that still fills the
    machine; the 16-row fused shape gets the weight-streaming kernel's stage shape."""
    from autotune import native

    def tile(fam, m, n, k):
        d = native.default_cfg(fam, m, n, k)
        assert native.cfg_check(fam, d, m, n, k)[0] == native.OK
        return d["tile_m"], d["tile_n"], d["tile_k"], d["stages"], d["cluster_m"]

    assert tile("matmul_lhsT_rhs", 8192, 8192, 8192) == (512, 256, 64, 4, 2)
    assert tile("matmul_lhsT_rhs", 131072, 4096, 4096) == (512, 256, 64, 4, 2)
    assert tile("matmul_lhs_rhs", 4096, 11008, 4096) == (512, 256, 64, 4, 2)
    assert tile("matmul_lhsT_rhs", 2048, 2048, 2048) == (256, 256, 128, 3, 2)
    assert tile("matmul_lhsT_rhs", 256, 4096, 4096) == (128, 64, 128, 4, 1)         # 128 tiles for 148 SMs
    assert tile("matmul_lhsT_rhs", 1024, 8192, 8192) == (512, 256, 64, 4, 2)
    assert tile("rmsnorm_matmul", 16, 28672, 8192)[:1] == (16,)
    assert tile("rmsnorm_matmul", 4096, 11008, 4096) == (128, 256, 128, 2, 1)      # inline variant (no scratch)
    with pytest.raises(native.NativeError):
        native.default_cfg("nope", 1, 1, 1)


def test_cfg_check_families_and_scratch_sizes(native_lib):
    import ctypes as C

    from autotune import native

    lib = native.load()
    pair = dict(tile_m=256, tile_n=256, tile_k=128, stages=3, cluster_m=2)
    assert native.cfg_check("matmul_lhs_rhs", pair, 4096, 4096, 4096)[0] == native.OK
    assert native.cfg_check("matmul_lhs_rhs", dict(pair, tile_k=32), 4096, 4096, 4096)[0] == native.ERR_UNSUPPORTED
    assert native.cfg_check("matmul_lhs_rhs", pair, 4096, 4096, 4100)[0] == native.ERR_BAD_SHAPE
    # fused kernel: the skinny path only looks at tile_k / stages; larger M follows norm_mode
    assert native.cfg_check("rmsnorm_matmul", dict(tile_m=16, tile_n=256, tile_k=128, stages=3), 16, 28672, 8192)[0] == native.OK
    assert native.cfg_check("rmsnorm_matmul", dict(tile_m=16, tile_n=256, tile_k=128, stages=4), 16, 28672, 8192)[0] == native.ERR_SMEM_OOM
    assert native.cfg_check("rmsnorm_matmul", dict(pair, norm_mode=2), 4096, 11008, 4096)[0] == native.OK
    assert native.cfg_check("rmsnorm_matmul", dict(pair, norm_mode=1, stages=6), 4096, 11008, 4096)[0] == native.ERR_SMEM_OOM
    assert native.cfg_check("rmsnorm_matmul", dict(pair, norm_mode=2), 4096, 11008, 4100)[0] == native.ERR_BAD_SHAPE

    def ws(cfg, M, N, K):
        c = native.Cfg.from_dict(cfg)
        return lib.b200_workspace_bytes(b"rmsnorm_matmul", C.byref(c) if c is not None else None, M, N, K)

    assert ws(None, 16, 28672, 8192) >= 16 * 28672 * 4 + 112 * 4
    assert ws(dict(pair, norm_mode=1), 4096, 11008, 4096) == 0
    assert ws(dict(pair, norm_mode=2), 4096, 11008, 4096) >= 4096 * 4096 * 2 + 4096 * 4
    assert lib.b200_workspace_bytes(b"matmul_lhsT_rhs", None, 8192, 8192, 8192) == 0


def test_compile_one_reports_rejections(native_lib, tmp_path):
    from autotune.runner.compile import compile_one

    good = Candidate("matmul_lhsT_rhs", dict(tile_m=128, tile_n=128, tile_k=64, stages=3, cluster_m=1))
    bad = Candidate("matmul_lhsT_rhs", dict(tile_m=256, tile_n=256, tile_k=128, stages=6, cluster_m=1))
    shapes = {"lhs_T": (512, 256), "rhs": (512, 384)}
    for i, (cand, expect_err) in enumerate([(good, False), (bad, True)]):
        p = tmp_path / f"c_{i}.py"
        p.write_text(cand.to_source())
        cr = compile_one(f"c_{i}.py", str(p), "matmul_lhsT_rhs", shapes, "bfloat16", (256, 384), log_path=str(tmp_path / f"log{i}.txt"))
        assert bool(cr.error) == expect_err
        assert ("rejected" if expect_err else "accepted") in (tmp_path / f"log{i}.txt").read_text()
    p = tmp_path / "c_9.py"
    p.write_text(good.to_source())
    cr = compile_one("c_9.py", str(p), "matmul_lhsT_rhs", {"lhs_T": (512, 256), "rhs": (500, 384)}, "bfloat16", (256, 384))
    assert "do not match" in cr.error


def test_kernels_refuse_cpu_tensors(native_lib):
    import torch

    from autotune import kernels
    from autotune.native import NativeError

    a = torch.zeros(64, 64, dtype=torch.bfloat16)
    with pytest.raises(NativeError):
        kernels.matmul_lhsT_rhs(a, a)
    with pytest.raises(NativeError):
        kernels.rmsnorm_matmul(a, None, a)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from autotune import native

    monkeypatch.setattr(native, "_lib", None)
    monkeypatch.setenv("B200_AUTOTUNE_LIB", str(tmp_path / "absent.so"))
    with pytest.raises(native.NativeError, match="no CPU fallback"):
        native.load()


def test_generate_tensors_follows_reference_recipe():
    from autotune.runner.benchmark import generate_tensors

    specs = {"lhs_T": {"shape": [8, 4], "dtype": "float32"}, "rhs": {"shape": [8, 6], "dtype": "bfloat16"},
             "g": {"shape": [6], "dtype": "float32", "dist": {"kind": "uniform", "low": 0.5, "high": 1.5}}}
    got = generate_tensors(specs, 7)
    rng = np.random.default_rng(7)
    assert np.array_equal(got["lhs_T"], rng.standard_normal((8, 4)).astype(np.float32))
    assert np.array_equal(got["rhs"], rng.standard_normal((8, 6)).astype(resolve_dtype("bfloat16")))
    assert np.array_equal(got["g"], rng.uniform(0.5, 1.5, (6,)).astype(np.float32))


def test_host_pipeline_has_no_cpu_path_and_numa_lookup_is_harmless():
    """Without a GPU the host-buffer pipeline refuses to exist (there is no CPU fallback), and the
    NUMA helpers answer "unknown" instead of raising."""
    import torch

    from autotune import pipeline
    from autotune.native import NativeError

    if not torch.cuda.is_available():
        with pytest.raises(NativeError, match="no CPU path"):
            pipeline.HostPipeline(64, 64, 64)
        assert pipeline.bind_to_gpu_numa_node(0) == {"numa_node": None, "bound": False}


def test_cyclic_rows_cover_c_once():
    from autotune.sharded import cyclic_rows

    for M, world, chunks in [(131072, 8, 8), (4096, 2, 4), (192, 3, 1)]:
        pieces = sorted(p for r in range(world) for p in cyclic_rows(M, r, world, chunks))
        assert pieces[0][0] == 0 and pieces[-1][1] == M
        assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        assert len({b - a for a, b in pieces}) == 1 and (pieces[0][1] - pieces[0][0]) % 8 == 0
    with pytest.raises(ValueError):
        cyclic_rows(1000, 0, 3, 2)


def test_guard_bands_notice_a_stray_write():
    """The output of a candidate sits between two canary bands (host logic, CPU tensors)."""
    import torch

    from autotune.runner import benchmark as B

    backing, out = B.guarded_output(5, 7, torch.bfloat16, "cpu")
    assert out.shape == (5, 7) and out.dtype == torch.bfloat16
    assert out.data_ptr() - backing.data_ptr() == B.GUARD_BYTES and B.GUARD_BYTES % 256 == 0
    out.fill_(3.0)
    assert B.guards_intact(backing)
    backing[B.GUARD_BYTES + 5 * 7 * 2] = 0           # first byte after the output
    assert not B.guards_intact(backing)
    backing[B.GUARD_BYTES + 5 * 7 * 2] = B.GUARD_PATTERN
    backing[B.GUARD_BYTES - 1] = 0                   # last byte before it
    assert not B.guards_intact(backing)


def test_peer_store_refuses_bad_arguments_before_touching_a_device(native_lib):
    """Argument checks of the exchange kernel's entry point need no GPU: nothing to do is fine, a
    missing table, too many peers or a misaligned source or size is a bad argument."""
    import ctypes as C

    from autotune import native

    table = (C.c_void_p * 9)(*[0x1000 * (i + 1) for i in range(9)])
    assert native_lib.b200_peer_store(None, None, 0, 0, 0, None) == native.OK
    assert native_lib.b200_peer_store(0x1000, table, 0, 4096, 0, None) == native.OK
    assert native_lib.b200_peer_store(0x1000, None, 2, 4096, 0, None) == native.ERR_BAD_ARG
    assert native_lib.b200_peer_store(0x1000, table, 9, 4096, 0, None) == native.ERR_BAD_ARG
    assert native_lib.b200_peer_store(0x1008, table, 2, 4096, 0, None) == native.ERR_BAD_ARG
    assert native_lib.b200_peer_store(0x1000, table, 2, 4100, 0, None) == native.ERR_BAD_ARG
    assert "16" in native.last_error()
    base = C.c_void_p()
    assert native_lib.b200_ipc_open(None, C.byref(base)) == native.ERR_BAD_ARG
    assert native_lib.b200_ipc_close(None) == native.OK


def test_header_is_plain_c_and_links_against_the_library(native_lib, tmp_path):
    """The boundary is a C ABI: the header compiles as C99 with warnings as errors, and a C program
    that calls into the library links and runs (no compute: version, a budget check, an error text)."""
    import shutil
    import subprocess

    from autotune import native

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use_header.c"
    src.write_text(
        '#include <stdio.h>\n#include <string.h>\n#include "b200_autotune.h"\n'
        "int main(void) {\n"
        "  b200_cfg c; long smem = 0; int tmem = 0; memset(&c, 0, sizeof c);\n"
        "  c.tile_m = 128; c.tile_n = 256; c.tile_k = 64; c.stages = 5; c.cluster_m = 1; c.cluster_n = 1;\n"
        '  int rc = b200_cfg_check("matmul_lhsT_rhs", &c, 8192, 8192, 8192, &smem, &tmem);\n'
        '  printf("%d %d %ld %d %s\\n", b200_abi_version(), rc, smem, tmem, b200_last_error());\n'
        "  return 0;\n}\n")
    exe = tmp_path / "use_header"
    lib_dir = str(native.LIB_PATH.parent)
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(REPO / "include"), str(src),
                    "-L", lib_dir, "-lb200_autotune", f"-Wl,-rpath,{lib_dir}", "-o", str(exe)], check=True, capture_output=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split(None, 4)
    assert out[0] == "1" and int(out[1]) == native.ERR_SMEM_OOM and int(out[2]) > 232448 and "Out of memory in smem" in out[4]


def test_cuda_ipc_handle_is_taken_out_of_what_torch_exports():
    from autotune.sharded import cuda_ipc_handle

    raw = bytes(range(64))
    assert cuda_ipc_handle(raw) == raw
    assert cuda_ipc_handle(b"c" + raw) == raw
    assert cuda_ipc_handle(b"\x01c" + raw) == raw
    for bad in (b"\x01e" + raw, b"e" + raw, raw[:63], b"\x01\x01c" + raw):
        with pytest.raises(RuntimeError, match="not a CUDA IPC handle"):
            cuda_ipc_handle(bad)


def test_planner_answers_every_candidate_with_a_status_and_consistent_budgets(native_lib):
    """Every point of a wide grid of meta-parameters, sensible or not, gets one of the declared status
    codes; an accepted point fits the budgets it reports, and its launch description parses."""
    import itertools

    from autotune import native

    known = {native.OK, native.ERR_BAD_SHAPE, native.ERR_UNSUPPORTED, native.ERR_SMEM_OOM, native.ERR_TMEM_OOM}
    shapes = [(8192, 8192, 8192), (4096, 11008, 4096), (16, 28672, 8192), (136, 72, 64), (8, 8, 64)]
    accepted = 0
    for fam in ("matmul_lhsT_rhs", "matmul_lhs_rhs", "rmsnorm_matmul"):
        for tm, tn, tk, st, cm, nm, sk in itertools.product((16, 64, 128, 256, 512), (32, 64, 128, 256, 512), (32, 64, 96, 128),
                                                            (1, 3, 6, 13), (1, 2), (0, 1, 2), (0, 4)):
            cfg = dict(tile_m=tm, tile_n=tn, tile_k=tk, stages=st, cluster_m=cm, norm_mode=nm, split_k=sk)
            M, N, K = shapes[(tm + tn + tk + st + cm + nm + sk) % len(shapes)]
            if fam == "rmsnorm_matmul" and M > 16 and nm == 0:
                cfg["norm_mode"] = 2   # as compile_one resolves it: the sweep always supplies scratch
            status, msg, smem, tmem = native.cfg_check(fam, cfg, M, N, K)
            assert status in known, (fam, cfg, status, msg)
            assert (status == native.OK) == (msg == "")
            if status == native.OK:
                accepted += 1
                assert 0 < smem <= 232448 and tmem in (32, 64, 128, 256, 512), (fam, cfg, smem, tmem)
                plan = native.describe_launch(fam, cfg, M, N, K)
                assert 1 <= plan["grid"] <= 160 and plan["threads"] % 32 == 0 and plan["threads"] > 0
                assert plan["smem_bytes"] <= 232448
    assert accepted > 100
