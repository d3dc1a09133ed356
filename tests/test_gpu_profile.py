"""profile() end to end on the GPU: validation, timing, parity gate, cache layout (GPU box only)."""

import json

import pytest

pytestmark = pytest.mark.gpu


def _mm_jobs(n, cands):
    from autotune.runner.candidate import jobs_from_candidates

    d = {"kind": "normal", "scale": n ** -0.5}
    return jobs_from_candidates(cands, (n, n), {"lhs_T": ((n, n), "bfloat16", d), "rhs": ((n, n), "bfloat16", d)})


def test_profile_sweep_writes_reference_cache_layout(native_lib, tmp_path):
    from autotune.runner.api import profile
    from autotune.runner.candidate import enumerate_grid

    cands = enumerate_grid("matmul_lhsT_rhs", stages=(3, 6))            # 32 points, some over budget
    out = profile(_mm_jobs(1024, cands), str(tmp_path), 1, "b200", True, warmup=1, iters=3)
    assert len(out.results) == 32
    assert out.successes and out.failures
    assert all("Out of memory in smem" in f.hardware_output for f in out.failures), [f.hardware_output[:80] for f in out.failures]
    for s in out.successes:
        assert s.total_time_s > 0 and 0 < s.mfu <= 100
    data = json.loads((tmp_path / "results.json").read_text())
    assert data["metadata"]["num_kernels"] == 32
    assert data["metrics"]["success"] == len(out.successes)
    assert data["metrics"]["smem_oom"] == len(out.failures) and data["metrics"]["sbuf_oom"] == 0
    names = [k["kernel_name"] for k in data["kernels"]]
    assert names == [f"matmul_lhsT_rhs_{i}.py" for i in range(32)]      # numeric order
    ok = out.successes[0].kernel_name[:-3]
    assert (tmp_path / ok / f"{ok}.py").exists() and (tmp_path / ok / "log-neuron-cc.txt").exists()
    summary = json.loads((tmp_path / ok / "profile_summary.json").read_text())
    assert summary["max_abs_rel_err"] <= 1e-2 and summary["total_time"] > 0
    assert summary["repeat_bit_identical"] and summary["guard_bands_intact"]
    detail = json.loads((tmp_path / ok / "profile.json").read_text())    # detailed run: plan + kernel's own cycle count
    assert detail["plan"]["kernel"].startswith("gemm_tcgen05_kernel") and detail["plan"]["registers"] > 0
    assert detail["cta_lifetime_sm_cycles"] > 0 and 0 < detail["tensor_pipe_busy_estimate"] <= 1.0
    assert len(detail["launches_ms"]) == 3
    neff = (tmp_path / ok / "file.neff").read_bytes()                    # descriptor + raw b200_cfg
    assert neff.startswith(b"B200CAND") and b"FAMILY = 'matmul_lhsT_rhs'" in neff
    ntff = (tmp_path / ok / "profile.ntff").read_bytes()                 # per-launch time series
    assert ntff.startswith(b"B200TIME") and len(ntff) == 12 + 4 * 3
    meta = data["metadata"]
    assert list(meta)[:2] == ["num_kernels", "wallclock_s"] and "B200" in meta["gpu_name"] and meta["seed"] == 1
    assert meta["peaks"]["bf16_tflops"] > 0 and meta["tolerance"]["bf16_max_abs_rel_err"] == 1e-2 and meta["n_gpus"] >= 1
    text = str(out)
    assert "Succeeded:" in text and "failures:" in text


def test_profile_fp32_config_and_rmsnorm(native_lib):
    from autotune.runner.api import profile
    from autotune.runner.candidate import Candidate, jobs_from_candidates

    # configs[0]: 512^3 fp32, 4 tile candidates; they run on the CUDA-core kernel and agree to 1e-5
    cands = [Candidate("matmul_lhsT_rhs", dict(tile_m=tm, tile_n=tn, tile_k=128, stages=2)) for tm in (128, 256) for tn in (128, 512)]
    jobs = jobs_from_candidates(cands, (512, 512), {"lhs_T": ((512, 512), "float32"), "rhs": ((512, 512), "float32")})
    out = profile(jobs, "", 0, "b200", False, warmup=1, iters=3)
    assert len(out.successes) == 4 and not out.failures
    # fused kernel, both norm placements, plus the skinny shape
    specs = lambda m, k, n: {"x": ((m, k), "bfloat16"), "gamma": ((k,), "bfloat16", {"kind": "uniform", "low": 0.5, "high": 1.5}),  # noqa: E731
                             "weight": ((k, n), "bfloat16", {"kind": "normal", "scale": k ** -0.5})}
    cands = [Candidate("rmsnorm_matmul", dict(tile_m=128, tile_n=128, tile_k=64, stages=3, norm_mode=nm), {"eps": 1e-6}) for nm in (1, 2)]
    out = profile(jobs_from_candidates(cands, (512, 768), specs(512, 1024, 768)), "", 2, "b200", False, warmup=1, iters=3)
    assert len(out.successes) == 2, [f.hardware_output[-300:] for f in out.failures]
    cands = [Candidate("rmsnorm_matmul", dict(tile_m=16, tile_n=256, tile_k=64, stages=4), {"eps": 1e-5})]
    out = profile(jobs_from_candidates(cands, (16, 2048), specs(16, 1024, 2048)), "", 3, "b200", False, warmup=1, iters=3)
    assert len(out.successes) == 1, [f.hardware_output[-300:] for f in out.failures]


def test_profile_matmul_lhs_rhs_family(native_lib):
    from autotune.runner.api import profile
    from autotune.runner.candidate import Candidate, jobs_from_candidates

    d = {"kind": "normal", "scale": 512 ** -0.5}
    cands = [Candidate("matmul_lhs_rhs", dict(tile_m=tm, tile_n=256, tile_k=64, stages=3, cluster_m=cm)) for tm, cm in ((128, 1), (256, 2))]
    out = profile(jobs_from_candidates(cands, (768, 512), {"lhs": ((768, 512), "bfloat16", d), "rhs": ((512, 512), "bfloat16", d)}),
                  "", 5, "b200", False, warmup=1, iters=3)
    assert len(out.successes) == 2, [f.hardware_output[-300:] for f in out.failures]


def test_vendor_baseline_row(native_lib, tmp_path):
    from autotune.runner.baseline import profile_numpy_baseline

    res, how = profile_numpy_baseline(lambda a, b: a.T @ b, {"lhs_T": ((512, 256), "bfloat16"), "rhs": ((512, 384), "bfloat16")},
                                      str(tmp_path / "compiler_baseline"), kernel_name="compiler_baseline", flops=2.0 * 256 * 384 * 512)
    assert res.hardware_output.startswith("[256, 384]") and res.profiler_summary["total_time"] > 0 and "torch" in how


def test_bad_candidate_is_a_failure_row_not_an_exception(native_lib):
    from autotune.runner.api import profile
    from autotune.runner.types import KernelJob

    jobs = {"broken_0.py": KernelJob("FAMILY = 'matmul_lhsT_rhs'\nCONFIG = {'tile_m': 100}\n", "matmul_lhsT_rhs", (256, 256),
                                     {"lhs_T": ((256, 256), "bfloat16"), "rhs": ((256, 256), "bfloat16")}),
            "garbage_1.py": KernelJob("this is not python (", "matmul_lhsT_rhs", (256, 256),
                                      {"lhs_T": ((256, 256), "bfloat16"), "rhs": ((256, 256), "bfloat16")})}
    out = profile(jobs, "", 0, "b200", False)
    assert len(out.failures) == 2 and not out.successes


def test_candidate_whose_wait_runs_out_does_not_poison_the_next_one(native_lib):
    """A candidate that ends with a device-side wait expiry leaves its scratch (row counters of the
    fused kernel's norm pass) undefined.  The sweep must drop that scratch: the next candidate of
    the same batch gets a fresh, zeroed buffer, succeeds, and leaves its counters at zero."""
    import torch

    from autotune import kernels
    from autotune.runner.api import profile
    from autotune.runner.candidate import Candidate, jobs_from_candidates

    m, k, n = 512, 1024, 768
    specs = {"x": ((m, k), "bfloat16"), "gamma": ((k,), "bfloat16", {"kind": "uniform", "low": 0.5, "high": 1.5}),
             "weight": ((k, n), "bfloat16", {"kind": "normal", "scale": k ** -0.5})}
    base = dict(tile_m=128, tile_n=128, tile_k=64, stages=3, norm_mode=2)
    cands = [Candidate("rmsnorm_matmul", dict(base, _debug_skip_producer=1, _wait_limit_us=2000), {"eps": 1e-6}),
             Candidate("rmsnorm_matmul", dict(base), {"eps": 1e-6})]
    kernels.reset_workspaces()
    out = profile(jobs_from_candidates(cands, (m, n), specs), "", 7, "b200", False, warmup=1, iters=3, n_gpus=1)
    assert len(out.failures) == 1 and "wait expired" in out.failures[0].hardware_output
    assert len(out.successes) == 1 and out.successes[0].kernel_name.endswith("_1.py")
    torch.cuda.synchronize()
    bufs = [b for key, b in kernels._WORKSPACES.items() if key[1] == "prologue"]
    assert len(bufs) == 1
    counters = bufs[0][-256:]  # next row to claim, departed CTAs, rows ready per 128-row block
    assert int((counters != 0).sum()) == 0


def test_resident_worker_serves_two_sweeps_on_the_gpu(native_lib):
    """keep_workers: the sweep runs in a worker process (also on one GPU); the process, with its CUDA
    context, serves the next profile() call, which therefore starts faster, and both give the same
    rows; shutdown_workers() ends it."""
    import time

    from autotune.runner import driver
    from autotune.runner.api import profile
    from autotune.runner.candidate import enumerate_grid, jobs_from_candidates

    driver.shutdown_workers()
    k = m = n = 1024
    s = {"kind": "normal", "scale": k ** -0.5}
    cands = enumerate_grid("matmul_lhsT_rhs", tile_m=(128, 256), tile_n=(128, 256), tile_k=(64,), stages=(3,), cluster_m=(1,))
    jobs = jobs_from_candidates(cands, (m, n), {"lhs_T": ((k, m), "bfloat16", s), "rhs": ((k, n), "bfloat16", s)})
    try:
        t0 = time.monotonic()
        first = profile(jobs, "", 3, "b200", False, warmup=2, iters=5, n_gpus=1, keep_workers=True)
        t1 = time.monotonic()
        pids = driver.resident_worker_pids()
        assert len(pids) == 1 and len(first.successes) == len(jobs) and not first.failures
        second = profile(jobs, "", 3, "b200", False, warmup=2, iters=5, n_gpus=1, keep_workers=True)
        t2 = time.monotonic()
        assert driver.resident_worker_pids() == pids
        assert [r.kernel_name for r in second.successes] == [r.kernel_name for r in first.successes]
        assert (t2 - t1) < (t1 - t0), (t1 - t0, t2 - t1)   # no process start, no CUDA context, no module load
    finally:
        driver.shutdown_workers()
    assert driver.resident_worker_pids() == {}
