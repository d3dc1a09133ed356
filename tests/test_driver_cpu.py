"""Sweep sharding and failure containment on CPU: the worker pool with host-injected failures,
and the per-rank sharding + host gather used under torchrun (gloo, world size 2)."""

import os
import subprocess
import sys
import textwrap

import pytest

from autotune.runner.driver import run_sharded, shard_round_robin

import fake_workers

from conftest import PKG, REPO


def _items(n, **inject):
    return [{"kernel_name": f"k_{i}.py", "i": i, "inject": inject.get(f"k_{i}.py")} for i in range(n)]


def test_round_robin_is_deterministic():
    shards = shard_round_robin(list(range(10)), 4)
    assert shards == [[0, 4, 8], [1, 5, 9], [2, 6], [3, 7]]
    assert shard_round_robin([], 3) == [[], [], []]
    assert shard_round_robin([1, 2], 1) == [[1, 2]]


def test_pool_gathers_all_results_and_pins_devices():
    items = _items(7)
    shards = shard_round_robin(items, 3)
    res = run_sharded(shards, fake_workers.well_behaved, {}, ["0", "1", "2"], deadline_s=30, startup_s=60)
    assert sorted(r.kernel_name for r in res) == sorted(i["kernel_name"] for i in items)
    env_of = {r.kernel_name: r.profiler_summary["device_env"] for r in res}
    assert env_of["k_0.py"] == "0" and env_of["k_1.py"] == "1" and env_of["k_5.py"] == "2" and env_of["k_3.py"] == "0"


def test_inputs_are_generated_once_and_reach_workers_through_shared_memory():
    """The parent publishes one set of tensors per batch; workers in other processes map them and
    see the same values (bf16 included); after close() the blocks are gone."""
    import ml_dtypes
    import numpy as np
    from multiprocessing import shared_memory

    from autotune.runner.benchmark import generate_tensors
    from autotune.runner.driver import SharedInputs

    specs = {"lhs_T": {"shape": [64, 48], "dtype": "bfloat16", "dist": {"kind": "normal", "scale": 0.125}},
             "rhs": {"shape": [64, 40], "dtype": "float32"}}
    tensors = generate_tensors(specs, 5)
    assert tensors["lhs_T"].dtype == ml_dtypes.bfloat16
    shared = SharedInputs()
    try:
        desc = shared.publish(tensors)
        items = [{"kernel_name": f"k_{i}.py", "batch": "b0"} for i in range(4)]
        res = run_sharded(shard_round_robin(items, 2), fake_workers.reads_shared_inputs, {"shared_inputs": {"b0": desc}},
                          [None, None], deadline_s=30, startup_s=60)
        assert len(res) == 4
        for r in res:
            assert r.profiler_summary["shapes"] == {"lhs_T": [64, 48], "rhs": [64, 40]}
            for name, arr in tensors.items():
                assert r.profiler_summary["sums"][name] == float(arr.astype(np.float64).sum())
        names = [d["shm"] for d in desc.values()]
    finally:
        shared.close()
    for n in names:
        with pytest.raises(FileNotFoundError):
            shared_memory.SharedMemory(name=n)


def test_top_k_is_timed_again_on_one_device():
    from autotune.runner.driver import retime_top_k

    items = _items(6)
    first = run_sharded(shard_round_robin(items, 3), fake_workers.well_behaved, {}, ["0", "1", "2"], deadline_s=30, startup_s=60)
    # candidate k_i "takes" (1 + i) ms in the fake worker; the three fastest are k_0, k_1, k_2
    out = retime_top_k(first, items, 3, {}, "5", 30, worker=fake_workers.well_behaved, startup_s=60)
    assert sorted(r.kernel_name for r in out) == sorted(r.kernel_name for r in first)
    by = {r.kernel_name: r.profiler_summary for r in out}
    for name in ("k_0.py", "k_1.py", "k_2.py"):
        assert by[name]["retimed_on_one_gpu"] and by[name]["device_env"] == "5"
        assert by[name]["first_pass_total_time"] == by[name]["total_time"]          # the fake is deterministic
    for name in ("k_3.py", "k_4.py", "k_5.py"):
        assert "retimed_on_one_gpu" not in by[name] and by[name]["device_env"] in ("0", "1", "2")
    assert retime_top_k(first, items, 0, {}, "5", 30, worker=fake_workers.well_behaved) == first


@pytest.mark.parametrize("kind,needle", [("raise", "injected failure"), ("exit", "died"), ("hang", "deadline")])
def test_one_bad_candidate_costs_one_row(kind, needle):
    items = _items(6, **{"k_2.py": kind})
    shards = shard_round_robin(items, 2)  # k_2 is the second item of worker 0
    res = run_sharded(shards, fake_workers.faulty, {}, [None, None], deadline_s=2.0, startup_s=20.0)
    by_name = {r.kernel_name: r for r in res}
    assert set(by_name) == {i["kernel_name"] for i in items}
    bad = by_name["k_2.py"]
    assert bad.profiler_summary is None and needle in bad.hardware_output
    ok = [n for n, r in by_name.items() if r.profiler_summary is not None]
    assert sorted(ok) == ["k_0.py", "k_1.py", "k_3.py", "k_4.py", "k_5.py"]  # k_4 ran in a fresh worker


def test_pipeline_rejects_mixed_lnc():
    from autotune.runner.driver import run_pipeline
    from autotune.runner.types import KernelJob

    jobs = {"a_0.py": KernelJob("x", "matmul_lhsT_rhs", (8, 8), {"a": ((8, 8), "bfloat16")}, lnc=1),
            "a_1.py": KernelJob("x", "matmul_lhsT_rhs", (8, 8), {"a": ((8, 8), "bfloat16")}, lnc=2)}
    with pytest.raises(RuntimeError, match="mixes lnc"):
        run_pipeline(jobs, 0, False, False)


def test_no_gpu_is_a_batch_level_error(native_lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from autotune.runner.api import profile
    from autotune.runner.candidate import enumerate_grid, jobs_from_candidates

    jobs = jobs_from_candidates(enumerate_grid("matmul_lhsT_rhs")[:1], (128, 128),
                                {"lhs_T": ((64, 128), "bfloat16"), "rhs": ((64, 128), "bfloat16")})
    with pytest.raises(RuntimeError):
        profile(jobs, "", 0, "b200", False)


RANK_SCRIPT = textwrap.dedent(
    """
    import sys, json
    sys.path.insert(0, {pkg!r}); sys.path.insert(0, {repo!r})
    import bench
    r = bench.Ranks()
    mine = list(range(10))[r.rank::r.world]          # candidate i -> rank i mod world
    mx = r.max(float(r.rank + 1))
    parts = r.gather([(i, r.rank) for i in mine])
    r.barrier()
    if r.rank == 0:
        flat = sorted(x for p in parts for x in p)
        print(json.dumps({{"max": mx, "flat": flat}}))
    r.close()
    """
)


def test_rank_sharding_and_host_gather_gloo_world2(tmp_path):
    script = tmp_path / "rank_script.py"
    script.write_text(RANK_SCRIPT.format(pkg=str(PKG), repo=str(REPO)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29631", str(script)]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stderr[-2000:]
    import json

    line = [l for l in proc.stdout.splitlines() if l.startswith("{")][-1]
    data = json.loads(line)
    assert data["max"] == 2.0
    assert data["flat"] == [[i, i % 2] for i in range(10)]


def test_reference_arm_non_zero_rank_exits_quietly(tmp_path):
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    proc = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--gpus", "2"],
                          capture_output=True, text=True, timeout=120, env=env)
    assert proc.returncode == 0 and proc.stdout.strip() == ""


def test_row_range_covers_m_once_and_keeps_alignment():
    from autotune.sharded import row_range

    for M, world in [(131072, 8), (1000, 3), (8, 4), (0, 2), (4099, 5)]:
        bounds = [row_range(M, r, world) for r in range(world)]
        assert bounds[0][0] == 0 and bounds[-1][1] == M
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
        assert all(b0 % 8 == 0 for b0, _ in bounds)
    assert row_range(131072, 3, 8) == (49152, 65536)
    with pytest.raises(ValueError):
        row_range(10, 2, 2)


ROW_SPLIT_SCRIPT = textwrap.dedent(
    """
    import sys, json
    sys.path.insert(0, {pkg!r})
    import torch, torch.distributed as dist
    from autotune.sharded import row_range, replicate, matmul_lhsT_rhs_row_split

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()

    def host_matmul(a, b, cfg=None, out=None):   # stand-in for the GPU kernel: the test is about the sharding
        out.copy_(a.T @ b)
        return out

    result = {{}}
    for M in (64, 1000):                          # equal blocks (in-place gather) and ragged blocks
        K, N = 24, 16
        g = torch.Generator().manual_seed(5)
        lhs_T = torch.randn(K, M, generator=g)
        rhs_src = torch.randn(K, N, generator=g)
        rhs = replicate(rhs_src if rank == 0 else None, (K, N), torch.float32, "cpu", src=0)
        m0, m1 = row_range(M, rank, world)
        block, full = matmul_lhsT_rhs_row_split(lhs_T[:, m0:m1], rhs, M, matmul=host_matmul)
        want = lhs_T.T @ rhs_src
        result[str(M)] = [bool(torch.equal(rhs, rhs_src)), bool(torch.allclose(block, want[m0:m1])),
                          bool(torch.allclose(full, want)), list(full.shape)]
        only, none = matmul_lhsT_rhs_row_split(lhs_T[:, m0:m1], rhs, M, matmul=host_matmul, gather=False)
        assert none is None and torch.allclose(only, want[m0:m1])
    # block-cyclic split: band i of C is gathered while band i+1 is multiplied
    from autotune.sharded import cyclic_rows
    M, K, N, chunks = 48 * world, 24, 16, 2
    g = torch.Generator().manual_seed(6)
    lhs_T = torch.randn(K, M, generator=g)
    rhs = torch.randn(K, N, generator=g)
    pieces = cyclic_rows(M, rank, world, chunks)
    mine = torch.cat([lhs_T[:, p0:p1] for p0, p1 in pieces], dim=1)
    none, full = matmul_lhsT_rhs_row_split(mine, rhs, M, matmul=host_matmul, chunks=chunks)
    result["cyclic"] = [none is None, bool(torch.allclose(full, lhs_T.T @ rhs)), list(full.shape) == [M, N],
                        sorted(p for r in range(world) for p in cyclic_rows(M, r, world, chunks)) ==
                        [(i * M // (world * chunks), (i + 1) * M // (world * chunks)) for i in range(world * chunks)]]
    oks = [None] * world
    dist.all_gather_object(oks, result)
    if rank == 0:
        print(json.dumps(oks))
    dist.destroy_process_group()
    """
)


@pytest.mark.parametrize("world,port", [(2, 29641), (3, 29643)])
def test_row_split_replicates_and_gathers_gloo(tmp_path, world, port):
    script = tmp_path / "row_split.py"
    script.write_text(ROW_SPLIT_SCRIPT.format(pkg=str(PKG)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert proc.returncode == 0, proc.stderr[-2000:]
    import json

    per_rank = json.loads([l for l in proc.stdout.splitlines() if l.startswith("[")][-1])
    assert len(per_rank) == world
    for res in per_rank:
        assert res["64"][:3] == [True, True, True] and res["64"][3] == [64, 16]
        assert res["1000"][:3] == [True, True, True] and res["1000"][3] == [1000, 16]
        assert res["cyclic"] == [True, True, True, True]


def test_resident_workers_serve_the_next_sweep_and_failed_ones_are_replaced():
    """keep_workers: the second call is served by the processes of the first (same PIDs, still pinned
    to their devices); a worker that crashes or hangs is replaced, never parked; shutdown ends them."""
    from autotune.runner import driver

    driver.shutdown_workers()
    items = [{"kernel_name": f"k_{i}.py", "i": i} for i in range(6)]
    shards = shard_round_robin(items, 2)
    try:
        first = run_sharded(shards, fake_workers.well_behaved, {}, ["0", "1"], deadline_s=30, startup_s=60, keep_workers=True)
        pids_1 = {r.profiler_summary["device_env"]: r.profiler_summary["pid"] for r in first}
        assert driver.resident_worker_pids() == pids_1 and len(pids_1) == 2
        second = run_sharded(shards, fake_workers.well_behaved, {}, ["0", "1"], deadline_s=30, startup_s=60, keep_workers=True)
        assert {r.profiler_summary["device_env"]: r.profiler_summary["pid"] for r in second} == pids_1
        assert sorted(r.kernel_name for r in second) == sorted(it["kernel_name"] for it in items)
        # a job that crashes on device "0" and hangs on device "1": both workers are replaced, the
        # remaining candidates of each shard still get their rows, and only healthy workers are parked
        bad = [dict(items[0], inject="raise"), dict(items[1], inject="hang")] + items[2:]
        third = run_sharded(shard_round_robin(bad, 2), fake_workers.faulty, {}, ["0", "1"], deadline_s=2.0, startup_s=20.0,
                            keep_workers=True)
        by_name = {r.kernel_name: r for r in third}
        assert "injected failure" in by_name["k_0.py"].hardware_output and "deadline" in by_name["k_1.py"].hardware_output
        assert all(by_name[f"k_{i}.py"].profiler_summary is not None for i in range(2, 6))
        pids_3 = driver.resident_worker_pids()
        assert set(pids_3) == {"0", "1"} and not (set(pids_3.values()) & set(pids_1.values()))
        # without keep_workers nothing is parked or taken from the pool
        fourth = run_sharded(shards, fake_workers.well_behaved, {}, ["0", "1"], deadline_s=30, startup_s=60)
        assert not ({r.profiler_summary["pid"] for r in fourth} & set(pids_3.values()))
        assert driver.resident_worker_pids() == pids_3
    finally:
        driver.shutdown_workers()
    assert driver.resident_worker_pids() == {}
    for pid in list(pids_1.values()) + list(pids_3.values()):
        with pytest.raises(OSError):
            os.kill(pid, 0)          # gone (signal 0 only probes)
