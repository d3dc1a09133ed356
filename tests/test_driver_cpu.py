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
