"""Large-M row split over two GPUs: NCCL replication of rhs, local tcgen05 GEMMs, device all-gather
(and the library's own peer-store exchange); every rank compares its own block and its gathered
copy of C with the CPU oracle.

Needs two GPUs; skipped on a one-GPU box.  The ranks run as child processes under torchrun."""

import json
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import PKG

pytestmark = pytest.mark.gpu

SCRIPT = textwrap.dedent(
    """
    import sys, json, os
    sys.path.insert(0, {pkg!r}); sys.path.insert(0, {repo!r})
    import ml_dtypes, numpy as np
    import torch, torch.distributed as dist
    from autotune import kernels
    from autotune.sharded import row_range, replicate, matmul_lhsT_rhs_row_split
    from oracle import oracle as O

    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    res = {{}}
    for M, K, N in ((4096, 512, 384), (1000, 264, 136)):   # equal blocks, ragged blocks
        # same seed on every rank: every rank can build the answer with the CPU oracle
        s = {{"kind": "normal", "scale": K ** -0.5}}
        t = O.generate_inputs(11, [("lhs_T", (K, M), s), ("rhs", (K, N), s)], bf16=True)
        want = O.matmul_lhsT_rhs(t["lhs_T"], t["rhs"])
        lhs_T = kernels.to_device(t["lhs_T"].astype(ml_dtypes.bfloat16))
        rhs_src = kernels.to_device(t["rhs"].astype(ml_dtypes.bfloat16))
        rhs = replicate(rhs_src if rank == 0 else None, (K, N), torch.bfloat16, "cuda", src=0)
        m0, m1 = row_range(M, rank, world)
        block, full = matmul_lhsT_rhs_row_split(lhs_T[:, m0:m1], rhs, M)
        torch.cuda.synchronize()
        err = O.max_abs_rel_err(kernels.to_host(full).astype(np.float32), want)
        err_block = O.max_abs_rel_err(kernels.to_host(block).astype(np.float32), want[m0:m1])
        res[str(M)] = [bool(torch.equal(rhs, rhs_src)), max(err, err_block), list(full.shape)]
        if M % (8 * world * 4) == 0:
            # the same products with the library's own exchange: rows pushed into every peer's copy of
            # C over NVLink (CUDA IPC mappings, plain stores), one block per rank and block-cyclic
            from autotune.sharded import PeerCopies, cyclic_rows
            peers = PeerCopies(M, N)
            errs = []
            for chunks in (1, 4):
                peers.local.zero_()
                torch.cuda.synchronize(); dist.barrier()
                spans = [row_range(M, rank, world)] if chunks == 1 else cyclic_rows(M, rank, world, chunks)
                cols = torch.cat([lhs_T[:, a:b] for a, b in spans], dim=1).contiguous()
                for _ in range(2):   # twice: the second run overwrites what the first pushed
                    _, c_all = matmul_lhsT_rhs_row_split(cols, rhs, M, chunks=chunks, peers=peers)
                torch.cuda.synchronize()
                errs.append(O.max_abs_rel_err(kernels.to_host(c_all).astype(np.float32), want))
                dist.barrier()
            res["peers"] = errs
            peers.close()
    out = [None] * world
    dist.all_gather_object(out, res)
    if rank == 0:
        print(json.dumps(out))
    dist.destroy_process_group()
    """
)


def test_row_split_two_gpus_nccl(native_lib, tmp_path):
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "row_split_gpu.py"
    script.write_text(SCRIPT.format(pkg=str(PKG), repo=str(PKG.parent)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29671", str(script)]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ))
    assert proc.returncode == 0, proc.stderr[-3000:]
    per_rank = json.loads([l for l in proc.stdout.splitlines() if l.startswith("[")][-1])
    assert len(per_rank) == 2
    for r in per_rank:
        for key, shape in (("4096", [4096, 384]), ("1000", [1000, 136])):
            same_rhs, err, got_shape = r[key]
            assert same_rhs and err <= 1e-2 and got_shape == shape
        assert len(r["peers"]) == 2 and max(r["peers"]) <= 1e-2, r["peers"]
