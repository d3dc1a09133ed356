"""The large-M product split by rows of C over the GPUs of one box.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        examples/row_split_large_m.py [--rows 131072] [--overlap] [--peer-stores]

C[M, 4096] = lhsT[4096, M]^T . rhs[4096, 4096] with M = 131072 (seed 4, N(0,1)/sqrt(K), bf16): rank r
multiplies its share of the columns of lhsT by the whole of rhs.  rhs is uploaded by rank 0 only and
replicated over NVLink; C is all-gathered on the device into every GPU's memory (``--overlap``: the
block-cyclic split, where the all-gather of one band runs beside the GEMM of the next;
``--peer-stores``: the same split with the library's own exchange, a kernel that stores each band's
rows into the other GPUs' copies of C over NVLink, in place of the collective).  Rank 0
then gathers nothing more: every rank checks rows of ITS copy of C against a host product of the same
inputs (fp32 BLAS on the bf16-rounded values) and the ranks' results are
collected on the host.  The reference has no multi-device path (its benchmark loop is one device:
``autotune/src/autotune/runner/driver.py:97``).
"""

import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "nki-autotune_b200"))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from autotune import kernels, sharded  # noqa: E402
from autotune.runner.benchmark import generate_tensors  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    # (not "--m": the launcher's own parser takes that for an abbreviation of its options)
    ap.add_argument("--rows", dest="m", type=int, default=131072, help="M, the rows of C")
    ap.add_argument("--overlap", action="store_true")
    ap.add_argument("--chunks", type=int, default=0, help="bands of the block-cyclic split (default: 8 with --overlap, 4 with --peer-stores)")
    ap.add_argument("--peer-stores", action="store_true")
    args = ap.parse_args()

    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    K, N, M = 4096, 4096, args.m
    d = {"kind": "normal", "scale": K ** -0.5}
    # every rank draws the same seeded tensors (the recipe of the benchmark configuration) and keeps its share
    t = generate_tensors({"lhs_T": {"shape": [K, M], "dtype": "bfloat16", "dist": d},
                          "rhs": {"shape": [K, N], "dtype": "bfloat16", "dist": d}}, seed=4)
    chunks = (args.chunks or (4 if args.peer_stores else 8)) if (args.overlap or args.peer_stores) else 1
    if chunks > 1:
        pieces = sharded.cyclic_rows(M, rank, world, chunks)
    else:
        pieces = [sharded.row_range(M, rank, world)]
    mine = np.concatenate([t["lhs_T"][:, p0:p1] for p0, p1 in pieces], axis=1)
    lhs_T_block = kernels.to_device(mine)
    rhs = sharded.replicate(kernels.to_device(t["rhs"]) if rank == 0 else None, (K, N), torch.bfloat16, "cuda", src=0)
    peers = sharded.PeerCopies(M, N) if args.peer_stores else None
    full = peers.local if peers is not None else torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    run = lambda: sharded.matmul_lhsT_rhs_row_split(lhs_T_block, rhs, M, out_full=full, chunks=chunks, peers=peers)  # noqa: E731
    for _ in range(2):
        run()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / 5], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    rows = np.arange(7, M, M // 64)[:64]
    expect = t["lhs_T"][:, rows].astype(np.float32).T @ t["rhs"].astype(np.float32)
    got = kernels.to_host(full[torch.from_numpy(rows).cuda()]).astype(np.float32)
    floor = float(np.sqrt(np.mean(expect * expect)))
    err = float(np.max(np.abs(got - expect) / (np.abs(expect) + floor)))
    errs = [None] * world
    dist.all_gather_object(errs, err)
    if rank == 0:
        flops = 2.0 * M * N * K
        how = " (peer stores beside the GEMM)" if peers is not None else (" (overlapped all-gather)" if chunks > 1 else "")
        print(f"[row split] M={M} over {world} GPUs{how}: {float(ms):.3f} ms per product "
              f"including the exchange = {flops / float(ms) / 1e9:.0f} TFLOP/s aggregate")
        print(f"[row split] max-abs-rel error of 64 rows of every rank's gathered copy: {['%.2e' % e for e in errs]} (tolerance 1e-2)")
    if peers is not None:
        peers.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
