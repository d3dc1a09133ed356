"""Large-M product split by rows of C over the GPUs of one node.

``C[M, N] = lhs_T[K, M].T @ rhs[K, N]`` with M much larger than N and K: rank r multiplies its
column block ``lhs_T[:, m0:m1]`` by the whole of ``rhs`` and owns rows ``m0:m1`` of C.  The GEMM
kernels only ever read and write memory of their own GPU.  The two exchange steps around them run
as NCCL collectives over NVLink, each landing in local memory before any kernel touches it:

* ``replicate`` -- ``rhs`` is uploaded once (by ``src``) and broadcast, instead of one
  host-to-device copy per GPU;
* ``gather_rows`` -- the row blocks of C are all-gathered on the device, instead of one
  device-to-host copy per GPU followed by a host-side concatenation.

The reference has no multi-device path (its benchmark loop is one device, serial:
autotune/src/autotune/runner/driver.py:97); this is the sharding its large-M configuration needs.
One process per GPU; ``group`` is a ``torch.distributed`` group whose backend can move the tensors
given (NCCL for device tensors; the host-logic tests use gloo with host tensors and a stand-in
``matmul``).
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

from autotune import kernels


def row_range(M: int, rank: int, world: int, align: int = 8) -> tuple[int, int]:
    """Rows of C owned by ``rank``: contiguous blocks of ``align``-row units, remainder units to the
    first ranks, ragged tail rows to the last rank.  ``align`` keeps every block's first column of
    ``lhs_T`` on a 16-byte boundary (8 bf16 elements), which the TMA tensor maps require."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if M < 0 or align < 1:
        raise ValueError("M must be >= 0 and align >= 1")
    units, tail = divmod(M, align)
    base, extra = divmod(units, world)
    start_units = rank * base + min(rank, extra)
    n_units = base + (1 if rank < extra else 0)
    start = start_units * align
    stop = start + n_units * align
    if rank == world - 1:
        stop += tail
    return start, stop


def replicate(t: torch.Tensor | None, shape, dtype, device, src: int = 0, group=None) -> torch.Tensor:
    """Copy of ``src``'s tensor in this rank's own memory (one broadcast; ``t`` is ignored elsewhere)."""
    rank = dist.get_rank(group)
    if rank == src:
        if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
            raise ValueError("replicate: the source rank must pass a tensor of the announced shape and dtype")
        local = t.contiguous()
    else:
        local = torch.empty(tuple(shape), dtype=dtype, device=device)
    dist.broadcast(local, src=dist.get_global_rank(group, src) if group is not None else src, group=group)
    return local


def gather_rows(c_block: torch.Tensor, M: int, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All ranks' row blocks of C, in rank order, in this rank's memory (``out[M, N]`` if given)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    n = c_block.shape[1]
    if out is None:
        out = torch.empty((M, n), dtype=c_block.dtype, device=c_block.device)
    if tuple(out.shape) != (M, n) or not out.is_contiguous():
        raise ValueError("gather_rows: out must be a contiguous [M, N] tensor")
    bounds = [row_range(M, r, world) for r in range(world)]
    if c_block.shape[0] != bounds[rank][1] - bounds[rank][0]:
        raise ValueError("gather_rows: this rank's block does not have the rows row_range assigns to it")
    sizes = {b1 - b0 for b0, b1 in bounds}
    block = c_block.contiguous()
    if len(sizes) == 1:
        dist.all_gather_into_tensor(out, block, group=group)  # equal blocks: straight into place
    else:
        # ragged blocks: one broadcast per owner (uneven all-gathers are not portable across backends)
        out[bounds[rank][0]:bounds[rank][1]].copy_(block)
        for r, (b0, b1) in enumerate(bounds):
            if b1 > b0:
                src = dist.get_global_rank(group, r) if group is not None else r
                dist.broadcast(out[b0:b1], src=src, group=group)
    return out


def matmul_lhsT_rhs_row_split(
    lhs_T_block: torch.Tensor,
    rhs: torch.Tensor,
    M: int,
    cfg: dict | None = None,
    group=None,
    gather: bool = True,
    out_full: torch.Tensor | None = None,
    matmul: Callable | None = None,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """This rank's rows of ``lhs_T.T @ rhs`` and, with ``gather``, the whole of C on every rank.

    ``lhs_T_block`` is ``lhs_T[:, m0:m1]`` for ``(m0, m1) = row_range(M, rank, world)`` -- a view with
    the full row stride is fine, no copy is made -- and ``rhs`` this rank's replica (see
    ``replicate``).  ``matmul(lhs_T_block, rhs, cfg=..., out=...)`` defaults to the tcgen05 GEMM.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    m0, m1 = row_range(M, rank, world)
    if lhs_T_block.shape[1] != m1 - m0:
        raise ValueError(f"rank {rank}: lhs_T block has {lhs_T_block.shape[1]} columns, row_range gives {m1 - m0}")
    run = matmul if matmul is not None else kernels.matmul_lhsT_rhs
    n = rhs.shape[1]
    if gather and out_full is None:
        out_full = torch.empty((M, n), dtype=lhs_T_block.dtype, device=lhs_T_block.device)
    if gather and len({b1 - b0 for b0, b1 in (row_range(M, r, world) for r in range(world))}) == 1:
        # equal blocks: the kernel writes its rows of the full array and the all-gather runs in place
        c_block = out_full[m0:m1]
        run(lhs_T_block, rhs, cfg=cfg, out=c_block)
        dist.all_gather_into_tensor(out_full, c_block, group=group)
        return c_block, out_full
    c_block = torch.empty((m1 - m0, n), dtype=lhs_T_block.dtype, device=lhs_T_block.device)
    run(lhs_T_block, rhs, cfg=cfg, out=c_block)
    if not gather:
        return c_block, None
    return c_block, gather_rows(c_block, M, group=group, out=out_full)
