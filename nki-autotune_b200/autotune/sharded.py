"""Large-M product split by rows of C over the GPUs of one node.

``C[M, N] = lhs_T[K, M].T @ rhs[K, N]`` with M much larger than N and K: rank r multiplies its
column block ``lhs_T[:, m0:m1]`` by the whole of ``rhs`` and owns rows ``m0:m1`` of C.  The GEMM
kernels only ever read and write memory of their own GPU.  The two exchange steps around them run
as NCCL collectives over NVLink, each landing in local memory before any kernel touches it:

* ``replicate`` -- ``rhs`` is uploaded once (by ``src``) and broadcast, instead of one
  host-to-device copy per GPU;
* ``gather_rows`` -- the row blocks of C are all-gathered on the device, instead of one
  device-to-host copy per GPU followed by a host-side concatenation;
* with ``chunks > 1`` the split is block-cyclic and the all-gather of one band of C overlaps the
  multiplication of the next.

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

from autotune import kernels, native


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


def cyclic_rows(M: int, rank: int, world: int, chunks: int) -> list[tuple[int, int]]:
    """Rows of C owned by ``rank`` when the split is block-cyclic: M is cut into ``chunks`` bands of
    ``world`` equal pieces and rank r owns piece r of every band.  The pieces of one band are one
    contiguous range of C, which is what lets the band be all-gathered in place while the next band
    is still being multiplied.  Needs M divisible by ``8 * world * chunks``."""
    if chunks < 1 or M % (8 * world * chunks) != 0:
        raise ValueError(f"M={M} must be a multiple of 8 * world * chunks = {8 * world * chunks}")
    piece = M // (world * chunks)
    return [((i * world + rank) * piece, (i * world + rank + 1) * piece) for i in range(chunks)]


def cuda_ipc_handle(exported: bytes) -> bytes:
    """The 64-byte ``cudaIpcMemHandle_t`` inside what ``UntypedStorage._share_cuda_()`` returns.

    torch prefixes the handle with a version byte and a kind byte (older versions: the kind byte
    only, or nothing): kind ``c`` is a plain ``cudaMalloc`` block.  Memory of an expandable segment
    (kind ``e``) is exported as file descriptors, not as a CUDA IPC handle, and is refused here.
    """
    exported = bytes(exported)
    if len(exported) not in (64, 65, 66) or (len(exported) > 64 and exported[-65:-64] != b"c"):
        raise RuntimeError(f"not a CUDA IPC handle of a cudaMalloc block: {len(exported)} bytes, prefix {exported[:-64]!r}")
    return exported[-64:]


class PeerCopies:
    """Every rank's copy of one ``[M, N]`` array, each mapped into every other rank's process.

    ``local`` is this rank's copy (ordinary device memory of this GPU); the other ranks' copies are
    mapped through CUDA IPC: every rank exports the allocation behind its copy, the 64-byte handles
    travel with ``all_gather_object``, and every rank opens them with ITS OWN GPU current -- the
    mapping is then valid for kernels of this GPU, and peer access to the owner is switched on.
    ``push_rows`` stores a row range of the local copy into the same rows of every peer's copy with
    the library's own kernel -- plain stores over NVLink, local reads only, no collective -- and
    ``barrier`` is the stream-ordered meeting point after which every copy holds what every rank
    pushed.  A rank may not push into rows that a peer is still reading: meet at ``barrier()``
    first (or alternate two buffers).  ``close()`` unmaps; the owner's memory must outlive that.
    """

    def __init__(self, M: int, N: int, dtype=torch.bfloat16, device=None, group=None):
        import ctypes as C

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.local = torch.empty((M, N), dtype=dtype, device=device)
        self.row_bytes = N * self.local.element_size()
        # (device, handle, size, offset of the storage inside the exported allocation, ...)
        shared = self.local.untyped_storage()._share_cuda_()
        mine = (bytes(shared[1]), int(shared[3]) + self.local.storage_offset() * self.local.element_size(), M * self.row_bytes)
        table: list = [None] * self.world
        dist.all_gather_object(table, mine, group=group)
        self._bases: dict[int, int] = {}
        self._ptrs: dict[int, int] = {}
        lib = native.load()
        problem = None
        try:
            with torch.cuda.device(device):
                for r, (handle, offset, nbytes) in enumerate(table):
                    if r == self.rank:
                        continue
                    if nbytes != M * self.row_bytes:
                        raise RuntimeError(f"rank {r} exported {nbytes} bytes, expected {M * self.row_bytes}")
                    base = C.c_void_p()
                    native.check(lib.b200_ipc_open(cuda_ipc_handle(handle), C.byref(base)))
                    self._bases[r] = base.value
                    self._ptrs[r] = base.value + offset
        except Exception as exc:  # noqa: BLE001 - reported to every rank below
            problem = f"rank {self.rank}: {exc}"
        # every rank learns whether every rank could map every copy: either all go on or all raise
        # (a rank that raised alone would leave the others waiting in the first barrier)
        problems: list = [None] * self.world
        dist.all_gather_object(problems, problem, group=group)
        if any(problems):
            with torch.cuda.device(device):
                for base in self._bases.values():
                    lib.b200_ipc_close(base)
            self._bases, self._ptrs = {}, {}
            raise RuntimeError("peer mappings could not be made: " + "; ".join(p for p in problems if p))
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.barrier()

    def push_rows(self, r0: int, r1: int, max_ctas: int = 0) -> None:
        """Rows ``[r0, r1)`` of the local copy -> the same rows of every peer's copy (current stream)."""
        import ctypes as C

        if r1 <= r0 or not self._ptrs:
            return
        if r0 < 0 or r1 > self.local.shape[0]:
            raise ValueError(f"rows [{r0}, {r1}) are outside the array of {self.local.shape[0]} rows")
        ptrs = (C.c_void_p * len(self._ptrs))(*[p + r0 * self.row_bytes for _, p in sorted(self._ptrs.items())])
        native.check(native.load().b200_peer_store(
            self.local.data_ptr() + r0 * self.row_bytes, ptrs, len(self._ptrs), (r1 - r0) * self.row_bytes, int(max_ctas),
            torch.cuda.current_stream(self.local.device).cuda_stream))

    def barrier(self) -> None:
        """Stream-ordered: past this point on the current stream, every rank's earlier pushes are in."""
        dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        """Unmap the peers' copies (after a barrier: nobody may still be pushing)."""
        if self._bases:
            self.barrier()
            torch.cuda.synchronize(self.local.device)
            lib = native.load()
            with torch.cuda.device(self.local.device):
                for base in self._bases.values():
                    lib.b200_ipc_close(base)
            self._bases, self._ptrs = {}, {}
            self.barrier()
            torch.cuda.synchronize(self.local.device)


def matmul_lhsT_rhs_row_split(
    lhs_T_block: torch.Tensor,
    rhs: torch.Tensor,
    M: int,
    cfg: dict | None = None,
    group=None,
    gather: bool = True,
    out_full: torch.Tensor | None = None,
    matmul: Callable | None = None,
    chunks: int = 1,
    spare_ctas: int = 16,
    peers: "PeerCopies | None" = None,
) -> tuple[torch.Tensor, torch.Tensor | None]:
    """This rank's rows of ``lhs_T.T @ rhs`` and, with ``gather``, the whole of C on every rank.

    ``chunks == 1``: ``lhs_T_block`` is ``lhs_T[:, m0:m1]`` for ``(m0, m1) = row_range(M, rank, world)``
    -- a view with the full row stride is fine, no copy is made -- and ``rhs`` this rank's replica
    (see ``replicate``); the all-gather runs after the kernel.

    ``chunks > 1`` (needs ``gather``): the split is block-cyclic (``cyclic_rows``); ``lhs_T_block``
    holds the columns of ``lhs_T`` for this rank's pieces, band after band.  Band i is multiplied on
    the current stream while band i-1 is all-gathered (in place, into its contiguous range of C) on
    a second stream, so that only the last band's exchange is not hidden.  The GEMM's grid is kept
    ``spare_ctas`` CTAs below the machine, which leaves the collective's CTAs room to be resident
    beside it.  Returns ``(None, out_full)`` in this mode: the rank's rows are not one block.

    ``peers`` (a ``PeerCopies`` of shape ``[M, N]``; needs ``gather``): C is ``peers.local`` and the
    exchange is this library's own peer-store kernel instead of the collective: each band's rows go
    straight into every other GPU's copy of C over NVLink while the next band is multiplied, and one
    small barrier at the end replaces the all-gathers.  Returns ``(None, peers.local)``.

    ``matmul(lhs_T_block, rhs, cfg=..., out=...)`` defaults to the tcgen05 GEMM.
    """
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    run = matmul if matmul is not None else kernels.matmul_lhsT_rhs
    n = rhs.shape[1]
    if peers is not None:
        if not gather or tuple(peers.local.shape) != (M, n):
            raise ValueError(f"peers must hold [{M}, {n}] and needs gather=True")
        if not lhs_T_block.is_cuda or peers.local.device != lhs_T_block.device:
            raise ValueError("the peer-store exchange runs on the GPU that holds this rank's copy of C")
        out_full = peers.local
        spans = [row_range(M, rank, world)] if chunks == 1 else cyclic_rows(M, rank, world, chunks)
        if lhs_T_block.shape[1] != sum(b - a for a, b in spans):
            raise ValueError(f"rank {rank}: lhs_T block has {lhs_T_block.shape[1]} columns, the split gives {sum(b - a for a, b in spans)}")
        use_cfg = cfg
        if matmul is None and spare_ctas > 0 and chunks > 1:
            sms = torch.cuda.get_device_properties(lhs_T_block.device).multi_processor_count
            base = dict(cfg) if cfg is not None else native.default_cfg("matmul_lhsT_rhs", spans[0][1] - spans[0][0], n, lhs_T_block.shape[0])
            use_cfg = dict(base, _max_ctas=max(2, sms - spare_ctas))
        comm = _comm_stream(lhs_T_block.device)
        main = torch.cuda.current_stream(lhs_T_block.device)
        comm.wait_stream(main)
        col = 0
        for p0, p1 in spans:
            run(lhs_T_block[:, col:col + (p1 - p0)], rhs, cfg=use_cfg, out=out_full[p0:p1])
            col += p1 - p0
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(done)
                # beside a GEMM the store kernel's CTAs crowd onto the SMs the GEMM leaves free: eight
                # 256-thread CTAs per free SM keep enough stores in flight to fill the links
                peers.push_rows(p0, p1, max_ctas=8 * spare_ctas if chunks > 1 else 0)
        main.wait_stream(comm)
        peers.barrier()
        return None, out_full
    if chunks > 1:
        if not gather:
            raise ValueError("chunks > 1 is the overlapped all-gather: it needs gather=True")
        pieces = cyclic_rows(M, rank, world, chunks)
        piece = pieces[0][1] - pieces[0][0]
        if lhs_T_block.shape[1] != piece * chunks:
            raise ValueError(f"rank {rank}: lhs_T block has {lhs_T_block.shape[1]} columns, the cyclic split gives {piece * chunks}")
        if out_full is None:
            out_full = torch.empty((M, n), dtype=lhs_T_block.dtype, device=lhs_T_block.device)
        use_cfg = cfg
        if matmul is None and lhs_T_block.is_cuda and spare_ctas > 0:
            sms = torch.cuda.get_device_properties(lhs_T_block.device).multi_processor_count
            base = dict(cfg) if cfg is not None else native.default_cfg("matmul_lhsT_rhs", piece, n, lhs_T_block.shape[0])
            use_cfg = dict(base, _max_ctas=max(2, sms - spare_ctas))
        on_gpu = lhs_T_block.is_cuda
        comm = _comm_stream(lhs_T_block.device) if on_gpu else None
        main = torch.cuda.current_stream(lhs_T_block.device) if on_gpu else None
        if on_gpu:
            comm.wait_stream(main)  # out_full may still be read by work queued earlier
        for i, (p0, p1) in enumerate(pieces):
            band = out_full[i * world * piece:(i + 1) * world * piece]
            run(lhs_T_block[:, i * piece:(i + 1) * piece], rhs, cfg=use_cfg, out=out_full[p0:p1])
            if on_gpu:
                done = torch.cuda.Event()
                done.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(done)
                    dist.all_gather_into_tensor(band, out_full[p0:p1], group=group)
            else:
                dist.all_gather_into_tensor(band, out_full[p0:p1].contiguous(), group=group)
        if on_gpu:
            main.wait_stream(comm)
        return None, out_full
    m0, m1 = row_range(M, rank, world)
    if lhs_T_block.shape[1] != m1 - m0:
        raise ValueError(f"rank {rank}: lhs_T block has {lhs_T_block.shape[1]} columns, row_range gives {m1 - m0}")
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


_COMM_STREAMS: dict = {}


def _comm_stream(device) -> "torch.cuda.Stream":
    """One side stream per device for the exchange steps that overlap the kernels."""
    key = torch.device(device).index
    if key not in _COMM_STREAMS:
        _COMM_STREAMS[key] = torch.cuda.Stream(device)
    return _COMM_STREAMS[key]
