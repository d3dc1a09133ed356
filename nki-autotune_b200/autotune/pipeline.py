"""Host-buffer path of ``matmul_lhsT_rhs``: operands in pinned host memory, result in pinned host
memory, every step moving all of its bytes over PCIe.

The reference's driver owns the input tensors and the output buffer of every run
(``autotune/src/autotune/runner/driver.py:41-42, 104-106``); on a GPU that means host memory on one
side of the kernel and device memory on the other.  :class:`HostPipeline` keeps the three engines
of a step busy at the same time: while the kernel of step i runs, the upload of step i+1 and the
download of step i-1 are in flight (PCIe is full duplex), on one CUDA stream each and over
``depth`` sets of device buffers.  With several ranks (one process per GPU) an operand that is the
same on every rank -- ``rhs`` of a row split -- crosses PCIe once in total, 1/world of it on every
rank, and reaches the other GPUs over NVLink by an NCCL all-gather on a fourth stream, so that it
never holds up a rank's own upload of ``lhs_T``.

Every stream records CUDA events around its part of each step; :meth:`HostPipeline.breakdown`
turns them into per-engine milliseconds and GB/s, which is how a run says what limited it.
"""

from __future__ import annotations

import os
import statistics
from pathlib import Path

import torch

from autotune import kernels
from autotune.native import NativeError


def gpu_numa_node(device_index: int) -> int | None:
    """NUMA node of a visible CUDA device, from sysfs (read-only); ``None`` when unknown."""
    bus_id = None
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus_id = "%04x:%02x:%02x.0" % (int(props.pci_domain_id), int(props.pci_bus_id), int(props.pci_device_id))
    except Exception:  # noqa: BLE001 - a torch without these fields: ask NVML
        bus_id = None
    if bus_id is None:
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = [v.strip() for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip()]
            phys = int(vis[device_index]) if vis and vis[device_index].isdigit() else device_index
            bus_id = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(phys)).busId
            if isinstance(bus_id, bytes):
                bus_id = bus_id.decode()
        except Exception:  # noqa: BLE001
            return None
    bus_id = str(bus_id).lower()
    if len(bus_id.split(":")[0]) == 8:  # NVML prints an 8-digit PCI domain, sysfs uses 4
        bus_id = bus_id[4:]
    node_file = Path("/sys/bus/pci/devices") / bus_id / "numa_node"
    try:
        node = int(node_file.read_text().strip())
    except (OSError, ValueError):
        return None
    return node if node >= 0 else None


def bind_to_gpu_numa_node(device_index: int) -> dict:
    """Restrict this process to the CPUs of the NUMA node its GPU hangs off (best effort), so that
    pinned staging buffers allocated afterwards are first-touched next to the GPU's PCIe root.
    Changes only this process's own CPU affinity.  Returns what was done, for the record."""
    node = gpu_numa_node(device_index)
    if node is None:
        return {"numa_node": None, "bound": False}
    try:
        text = (Path("/sys/devices/system/node") / f"node{node}" / "cpulist").read_text().strip()
        cpus: set[int] = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if not use:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, use)
        return {"numa_node": node, "bound": True, "cpus": len(use)}
    except (OSError, ValueError):
        return {"numa_node": node, "bound": False}


class _Slot:
    """One set of device buffers and the events that order its reuse."""

    def __init__(self, k: int, m: int, n: int, device):
        self.a = torch.empty((k, m), dtype=torch.bfloat16, device=device)
        self.b = torch.empty((k, n), dtype=torch.bfloat16, device=device)
        self.out = torch.empty((m, n), dtype=torch.bfloat16, device=device)
        self.kernel_done: torch.cuda.Event | None = None
        self.d2h_done: torch.cuda.Event | None = None


class HostPipeline:
    """``out_host = lhs_T_host.T @ rhs_host`` step after step, with uploads, kernels and downloads
    overlapped.

    ``group``: a NCCL process group when ``rhs`` is the same on every rank.  With
    ``share_rhs_upload`` every rank uploads 1/world of its rows and the parts are all-gathered over
    NVLink into every rank's own buffer; otherwise rank ``src`` uploads all of it and broadcasts.
    Either way kernels only ever read local memory.  ``cfg`` is the kernel configuration
    (``None`` = the library's default).
    """

    def __init__(self, K: int, M: int, N: int, cfg: dict | None = None, depth: int = 2, device=None,
                 group=None, src: int = 0, record: int = 64, share_rhs_upload: bool = True):
        if not torch.cuda.is_available():
            raise NativeError(-1, "HostPipeline needs a CUDA device (there is no CPU path)")
        self.K, self.M, self.N = K, M, N
        self.cfg = cfg
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.group = group
        self.src = src
        self.rank = 0
        self._split_rows = None
        if group is not None:
            import torch.distributed as dist

            self._dist = dist
            self.rank = dist.get_rank(group)
            self._src_global = dist.get_global_rank(group, src)
            world = dist.get_world_size(group)
            if share_rhs_upload and K % world == 0:
                self._split_rows = (self.rank * (K // world), (self.rank + 1) * (K // world))
        self.slots = [_Slot(K, M, N, self.device) for _ in range(max(2, depth))]
        self.h2d = torch.cuda.Stream(self.device)
        self.d2h = torch.cuda.Stream(self.device)
        self.bcast = torch.cuda.Stream(self.device) if group is not None else None
        self.status = kernels.new_status(self.device)
        self.steps = 0
        self._record = record
        self._events: list[dict] = []

    # -- one step -------------------------------------------------------------------------------
    def step(self, lhs_T_host: torch.Tensor, rhs_host: torch.Tensor | None, out_host: torch.Tensor) -> None:
        """Enqueue one product; returns at once.  The tensors must be pinned host memory
        (``rhs_host`` may be ``None`` on ranks other than ``src`` when a group replicates it);
        ``out_host`` is complete after :meth:`drain` (or once a later step has reused its slot)."""
        for t in (lhs_T_host, rhs_host, out_host):
            if t is not None and (t.is_cuda or not t.is_pinned()):
                raise NativeError(-1, "HostPipeline.step takes pinned host tensors")
        slot = self.slots[self.steps % len(self.slots)]
        self.steps += 1
        main = torch.cuda.current_stream(self.device)
        ev = {name: torch.cuda.Event(enable_timing=True) for name in
              ("h2d0", "h2d1", "bc0", "bc1", "k0", "k1", "d2h0", "d2h1")}
        # who uploads rhs: without a group this rank, all of it; with a group every rank uploads its
        # 1/world of the rows and the parts are all-gathered over NVLink (the PCIe load is the same
        # on every rank); if K does not divide, or a rank has no copy, rank `src` uploads all of it
        # and broadcasts
        split = self.group is not None and self._split_rows is not None
        if split and rhs_host is None:
            raise NativeError(-1, "every rank must pass rhs when its upload is shared between the ranks")
        uploads_all = self.group is None or (not split and self.rank == self.src)
        with torch.cuda.stream(self.h2d):
            if slot.kernel_done is not None:
                self.h2d.wait_event(slot.kernel_done)  # the kernel that last read this set has finished
            ev["h2d0"].record(self.h2d)
            slot.a.copy_(lhs_T_host, non_blocking=True)
            a_up = torch.cuda.Event()
            a_up.record(self.h2d)
            if uploads_all:
                if rhs_host is None:
                    raise NativeError(-1, "the rank that owns rhs must pass it")
                slot.b.copy_(rhs_host, non_blocking=True)
            elif split:
                k0, k1 = self._split_rows
                slot.b[k0:k1].copy_(rhs_host[k0:k1], non_blocking=True)
            ev["h2d1"].record(self.h2d)
        main.wait_event(a_up if self.group is not None else ev["h2d1"])
        if self.group is not None:
            with torch.cuda.stream(self.bcast):
                if slot.kernel_done is not None:
                    self.bcast.wait_event(slot.kernel_done)
                self.bcast.wait_event(ev["h2d1"])  # this rank's part of rhs has been uploaded
                ev["bc0"].record(self.bcast)
                if split:
                    k0, k1 = self._split_rows
                    self._dist.all_gather_into_tensor(slot.b, slot.b[k0:k1], group=self.group)
                else:
                    self._dist.broadcast(slot.b, src=self._src_global, group=self.group)
                ev["bc1"].record(self.bcast)
            main.wait_event(ev["bc1"])
        if slot.d2h_done is not None:
            main.wait_event(slot.d2h_done)  # this set's previous result has left the device
        ev["k0"].record(main)
        kernels.matmul_lhsT_rhs(slot.a, slot.b, cfg=self.cfg, out=slot.out, status=self.status)
        ev["k1"].record(main)
        slot.kernel_done = ev["k1"]
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(ev["k1"])
            ev["d2h0"].record(self.d2h)
            out_host.copy_(slot.out, non_blocking=True)
            ev["d2h1"].record(self.d2h)
        slot.d2h_done = ev["d2h1"]
        self._events.append(ev)
        if len(self._events) > self._record:
            self._events.pop(0)

    def start(self) -> None:
        """Order the side streams after the work already queued on the current stream (call once
        before the first step of a timed region, after its start event)."""
        main = torch.cuda.current_stream(self.device)
        self.h2d.wait_stream(main)
        self.d2h.wait_stream(main)
        if self.bcast is not None:
            self.bcast.wait_stream(main)

    def drain(self) -> None:
        """Make the current stream wait for every download queued so far (does not block the host)."""
        torch.cuda.current_stream(self.device).wait_stream(self.d2h)

    def finish(self) -> None:
        """Block until everything queued has completed and raise if a device-side wait expired."""
        self.drain()
        torch.cuda.synchronize(self.device)
        kernels.raise_on_status(self.status)

    # -- record ---------------------------------------------------------------------------------
    def breakdown(self) -> dict:
        """Median milliseconds each engine spent per step over the recorded steps (call after
        :meth:`finish`), with the bytes moved and the rates they imply."""
        if not self._events:
            return {}
        def med(a: str, b: str) -> float:
            return statistics.median(e[a].elapsed_time(e[b]) for e in self._events)

        elem = 2
        if self.group is None:
            rhs_up = self.K * self.N * elem
        elif self._split_rows is not None:
            rhs_up = (self._split_rows[1] - self._split_rows[0]) * self.N * elem
        else:
            rhs_up = self.K * self.N * elem if self.rank == self.src else 0
        h2d_bytes = self.K * self.M * elem + rhs_up
        d2h_bytes = self.M * self.N * elem
        out = {"h2d_ms": round(med("h2d0", "h2d1"), 4), "kernel_ms": round(med("k0", "k1"), 4),
               "d2h_ms": round(med("d2h0", "d2h1"), 4), "h2d_bytes": h2d_bytes, "d2h_bytes": d2h_bytes,
               "steps_recorded": len(self._events)}
        out["h2d_gbs"] = round(h2d_bytes / out["h2d_ms"] / 1e6, 1) if out["h2d_ms"] > 0 else None
        out["d2h_gbs"] = round(d2h_bytes / out["d2h_ms"] / 1e6, 1) if out["d2h_ms"] > 0 else None
        if self.group is not None:
            out["bcast_ms"] = round(med("bc0", "bc1"), 4)
            out["bcast_bytes"] = self.K * self.N * elem
        return out


def matmul_lhsT_rhs_pipelined(lhs_T_batches, rhs_batches, cfg: dict | None = None) -> list:
    """Products of a sequence of host operand pairs (numpy bf16 arrays of one shape each), through
    pinned staging buffers and a :class:`HostPipeline`; returns numpy bf16 arrays."""
    import ml_dtypes
    import numpy as np

    lhs_T_batches, rhs_batches = list(lhs_T_batches), list(rhs_batches)
    if not lhs_T_batches or len(lhs_T_batches) != len(rhs_batches):
        raise NativeError(-1, "need as many lhs_T arrays as rhs arrays, and at least one")
    K, M = lhs_T_batches[0].shape
    N = rhs_batches[0].shape[1]
    pipe = HostPipeline(K, M, N, cfg=cfg)
    depth = len(pipe.slots)

    def pinned(shape):
        return torch.empty(shape, dtype=torch.bfloat16).pin_memory()

    a_st = [pinned((K, M)) for _ in range(depth)]
    b_st = [pinned((K, N)) for _ in range(depth)]
    c_st = [pinned((M, N)) for _ in range(depth)]
    results: list = [None] * len(lhs_T_batches)
    pipe.start()
    for i, (a, b) in enumerate(zip(lhs_T_batches, rhs_batches)):
        s = i % depth
        if i >= depth:
            # staging set s is about to be overwritten: its download must be on the host first
            pipe.slots[s].d2h_done.synchronize()
            results[i - depth] = c_st[s].view(torch.uint16).numpy().view(ml_dtypes.bfloat16).copy()
        a_st[s].view(torch.uint16).numpy()[...] = np.ascontiguousarray(a).view(np.uint16)
        b_st[s].view(torch.uint16).numpy()[...] = np.ascontiguousarray(b).view(np.uint16)
        pipe.step(a_st[s], b_st[s], c_st[s])
    pipe.finish()
    for i in range(max(0, len(results) - depth), len(results)):
        results[i] = c_st[i % depth].view(torch.uint16).numpy().view(ml_dtypes.bfloat16).copy()
    return results
