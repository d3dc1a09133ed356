"""Sweep orchestration: validate every candidate, shard the accepted ones over the GPUs of
the box, time each on its GPU, gather the results on the host.

Mirrors ``run_pipeline`` (``autotune/src/autotune/runner/driver.py:126-165``): per-candidate
failures never raise, batch misuse does.  Differences that follow from the hardware: the
"compile" stage is a budget check (no compiler runs), and the serial benchmark loop on one
NeuronCore becomes one worker process per GPU.  Candidate ``i`` of the accepted list goes to
GPU ``i mod G``; workers are independent, there is no collective and no peer access -- results
travel back over pipes.  A worker that dies or overruns its deadline costs only the candidate
it was on: that candidate becomes a failure row and a fresh worker takes over the rest.
"""

from __future__ import annotations

import atexit
import logging
import multiprocessing as mp
import os
import shutil
import tempfile
import time
from pathlib import Path
from typing import Any, Callable

from autotune.runner.candidate import parse_source
from autotune.runner.compile import compile_one
from autotune.runner.types import (
    CompileResult,
    KernelJob,
    OutputSpec,
    ProfileResult,
    capture_error,
    compile_failure_result,
    make_failure,
    resolve_dtype,
)

logger = logging.getLogger(__name__)

_OUTPUT_TENSOR_NAME = "hbm_tensor_0"
DEFAULT_DEADLINE_S = 300.0


def _tensor_specs(job: KernelJob) -> dict[str, dict]:
    specs = {}
    for name, spec in job.input_specs.items():
        shape, dtype = spec[0], spec[1]
        entry: dict[str, Any] = {"shape": list(shape), "dtype": dtype}
        if len(spec) > 2 and spec[2]:
            entry["dist"] = dict(spec[2])
        specs[name] = entry
    return specs


def _prepare_kernel(kname: str, job: KernelJob, nki_dir: Path) -> dict[str, Any]:
    """Write the descriptor to disk and collect what a worker needs (reference: driver.py:35-52)."""
    filename = kname if kname.endswith(".py") else f"{kname}.py"
    path = nki_dir / filename
    path.write_text(job.source)
    return {
        "kernel_name": kname,
        "nki_path": str(path),
        "func_name": job.func_name,
        "output_shape": tuple(job.output_shape),
        "tensor_specs": _tensor_specs(job),
        "input_dtype_name": next(iter(job.input_specs.values()))[1],
        "source": job.source,
    }


def shard_round_robin(items: list, n_workers: int) -> list[list]:
    """Item ``i`` goes to worker ``i mod n_workers`` (deterministic)."""
    shards: list[list] = [[] for _ in range(max(1, n_workers))]
    for i, item in enumerate(items):
        shards[i % len(shards)].append(item)
    return shards


# ----------------------------------------------------------------------------- GPU worker body
def batch_key(kd: dict) -> str:
    """Candidates with the same key share one set of input tensors (same family, specs, output, scalars)."""
    cand = parse_source(kd["source"])
    return repr((kd["func_name"], kd["tensor_specs"], kd["output_shape"], sorted(cand.scalars.items())))


class SharedInputs:
    """Seeded input tensors generated once by the parent and handed to every worker process
    through POSIX shared memory, so that a sweep sharded over G GPUs does not pay G times for
    the host-side random number generation (which costs more than timing a dozen candidates).

    ``publish`` copies the arrays of one batch into named blocks and returns a small descriptor
    (names, shapes, dtypes) that travels to the workers inside ``opts``; ``attach`` maps them
    read-only as numpy arrays in the worker.  The parent keeps the blocks alive until ``close``.
    """

    def __init__(self):
        self._blocks = []

    def publish(self, tensors: dict) -> dict:
        from multiprocessing import shared_memory

        import numpy as np

        desc = {}
        for name, arr in tensors.items():
            arr = np.ascontiguousarray(arr)
            raw = arr.view(np.uint8).reshape(-1)
            shm = shared_memory.SharedMemory(create=True, size=max(1, raw.nbytes))
            np.frombuffer(shm.buf, dtype=np.uint8, count=raw.nbytes)[:] = raw
            self._blocks.append(shm)
            desc[name] = {"shm": shm.name, "shape": list(arr.shape), "dtype": arr.dtype.name}
        return desc

    @staticmethod
    def attach(desc: dict) -> tuple[dict, list]:
        """-> (arrays by tensor name, handles to close when the arrays are no longer needed)."""
        from multiprocessing import shared_memory

        import numpy as np

        arrays, handles = {}, []
        for name, d in desc.items():
            shm = shared_memory.SharedMemory(name=d["shm"])
            handles.append(shm)
            dtype = resolve_dtype(d["dtype"])
            count = int(np.prod(d["shape"])) if d["shape"] else 1
            arrays[name] = np.frombuffer(shm.buf, dtype=dtype, count=count).reshape(d["shape"])
        return arrays, handles

    def close(self) -> None:
        for shm in self._blocks:
            try:
                shm.close()
                shm.unlink()
            except FileNotFoundError:
                pass
        self._blocks = []


def gpu_shard_worker(items: list[dict], opts: dict, emit: Callable[[ProfileResult], None]) -> None:
    """Time every candidate of one shard on the current process's GPU 0.

    Inputs come, in this order of preference, from ``opts["inputs"]`` (arrays the caller already
    holds), from ``opts["shared_inputs"]`` (shared-memory blocks published by the parent, keyed
    by batch) or from the seed (same seed -> same tensors on every GPU).  Candidates that share
    input specs share one device copy.
    """
    from autotune.runner.benchmark import DeviceBatch, benchmark_one, generate_tensors

    batches: dict[str, Any] = {}
    for kd in items:
        cr = CompileResult(kd["kernel_name"], kd["nki_path"], "", "")
        try:
            cand = parse_source(kd["source"])
            key = batch_key(kd)
            if key not in batches:
                batches.clear()  # one batch resident at a time bounds device memory
                handles: list = []
                if opts.get("inputs") is not None:
                    kwargs = {n: opts["inputs"][n] for n in kd["tensor_specs"]}
                elif key in (opts.get("shared_inputs") or {}):
                    kwargs, handles = SharedInputs.attach(opts["shared_inputs"][key])
                else:
                    kwargs = generate_tensors(kd["tensor_specs"], opts["seed"])
                out = OutputSpec(_OUTPUT_TENSOR_NAME, kd["output_shape"], resolve_dtype(kd["input_dtype_name"]))
                batches[key] = DeviceBatch(kd["func_name"], kwargs, out, cand.scalars)
                del kwargs  # (DeviceBatch keeps no reference to the host arrays)
                for h in handles:  # the device copy exists: the mapping can go
                    try:
                        h.close()
                    except BufferError:  # a view of the block is still alive somewhere: leave it mapped
                        logger.warning("shared input block %s stays mapped in worker %d", h.name, os.getpid())
            result = benchmark_one(
                batches[key], cr, cand, warmup=opts["warmup"], iters=opts["iters"],
                collect_detailed_profile=opts["detailed"],
            )
        except Exception as exc:  # noqa: BLE001
            result = make_failure(kd["kernel_name"], capture_error(exc))
        emit(result)


# ----------------------------------------------------------------------------- process pool
def _child_main(worker_fn, items, opts, device_env, conn) -> None:
    """Entry point of a worker process: pin the GPU before any CUDA library is imported."""
    if device_env is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = device_env
    try:
        worker_fn(items, opts, lambda r: conn.send(("result", tuple(r))))
        conn.send(("done", None))
    except BaseException as exc:  # noqa: BLE001
        try:
            conn.send(("crash", capture_error(exc)))
        except Exception:  # noqa: BLE001
            pass
    finally:
        conn.close()


def _service_main(device_env, conn) -> None:
    """Entry point of a resident worker: pins the GPU, then serves jobs until told to stop (or
    until the parent's end of the pipe closes).  One job = one shard of one ``profile()`` call."""
    if device_env is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = device_env
    try:
        while True:
            try:
                msg = conn.recv()
            except (EOFError, OSError):
                return
            if msg[0] != "job":
                return
            _, worker_fn, items, opts = msg
            try:
                worker_fn(items, opts, lambda r: conn.send(("result", tuple(r))))
                conn.send(("done", None))
            except BaseException as exc:  # noqa: BLE001
                conn.send(("crash", capture_error(exc)))
                return  # a worker that crashed is not reused
    finally:
        conn.close()


# Resident workers, by the device they are pinned to: processes that finished a shard cleanly and
# wait for the next profile() call of this process (keep_workers=True).  A second sweep then pays
# neither the process start nor the CUDA context again.
_RESIDENT: dict[str | None, tuple] = {}


def shutdown_workers() -> None:
    """Stop every resident worker of this process (also runs at interpreter exit)."""
    for key in list(_RESIDENT):
        proc, conn = _RESIDENT.pop(key)
        try:
            conn.send(("stop",))
        except (OSError, ValueError, BrokenPipeError):
            pass
        proc.join(timeout=10)
        if proc.is_alive():
            proc.terminate()  # exactly the PID this pool started
            proc.join(timeout=10)
        conn.close()


atexit.register(shutdown_workers)


def resident_worker_pids() -> dict:
    """{device: pid} of the workers that are waiting for a next sweep."""
    return {key: proc.pid for key, (proc, _) in _RESIDENT.items() if proc.is_alive()}


def run_sharded(
    shards: list[list[dict]],
    worker_fn: Callable,
    opts: dict,
    device_envs: list[str | None],
    deadline_s: float = DEFAULT_DEADLINE_S,
    startup_s: float = 600.0,
    keep_workers: bool = False,
) -> list[ProfileResult]:
    """Run one worker process per shard and gather ``ProfileResult`` rows on the host.

    Each item must carry ``"kernel_name"``.  ``worker_fn(items, opts, emit)`` must call
    ``emit`` once per item, in order.  The first result of a worker may take ``startup_s``
    (process start, CUDA context, input generation); every later one ``deadline_s``.

    ``keep_workers``: a worker that finishes its shard cleanly stays alive, pinned to its GPU,
    and serves the matching shard of the next call (``shutdown_workers()`` ends them; so does the
    end of this process).  Workers that crash or overrun a deadline are always replaced.
    """
    ctx = mp.get_context("spawn")
    results: list[ProfileResult] = []

    class _Slot:
        def __init__(self, idx: int, items: list[dict]):
            self.idx = idx
            self.pending = list(items)
            self.proc = None
            self.conn = None
            self.deadline = 0.0
            self.fresh = True

        def start(self) -> None:
            key = device_envs[self.idx]
            if keep_workers:
                resident = _RESIDENT.pop(key, None)
                if resident is not None and not resident[0].is_alive():
                    resident[1].close()
                    resident = None
                if resident is None:
                    parent, child = ctx.Pipe(duplex=True)
                    proc = ctx.Process(target=_service_main, args=(key, child), daemon=True)
                    proc.start()
                    child.close()
                    resident = (proc, parent)
                self.proc, self.conn = resident
                self.conn.send(("job", worker_fn, list(self.pending), opts))
            else:
                parent, child = ctx.Pipe(duplex=False)
                self.proc = ctx.Process(
                    target=_child_main, args=(worker_fn, list(self.pending), opts, key, child),
                    daemon=True,
                )
                self.proc.start()
                child.close()
                self.conn = parent
            self.fresh = True
            self.deadline = time.monotonic() + startup_s

        def park(self) -> None:
            """The shard is done and the worker is healthy: keep it for the next call."""
            _RESIDENT[device_envs[self.idx]] = (self.proc, self.conn)
            self.proc = None
            self.conn = None

        def stop(self) -> None:
            if self.proc is not None:
                if self.proc.is_alive():
                    self.proc.terminate()  # exactly the PID this pool started
                self.proc.join(timeout=10)
                if self.proc.is_alive():
                    self.proc.kill()
                    self.proc.join(timeout=10)
            if self.conn is not None:
                self.conn.close()
            self.proc = None
            self.conn = None

    slots = [_Slot(i, items) for i, items in enumerate(shards) if items]
    for s in slots:
        s.start()

    def _fail_current(slot: _Slot, why: str) -> None:
        item = slot.pending.pop(0)
        results.append(make_failure(item["kernel_name"], why))
        slot.stop()
        if slot.pending:
            slot.start()

    active = [s for s in slots if s.pending]
    while active:
        progressed = False
        for slot in list(active):
            try:
                has_msg = slot.conn.poll(0.05)
            except (EOFError, OSError):
                has_msg = False
            if has_msg:
                try:
                    kind, payload = slot.conn.recv()
                except (EOFError, OSError):
                    kind, payload = "eof", None
                progressed = True
                if kind == "result":
                    res = ProfileResult(*payload)
                    if slot.pending and slot.pending[0]["kernel_name"] == res.kernel_name:
                        slot.pending.pop(0)
                    else:
                        slot.pending = [it for it in slot.pending if it["kernel_name"] != res.kernel_name]
                    results.append(res)
                    slot.fresh = False
                    slot.deadline = time.monotonic() + deadline_s
                elif kind == "done":
                    for item in slot.pending:
                        results.append(make_failure(item["kernel_name"], "worker finished without a result"))
                    slot.pending = []
                    if keep_workers and device_envs[slot.idx] not in _RESIDENT:
                        slot.park()
                    else:
                        slot.stop()
                elif kind == "crash":
                    _fail_current(slot, f"worker crashed:\n{payload}")
                else:
                    _fail_current(slot, "worker process died without reporting (pipe closed)")
            elif slot.proc is not None and not slot.proc.is_alive():
                # drain anything it managed to send before dying
                if not slot.conn.poll(0):
                    _fail_current(slot, f"worker process died (exit code {slot.proc.exitcode})")
                    progressed = True
            elif time.monotonic() > slot.deadline:
                limit = startup_s if slot.fresh else deadline_s
                _fail_current(slot, f"worker exceeded its {limit:.0f} s deadline and was stopped")
                progressed = True
            if not slot.pending:
                if keep_workers and slot.proc is not None and device_envs[slot.idx] not in _RESIDENT:
                    # every row is in; the worker's own "done" follows at once -- park it when it does
                    try:
                        if slot.conn.poll(5.0) and slot.conn.recv()[0] == "done":
                            slot.park()
                    except (EOFError, OSError):
                        pass
                slot.stop()
                active.remove(slot)
        if not progressed:
            time.sleep(0.01)
    return results


# ----------------------------------------------------------------------------- pipeline
def _publish_inputs(shared: SharedInputs, accepted: list[dict], seed: int, inputs: dict | None) -> dict:
    """One set of input tensors per distinct batch of the accepted candidates, generated (or taken
    from ``inputs``) once in this process and published to shared memory -> {batch key: descriptor}."""
    from autotune.runner.benchmark import generate_tensors

    published: dict[str, dict] = {}
    for kd in accepted:
        try:
            key = batch_key(kd)
        except Exception:  # noqa: BLE001 - a candidate that does not parse fails in its worker, as a row
            continue
        if key in published:
            continue
        if inputs is not None:
            tensors = {n: inputs[n] for n in kd["tensor_specs"]}
        else:
            tensors = generate_tensors(kd["tensor_specs"], seed)
        published[key] = shared.publish(tensors)
    return published


def _visible_devices(n_detected: int) -> list[str]:
    env = os.environ.get("CUDA_VISIBLE_DEVICES")
    if env:
        return [d.strip() for d in env.split(",") if d.strip()][:n_detected]
    return [str(i) for i in range(n_detected)]


def retime_top_k(
    results: list[ProfileResult],
    items: list[dict],
    k: int,
    opts: dict,
    device: str | None,
    deadline_s: float,
    worker: Callable = None,
    startup_s: float | None = None,
) -> list[ProfileResult]:
    """Time the ``k`` fastest candidates of a sharded sweep again, all on one GPU.

    A sweep sharded over several GPUs ranks candidates that were timed on different devices, and
    GPUs of one node differ by several percent under their power caps.  The fastest ``k`` rows are
    run again by one worker on ``device``; a row that succeeds again keeps its first timing as
    ``first_pass_total_time`` / ``first_pass_mfu_estimated_percent`` and takes the new figures, so
    the final order among the leaders comes from one device.  Rows that fail the second time keep
    their first result.
    """
    def ok_time(r: ProfileResult):
        t = (r.profiler_summary or {}).get("total_time")
        return t if isinstance(t, (int, float)) and t > 0 else None

    ranked = sorted((r for r in results if ok_time(r) is not None), key=ok_time)[: max(0, k)]
    if not ranked:
        return results
    by_name = {it["kernel_name"]: it for it in items}
    again = [by_name[r.kernel_name] for r in ranked if r.kernel_name in by_name]
    kwargs = {} if startup_s is None else {"startup_s": startup_s}
    second = run_sharded([again], worker or gpu_shard_worker, opts, [device], deadline_s, **kwargs)
    new_by_name = {r.kernel_name: r for r in second if ok_time(r) is not None}
    out = []
    for r in results:
        n = new_by_name.get(r.kernel_name)
        if n is None:
            out.append(r)
            continue
        summary = dict(n.profiler_summary)
        summary["first_pass_total_time"] = r.profiler_summary["total_time"]
        summary["first_pass_mfu_estimated_percent"] = r.profiler_summary.get("mfu_estimated_percent")
        summary["retimed_on_one_gpu"] = True
        out.append(ProfileResult(n.kernel_name, n.hardware_output, summary, n.profile_detailed, n.neff_b64, n.ntff_b64))
    return out


def run_pipeline(
    kernels: dict[str, KernelJob],
    seed: int,
    collect_compiler_logs: bool,
    collect_detailed_profile: bool,
    n_gpus: int | None = None,
    warmup: int = 10,
    iters: int = 50,
    deadline_s: float = DEFAULT_DEADLINE_S,
    shard: tuple[int, int] | None = None,
    retime_top: int = 0,
    inputs: dict | None = None,
    keep_workers: bool = False,
) -> tuple[list[ProfileResult], dict[str, str]]:
    """Validate + time every candidate; returns ``(results, compiler_logs)``.

    ``keep_workers``: the per-GPU worker processes of the sweep stay alive for the next call of
    this process (see ``run_sharded``); the sweep then runs in worker processes even on one GPU.

    ``inputs``: input arrays by tensor name that the caller already holds (they must be what the
    seed and specs would give); the sweep then generates nothing.  Without it the tensors are
    generated from the seed once, in this process, and reach the worker processes through
    shared memory.

    ``retime_top`` > 0: after a sweep sharded over several GPUs by this process, the fastest
    ``retime_top`` candidates are timed again on the first GPU (see ``retime_top_k``).

    ``shard=(rank, world)`` is for callers that already run one process per GPU (for example
    under ``torchrun``): this process times only accepted candidates ``rank, rank+world, ...``
    on its current device and returns their rows (rank 0 also returns the rejected ones); the
    caller gathers the per-rank lists on the host.

    ``n_gpus`` (or the environment variable ``B200_AUTOTUNE_GPUS``) caps the number of GPUs
    used; the default is every visible GPU.  With one GPU the shard runs in this process.
    """
    from autotune.runner.detect import detect_gpus

    lncs = {int(job.lnc) for job in kernels.values()}
    if len(lncs) > 1:
        raise RuntimeError(f"Batch mixes lnc values {lncs}; submit one lnc per profile() call")
    if not kernels:
        return [], {}

    first_job = next(iter(kernels.values()))
    work_dir = Path(tempfile.mkdtemp(prefix=f"autotune-{first_job.func_name}-"))
    nki_dir = work_dir / "nki"
    log_dir = work_dir / "log"
    nki_dir.mkdir()
    log_dir.mkdir()
    try:
        detected = detect_gpus()
        want = n_gpus if n_gpus is not None else int(os.environ.get("B200_AUTOTUNE_GPUS", "0") or 0)
        n_use = min(detected, want) if want > 0 else detected
        logger.info("Driver ready: %d kernels, %d CPU, %d/%d GPU", len(kernels), os.cpu_count() or 1, n_use, detected)

        prepared = {k: _prepare_kernel(k, job, nki_dir) for k, job in kernels.items()}

        compile_results: list[CompileResult] = []
        compile_errors: list[ProfileResult] = []
        accepted: list[dict] = []
        for kname, kd in prepared.items():
            shapes = {n: tuple(s["shape"]) for n, s in kd["tensor_specs"].items()}
            stem_dir = log_dir / Path(kname).stem
            stem_dir.mkdir(parents=True, exist_ok=True)
            cr = compile_one(
                kname, kd["nki_path"], kd["func_name"], shapes, kd["input_dtype_name"], kd["output_shape"],
                log_path=str(stem_dir / "log-neuron-cc.txt"),
            )
            compile_results.append(cr)
            if cr.error:
                compile_errors.append(compile_failure_result(cr))
            else:
                accepted.append(kd)

        opts = {"seed": seed, "warmup": warmup, "iters": iters, "detailed": collect_detailed_profile,
                "inputs": inputs}
        hw_results: list[ProfileResult] = []
        if shard is not None:
            rank, world = shard
            accepted = accepted[rank::world]
            if rank != 0:
                compile_errors = []
            n_use = 1
        if accepted:
            if n_use <= 1 and not (keep_workers and shard is None):
                gpu_shard_worker(accepted, opts, hw_results.append)
            else:
                shared = SharedInputs()
                try:
                    opts["shared_inputs"] = _publish_inputs(shared, accepted, seed, inputs)
                    opts["inputs"] = None  # the arrays travel as shared-memory names, not through pickles
                    shards = shard_round_robin(accepted, n_use)
                    devices = _visible_devices(n_use)
                    hw_results = run_sharded(shards, gpu_shard_worker, opts, devices, deadline_s, keep_workers=keep_workers)
                    if retime_top > 0:
                        hw_results = retime_top_k(hw_results, accepted, retime_top, opts, devices[0], deadline_s)
                finally:
                    shared.close()

        logs: dict[str, str] = {}
        if collect_compiler_logs:
            for cr in compile_results:
                p = log_dir / Path(cr.kernel_name).stem / "log-neuron-cc.txt"
                if p.exists():
                    logs[cr.kernel_name] = p.read_text()
        return compile_errors + hw_results, logs
    finally:
        shutil.rmtree(work_dir, ignore_errors=True)
