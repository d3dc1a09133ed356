"""Candidate validation: the step that stands where the reference compiles.

Upstream ``compile_one`` (``autotune/src/autotune/runner/compile.py:197-244``) turns NKI source
into a NEFF inside a worker process and reports compiler failures (including on-chip memory
over-subscription) as an error string.  The B200 device code is precompiled into
``libb200_autotune.so``; what remains per candidate is parsing its descriptor and checking
its meta-parameters against the shared-memory and tensor-memory budgets.  A rejected
candidate yields ``CompileResult.error`` and later a failure row -- it is never dropped.
"""

from __future__ import annotations

from autotune import native
from autotune.runner.candidate import Candidate, parse_source
from autotune.runner.types import CompileResult, capture_error


def load_kernel(nki_path: str, func_name: str) -> Candidate:
    """Read a descriptor file and check it names ``func_name`` (reference: compile.py:26-43)."""
    with open(nki_path) as fh:
        cand = parse_source(fh.read())
    if cand.family != func_name:
        raise ValueError(f"{nki_path}: descriptor is for {cand.family!r}, job says {func_name!r}")
    return cand


def problem_dims(family: str, input_shapes: dict[str, tuple[int, ...]], output_shape: tuple[int, ...]) -> tuple[int, int, int]:
    """(M, N, K) of a job from its input shapes (first input carries K)."""
    shapes = list(input_shapes.values())
    if len(output_shape) != 2 or len(shapes) < 2:
        raise ValueError("expected two or three 2-D inputs and a 2-D output")
    M, N = output_shape
    first = shapes[0]
    K = first[0] if family == "matmul_lhsT_rhs" else first[1]
    expect_first = (K, M) if family == "matmul_lhsT_rhs" else (M, K)
    if tuple(first) != expect_first or tuple(shapes[-1]) != (K, N):
        raise ValueError(f"{family}: input shapes {shapes} do not match output {tuple(output_shape)}")
    return int(M), int(N), int(K)


def compile_one(
    kernel_name: str,
    nki_path: str,
    func_name: str,
    input_shapes: dict[str, tuple[int, ...]],
    input_dtype_name: str,
    output_shape: tuple[int, ...],
    log_path: str | None = None,
) -> CompileResult:
    """Validate one candidate; never raises (reference: compile.py:197-244)."""
    error = ""
    log_lines = [f"candidate {kernel_name} ({func_name}, {input_dtype_name})"]
    try:
        cand = load_kernel(nki_path, func_name)
        M, N, K = problem_dims(func_name, input_shapes, output_shape)
        log_lines.append(f"problem M={M} N={N} K={K}; config {cand.config}")
        if input_dtype_name == "float32":
            log_lines.append("fp32 inputs: CUDA-core kernel; tile meta-parameters do not apply to it")
        else:
            config = dict(cand.config)
            if func_name == "rmsnorm_matmul" and M > 16 and int(config.get("norm_mode", 0) or 0) == 0:
                # the timing path always hands the kernel its scratch, and with scratch the library
                # resolves norm_mode 0 to the prologue variant: validate the plan that will run
                config["norm_mode"] = 2
                log_lines.append("norm_mode 0 with scratch supplied: validated as norm_mode 2 (prologue variant)")
            status, message, smem, tmem = native.cfg_check(func_name, config, M, N, K)
            log_lines.append(f"shared memory {smem} B of 232448 B; tensor memory {tmem} of 512 columns")
            if status != native.OK:
                error = message
    except Exception as exc:  # noqa: BLE001 - every failure becomes a row
        error = capture_error(exc)
    log_lines.append("rejected: " + error if error else "accepted")
    if log_path:
        with open(log_path, "w") as fh:
            fh.write("\n".join(log_lines) + "\n")
    return CompileResult(kernel_name=kernel_name, nki_path=nki_path, neff_path=str(native.LIB_PATH), error=error)
