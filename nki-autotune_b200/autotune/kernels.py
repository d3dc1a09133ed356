"""Tensor-level entry points of the hot path.

PyTorch is used for device memory and streams only; the arithmetic happens in the sm_100a
kernels of ``libb200_autotune.so`` reached through its C ABI.  Nothing here falls back to
torch or numpy arithmetic: without a GPU or without the built library the calls raise.

* :func:`matmul_lhsT_rhs` replaces ``matmul_lhsT_rhs_nkigym``
  (``kernel_library/matmul/lhsT_rhs/kernel_hand_90.92mfu.py:101-131``).
* :func:`rmsnorm_matmul` replaces ``rmsnorm_matmul_online``
  (``kernel_library/rmsnorm_matmul/kernel_hand_online.py:198-353``), with an optional gamma.
* the ``*_host`` variants take and return numpy arrays in host memory and do the copies.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from autotune import native
from autotune.native import Cfg, NativeError, Problem


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NativeError(-1, "operands must live on a CUDA device (there is no CPU path)")


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def new_status(device=None) -> torch.Tensor:
    """A zeroed device status block for the bounded-wait diagnostics."""
    return torch.zeros(native.DEV_STATUS_INTS, dtype=torch.int32, device=device or "cuda")


def raise_on_status(status: torch.Tensor) -> None:
    """Read a status block back (synchronises) and raise if a device-side wait expired."""
    host = status.cpu().tolist()
    if host[0] != 0:
        reset_workspaces()
        raise NativeError(
            native.ERR_DEVICE_WAIT,
            f"device-side wait expired: role {host[1]} barrier {host[2]} tile {host[3]} "
            f"k-block {host[4]} CTA {host[5]}",
        )


_WORKSPACES: dict[tuple, torch.Tensor] = {}


def workspace_for(family: str, M: int, N: int, K: int, device, cfg: dict | None = None) -> torch.Tensor | None:
    """Device scratch for the kernels that use it (``None`` when they do not).

    The buffers are zero-filled once; the kernels leave them reusable (partial sums and
    barrier counters back at zero), so one cached buffer per (device, kind, size) serves every
    launch.  :func:`reset_workspaces` drops the cache after a failed launch.
    """
    c = Cfg.from_dict(cfg)
    need = native.load().b200_workspace_bytes(family.encode(), C.byref(c) if c is not None else None, M, N, K)
    if need == 0:
        return None
    dev = torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    kind = "split_k" if family != "rmsnorm_matmul" else ("skinny" if M <= 16 else "prologue")
    key = (index, kind, int(need))
    buf = _WORKSPACES.get(key)
    if buf is None:
        buf = torch.zeros(int(need), dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = buf
    return buf


def reset_workspaces() -> None:
    """Forget cached scratch buffers (their contents are undefined after an aborted launch)."""
    _WORKSPACES.clear()


def _ld(t: torch.Tensor) -> int:
    if t.dim() != 2 or t.stride(1) != 1:
        raise NativeError(native.ERR_BAD_SHAPE, "operands must be 2-D with a unit inner stride")
    return t.stride(0) if t.shape[0] > 1 else t.shape[1]


def matmul_lhsT_rhs(
    lhs_T: torch.Tensor,
    rhs: torch.Tensor,
    cfg: dict | None = None,
    out: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> torch.Tensor:
    """``lhs_T.T @ rhs`` for ``lhs_T[K, M]`` and ``rhs[K, N]``.

    bf16 operands run on the tcgen05 kernel (fp32 accumulation, bf16 result); fp32 operands
    run on the fp32 CUDA-core kernel (fp32 result).  ``cfg`` is a dict of meta-parameters
    (``tile_m``, ``tile_n``, ``tile_k``, ``stages``, ``cluster_m``, ``swizzle``) or ``None``
    for the default.  Asynchronous on the current stream.
    """
    _require_cuda(lhs_T, rhs)
    lib = native.load()
    K, M = lhs_T.shape
    K2, N = rhs.shape
    if K != K2:
        raise NativeError(native.ERR_BAD_SHAPE, f"contraction mismatch: lhs_T has K={K}, rhs has K={K2}")
    if lhs_T.dtype != rhs.dtype:
        raise NativeError(native.ERR_BAD_ARG, "operand dtypes differ")
    if out is None:
        out = torch.empty((M, N), dtype=lhs_T.dtype, device=lhs_T.device)
    if lhs_T.dtype == torch.float32:
        native.check(
            lib.b200_matmul_lhsT_rhs_f32(
                lhs_T.data_ptr(), rhs.data_ptr(), out.data_ptr(), M, N, K, _ld(lhs_T), _ld(rhs), _ld(out),
                _stream_ptr(),
            )
        )
        return out
    if lhs_T.dtype != torch.bfloat16:
        raise NativeError(native.ERR_BAD_ARG, f"unsupported dtype {lhs_T.dtype}")
    c = Cfg.from_dict(cfg)
    ws = workspace_for("matmul_lhsT_rhs", M, N, K, lhs_T.device, cfg)  # split-K candidates only
    native.check(
        lib.b200_matmul_lhsT_rhs(
            lhs_T.data_ptr(), rhs.data_ptr(), out.data_ptr(), M, N, K, _ld(lhs_T), _ld(rhs), _ld(out),
            C.byref(c) if c is not None else None,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status.data_ptr() if status is not None else None, _stream_ptr(),
        )
    )
    return out


def matmul_lhs_rhs(
    lhs: torch.Tensor,
    rhs: torch.Tensor,
    cfg: dict | None = None,
    out: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> torch.Tensor:
    """``lhs @ rhs`` for bf16 ``lhs[M, K]`` (K contiguous) and ``rhs[K, N]``: replaces
    ``matmul_lhs_rhs_nkigym`` (``kernel_library/matmul/lhs_rhs/kernel_handtuned_89.26mfu.py:226-287``)."""
    _require_cuda(lhs, rhs)
    lib = native.load()
    M, K = lhs.shape
    K2, N = rhs.shape
    if K != K2:
        raise NativeError(native.ERR_BAD_SHAPE, f"contraction mismatch: lhs has K={K}, rhs has K={K2}")
    if lhs.dtype != torch.bfloat16 or rhs.dtype != torch.bfloat16:
        raise NativeError(native.ERR_BAD_ARG, "matmul_lhs_rhs: bf16 operands only")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=lhs.device)
    c = Cfg.from_dict(cfg)
    ws = workspace_for("matmul_lhs_rhs", M, N, K, lhs.device, cfg)  # split-K candidates only
    native.check(
        lib.b200_matmul_lhs_rhs(
            lhs.data_ptr(), rhs.data_ptr(), out.data_ptr(), M, N, K, _ld(lhs), _ld(rhs), _ld(out),
            C.byref(c) if c is not None else None,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status.data_ptr() if status is not None else None, _stream_ptr(),
        )
    )
    return out


def rmsnorm_matmul(
    x: torch.Tensor,
    gamma: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float = 1e-6,
    cfg: dict | None = None,
    out: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> torch.Tensor:
    """``(x / sqrt(mean(x**2, -1) + eps) * gamma) @ weight`` for bf16 ``x[M, K]``, ``weight[K, N]``."""
    _require_cuda(x, weight, gamma)
    lib = native.load()
    M, K = x.shape
    K2, N = weight.shape
    if K != K2 or (gamma is not None and gamma.numel() != K):
        raise NativeError(native.ERR_BAD_SHAPE, "rmsnorm_matmul: K of x, gamma and weight differ")
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise NativeError(native.ERR_BAD_ARG, "rmsnorm_matmul: bf16 operands only")
    if not x.is_contiguous() or not weight.is_contiguous():
        raise NativeError(native.ERR_BAD_SHAPE, "rmsnorm_matmul: operands must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    c = Cfg.from_dict(cfg)
    ws = workspace_for("rmsnorm_matmul", M, N, K, x.device, cfg)
    native.check(
        lib.b200_rmsnorm_matmul(
            x.data_ptr(), gamma.data_ptr() if gamma is not None else None, weight.data_ptr(), out.data_ptr(),
            M, N, K, float(eps), C.byref(c) if c is not None else None,
            ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
            status.data_ptr() if status is not None else None, _stream_ptr(),
        )
    )
    return out


def rmsnorm_matmul_f32(x: torch.Tensor, gamma: torch.Tensor | None, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 CUDA-core evaluation of the fused expression on bf16 inputs (cross-check kernel)."""
    _require_cuda(x, weight, gamma)
    lib = native.load()
    M, K = x.shape
    N = weight.shape[1]
    out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    native.check(
        lib.b200_rmsnorm_matmul_f32(
            x.data_ptr(), gamma.data_ptr() if gamma is not None else None, weight.data_ptr(), out.data_ptr(),
            M, N, K, float(eps), _stream_ptr(),
        )
    )
    return out


def time_kernel(
    family: str,
    a: torch.Tensor,
    b: torch.Tensor,
    out: torch.Tensor,
    cfg: dict | None,
    gamma: torch.Tensor | None = None,
    eps: float = 0.0,
    warmup: int = 3,
    iters: int = 10,
    flush: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> list[float]:
    """Per-launch milliseconds of one candidate, measured with CUDA events inside the library."""
    _require_cuda(a, b, out)
    lib = native.load()
    if family == "matmul_lhsT_rhs":
        K, M = a.shape
    else:
        M, K = a.shape
    N = b.shape[1]
    prob = Problem()
    prob.family = family.encode()
    prob.a, prob.b, prob.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    prob.gamma = gamma.data_ptr() if gamma is not None else None
    prob.M, prob.N, prob.K = M, N, K
    prob.ld_a, prob.ld_b, prob.ld_out = _ld(a), _ld(b), _ld(out)
    prob.eps = float(eps)
    ms = (C.c_float * iters)()
    c = Cfg.from_dict(cfg)
    ws = workspace_for(family, M, N, K, a.device, cfg)
    rc = lib.b200_time_kernel(
        C.byref(prob), C.byref(c) if c is not None else None,
        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
        status.data_ptr() if status is not None else None,
        flush.data_ptr() if flush is not None else None,
        flush.numel() * flush.element_size() if flush is not None else 0,
        warmup, iters, ms, _stream_ptr(),
    )
    if rc == native.ERR_DEVICE_WAIT:
        # a launch gave up on a device-side wait: whatever scratch it used (counters, partial
        # tiles) is undefined now, and the cached buffers would poison every later candidate
        message = native.last_error()
        torch.cuda.synchronize()
        reset_workspaces()
        raise NativeError(rc, message)
    native.check(rc)
    return list(ms)


# ------------------------------------------------------------------------------- host arrays
def to_device(arr: np.ndarray, device="cuda", pinned: bool = False) -> torch.Tensor:
    """numpy (fp32 or ml_dtypes bfloat16) -> device tensor of the matching torch dtype."""
    if arr.dtype == np.float32:
        t = torch.from_numpy(np.ascontiguousarray(arr))
    elif arr.dtype.name == "bfloat16":
        t = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint16)).view(torch.bfloat16)
    else:
        raise NativeError(native.ERR_BAD_ARG, f"unsupported host dtype {arr.dtype}")
    if pinned:
        t = t.pin_memory()
    return t.to(device, non_blocking=pinned)


def to_host(t: torch.Tensor) -> np.ndarray:
    """device tensor -> numpy (bf16 comes back as ml_dtypes bfloat16)."""
    import ml_dtypes

    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).cpu().numpy().view(ml_dtypes.bfloat16)
    return t.cpu().numpy()


def matmul_lhsT_rhs_host(lhs_T: np.ndarray, rhs: np.ndarray, cfg: dict | None = None) -> np.ndarray:
    """Host arrays in, host array out: H2D copies, one kernel, D2H copy (synchronous)."""
    status = new_status()
    out = matmul_lhsT_rhs(to_device(lhs_T), to_device(rhs), cfg=cfg, status=status)
    result = to_host(out)
    raise_on_status(status)
    return result


def rmsnorm_matmul_host(
    x: np.ndarray, gamma: np.ndarray | None, weight: np.ndarray, eps: float = 1e-6, cfg: dict | None = None
) -> np.ndarray:
    """Host arrays in, host array out for the fused kernel (synchronous)."""
    status = new_status()
    g = to_device(gamma) if gamma is not None else None
    out = rmsnorm_matmul(to_device(x), g, to_device(weight), eps=eps, cfg=cfg, status=status)
    result = to_host(out)
    raise_on_status(status)
    return result
