"""ctypes binding of ``libb200_autotune.so`` (C ABI declared in ``include/b200_autotune.h``).

There is no CPU fallback: :func:`load` raises when the library is missing, and every
wrapper raises :class:`NativeError` on a non-zero status.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent
LIB_PATH = PKG_ROOT / "lib" / "libb200_autotune.so"

OK = 0
ERR_BAD_ARG, ERR_BAD_SHAPE, ERR_UNSUPPORTED, ERR_SMEM_OOM, ERR_TMEM_OOM = 1, 2, 3, 4, 5
ERR_CUDA, ERR_DEVICE_WAIT, ERR_WORKSPACE = 6, 7, 8
DEV_STATUS_INTS = 8

CFG_FIELDS = ("tile_m", "tile_n", "tile_k", "stages", "cluster_m", "cluster_n", "swizzle", "split_k", "norm_mode")


class Cfg(C.Structure):
    """``b200_cfg``."""

    _fields_ = [(name, C.c_int) for name in CFG_FIELDS] + [("reserved", C.c_int * 7)]

    @classmethod
    def from_dict(cls, d: dict | None) -> "Cfg | None":
        if d is None:
            return None
        cfg = cls()
        for name in CFG_FIELDS:
            setattr(cfg, name, int(d.get(name, 0)))
        if d.get("cluster_m", 0) == 0:
            cfg.cluster_m = 1
        if d.get("cluster_n", 0) == 0:
            cfg.cluster_n = 1
        cfg.reserved[0] = int(d.get("_debug_mode", d.get("_debug_skip_producer", 0)))
        cfg.reserved[1] = int(d.get("_wait_limit_us", 0))
        cfg.reserved[2] = int(d.get("_record_clocks", 0))
        cfg.reserved[3] = int(d.get("_max_ctas", 0))
        cfg.reserved[4] = int(d.get("_serial_launch", 0))
        return cfg


class Problem(C.Structure):
    """``b200_problem``."""

    _fields_ = [
        ("family", C.c_char_p),
        ("a", C.c_void_p),
        ("b", C.c_void_p),
        ("gamma", C.c_void_p),
        ("out", C.c_void_p),
        ("M", C.c_long),
        ("N", C.c_long),
        ("K", C.c_long),
        ("ld_a", C.c_long),
        ("ld_b", C.c_long),
        ("ld_out", C.c_long),
        ("eps", C.c_float),
        ("reserved", C.c_int * 7),
    ]


class NativeError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[b200 status {code}] {message}")
        self.code = code
        self.message = message


_lib: C.CDLL | None = None

# symbol -> (restype, argtypes); must list every function the header declares
SIGNATURES = {
    "b200_last_error": (C.c_char_p, []),
    "b200_abi_version": (C.c_int, []),
    "b200_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "b200_cfg_check": (
        C.c_int,
        [C.c_char_p, C.POINTER(Cfg), C.c_long, C.c_long, C.c_long, C.POINTER(C.c_long), C.POINTER(C.c_int)],
    ),
    "b200_describe_launch": (C.c_int, [C.c_char_p, C.POINTER(Cfg), C.c_long, C.c_long, C.c_long, C.c_char_p, C.c_size_t]),
    "b200_checked_build_report": (C.c_int, [C.POINTER(C.c_longlong), C.c_int]),
    "b200_ipc_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "b200_ipc_close": (C.c_int, [C.c_void_p]),
    "b200_peer_store": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int, C.c_void_p]),
    "b200_default_cfg": (C.c_int, [C.c_char_p, C.c_long, C.c_long, C.c_long, C.POINTER(Cfg)]),
    "b200_workspace_bytes": (C.c_size_t, [C.c_char_p, C.POINTER(Cfg), C.c_long, C.c_long, C.c_long]),
    "b200_matmul_lhsT_rhs": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long,
         C.POINTER(Cfg), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "b200_matmul_lhs_rhs": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long,
         C.POINTER(Cfg), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "b200_matmul_lhsT_rhs_f32": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long, C.c_long, C.c_void_p],
    ),
    "b200_rmsnorm_matmul": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_float,
         C.POINTER(Cfg), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p],
    ),
    "b200_rmsnorm_matmul_noalloc": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_float,
         C.POINTER(Cfg), C.c_void_p, C.c_void_p],
    ),
    "b200_rmsnorm_matmul_f32": (
        C.c_int,
        [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_long, C.c_long, C.c_long, C.c_float, C.c_void_p],
    ),
    "b200_time_kernel": (
        C.c_int,
        [C.POINTER(Problem), C.POINTER(Cfg), C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_size_t,
         C.c_int, C.c_int, C.POINTER(C.c_float), C.c_void_p],
    ),
}


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        path = os.environ.get("B200_AUTOTUNE_LIB", str(LIB_PATH))
        if not os.path.isfile(path):
            raise NativeError(
                -1,
                f"{path} not found: build it with `python {PKG_ROOT / 'build.py'}` "
                "(there is no CPU fallback for the kernels)",
            )
        lib = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    msg = load().b200_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int) -> None:
    if status != OK:
        raise NativeError(status, last_error())


def default_cfg(family: str, M: int, N: int, K: int) -> dict:
    """The candidate the library picks for this family and shape when no cfg is given."""
    c = Cfg()
    check(load().b200_default_cfg(family.encode(), M, N, K, C.byref(c)))
    return {name: int(getattr(c, name)) for name in CFG_FIELDS}


def cfg_check(family: str, cfg: dict | None, M: int = 0, N: int = 0, K: int = 0) -> tuple[int, str, int, int]:
    """Validate a candidate without a GPU -> (status, message, smem_bytes, tmem_cols)."""
    lib = load()
    smem = C.c_long(0)
    tmem = C.c_int(0)
    c = Cfg.from_dict(cfg)
    status = lib.b200_cfg_check(family.encode(), C.byref(c) if c is not None else None, M, N, K,
                                C.byref(smem), C.byref(tmem))
    return status, (last_error() if status else ""), smem.value, tmem.value


def describe_launch(family: str, cfg: dict | None, M: int, N: int, K: int) -> dict:
    """The launch plan of a candidate at a shape (kernel variant, grid, shared / tensor memory, waves,
    UMMA-bound cycles, registers); nothing is launched."""
    import json

    buf = C.create_string_buffer(2048)
    c = Cfg.from_dict(cfg)
    check(load().b200_describe_launch(family.encode(), C.byref(c) if c is not None else None, M, N, K, buf, len(buf)))
    return json.loads(buf.value.decode())


CHECK_CODES = {1: "shared-memory range", 2: "barrier address", 3: "TMA load", 4: "TMA store", 5: "tensor-memory address",
               6: "global index", 7: "schedule index"}


def checked_build_report(clear: bool = True, selftest: bool = False) -> dict | None:
    """The device-side check record of the checked build (``libb200_autotune_checked.so``, selected
    with ``B200_AUTOTUNE_LIB``); ``None`` when the loaded library is the normal one.  Synchronises
    the device.  ``{"failures": n, "code": ..., "what": ..., "line": ..., "value": ..., "limit": ...}``."""
    out = (C.c_longlong * 4)()
    status = load().b200_checked_build_report(out, (1 if clear else 0) | (2 if selftest else 0))
    if status == ERR_UNSUPPORTED:
        return None
    check(status)
    code, line = int(out[1]) >> 32, int(out[1]) & 0xFFFFFFFF
    return {"failures": int(out[0]), "code": code, "what": CHECK_CODES.get(code, ""), "line": line,
            "value": int(out[2]), "limit": int(out[3])}


def device_count() -> int:
    n = C.c_int(0)
    check(load().b200_device_count(C.byref(n)))
    return n.value
