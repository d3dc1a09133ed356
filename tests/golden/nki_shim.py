"""numpy stand-in for the third-party ``nki`` package, used ONLY to generate golden vectors.

The reference's hand kernels (``kernel_library/*``) and its fp32 simulator wrapper
(``nkigym/src/nkigym/synthesis/simulate_nki.py``) call ``nki.isa`` / ``nki.language``, which are
not part of the reference tree and are not installed here.  This module provides the handful
of names those files use, with the semantics the reference's own per-op ``_run`` methods give
them (``nkigym/src/nkigym/ops/*.py``): every ``nisa.*`` call is one numpy statement on array
views.  It is test infrastructure for ``make_golden.py`` and is never imported by the package.
"""

from __future__ import annotations

import sys
import types

import numpy as np


def install() -> None:
    """Register ``nki``, ``nki.isa`` and ``nki.language`` in ``sys.modules``."""
    if "nki" in sys.modules:
        return
    import ml_dtypes

    nki = types.ModuleType("nki")
    nisa = types.ModuleType("nki.isa")
    nl = types.ModuleType("nki.language")

    class _Jit:
        def __init__(self, func):
            self.func = func
            self.__name__ = func.__name__
            self.__wrapped__ = func

        def __call__(self, *a, **k):
            return self.func(*a, **k)

    nki.jit = _Jit
    nki.simulate = lambda f: (f.func if hasattr(f, "func") else f)

    # language: dtypes, buffers, elementwise function handles
    nl.float32 = np.float32
    nl.bfloat16 = ml_dtypes.bfloat16
    nl.float16 = np.float16
    nl.sbuf, nl.psum, nl.shared_hbm, nl.hbm = "sbuf", "psum", "shared_hbm", "hbm"
    nl.ndarray = lambda shape, dtype, buffer=None, **_: np.zeros(shape, dtype=dtype)
    nl.full = lambda shape, value, dtype, **_: np.full(shape, value, dtype=dtype)
    nl.add, nl.multiply, nl.subtract = np.add, np.multiply, np.subtract
    nl.square = np.square
    nl.rsqrt = lambda x: 1.0 / np.sqrt(x)
    nl.copy = lambda x: x

    def _assign(dst, value):
        dst[...] = np.asarray(value).astype(dst.dtype, copy=False)

    def dma_copy(dst, src, **_):                     # ops/load.py:32-35
        _assign(dst, src)

    def dma_transpose(dst, src, **_):                # ops/dma_transpose.py:40-42
        _assign(dst, np.asarray(src).T)

    def nc_transpose(dst, data, **_):                # ops/transpose.py:38-40
        _assign(dst, np.asarray(data).T)

    def memset(dst, value, **_):                     # ops/memset.py:28-33
        dst[...] = value

    def tensor_copy(dst, src, **_):                  # ops/tensor_copy.py:31-33
        _assign(dst, src)

    def nc_matmul(dst, stationary, moving, **_):     # ops/matmul.py:43-45, accumulates into dst
        prod = np.asarray(stationary).astype(np.float32).T @ np.asarray(moving).astype(np.float32)
        _assign(dst, dst.astype(np.float32) + prod)

    def tensor_tensor(dst, data1, data2, op, **_):   # kernel_hand_90.92mfu.py:93-98
        _assign(dst, op(np.asarray(data1).astype(np.float32), np.asarray(data2).astype(np.float32)))

    def tensor_scalar(dst, data, op0, operand0, **_):  # ops/tensor_scalar.py:48-53
        _assign(dst, op0(np.asarray(data).astype(np.float32), np.asarray(operand0, dtype=np.float32)))

    def activation(dst, op, data, scale=1.0, bias=0.0, **_):  # ops/activation.py:58-64
        _assign(dst, op(np.asarray(data).astype(np.float32) * scale + bias))

    def activation_reduce(dst, op, data, reduce_op, reduce_res, **_):  # ops/activation_reduce.py:96-100
        act = op(np.asarray(data).astype(np.float32))
        _assign(dst, act)
        assert reduce_op is np.add
        _assign(reduce_res, act.sum(axis=1, keepdims=True))

    def reciprocal(dst, data, **_):                  # 1/inf = 0 (kernel_hand_online.py:236-249)
        with np.errstate(divide="ignore"):
            _assign(dst, 1.0 / np.asarray(data).astype(np.float32))

    def scalar_tensor_tensor(dst, data, op0, operand0, op1, operand1, **_):  # kernel_hand_online.py:184-192
        first = op0(np.asarray(data).astype(np.float32), np.asarray(operand0, dtype=np.float32))
        _assign(dst, op1(first, np.asarray(operand1).astype(np.float32)))

    def tensor_reduce(dst, op, data, axis, **_):     # ops/tensor_reduce.py:37-40
        _assign(dst, op.reduce(np.asarray(data).astype(np.float32), axis=axis, keepdims=True))

    for fn in (dma_copy, dma_transpose, nc_transpose, memset, tensor_copy, nc_matmul, tensor_tensor,
               tensor_scalar, activation, activation_reduce, reciprocal, scalar_tensor_tensor, tensor_reduce):
        setattr(nisa, fn.__name__, fn)

    nki.isa, nki.language = nisa, nl
    sys.modules.update({"nki": nki, "nki.isa": nisa, "nki.language": nl})
