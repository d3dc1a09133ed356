"""The allocation-free entry point against the regular one (GPU box only; collected last).

Callers that cannot allocate device memory where the call is made -- a serving engine that gave
the whole device heap to its own pools, a thread that must not touch the allocator -- use
``b200_rmsnorm_matmul_noalloc``: same skinny fused kernel, scratch inside the library.  Two calls
in a row must both match the workspace-based entry point (the second one runs on whatever the
first left in the shared array).
"""

import ctypes as C

import ml_dtypes
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu
TOL_BF16 = 1e-2


def test_noalloc_entry_matches_workspace_entry_twice_in_a_row(native_lib):
    import torch

    from autotune import kernels, native

    lib = native.load()
    m, k, n = 16, 2048, 3080
    t = O.generate_inputs(31, [("x", (m, k), None), ("gamma", (k,), {"kind": "uniform", "low": 0.5, "high": 1.5}),
                               ("weight", (k, n), {"kind": "normal", "scale": k ** -0.5})], bf16=True)
    x, g, w = (kernels.to_device(t[name].astype(ml_dtypes.bfloat16)) for name in ("x", "gamma", "weight"))
    expect = O.rmsnorm_matmul(t["x"], t["gamma"], t["weight"], 1e-5)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        ref = kernels.rmsnorm_matmul(x, g, w, eps=1e-5)                      # existing entry point, caller workspace
        out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        status = kernels.new_status()
        torch.cuda.synchronize()
        # free device memory as the driver sees it: an allocation made inside the library (which
        # torch's own counters cannot see) would show up here.  The first call may still load the
        # kernel's module lazily, so the comparison is made on the second, warm call.
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.b200_rmsnorm_matmul_noalloc(x.data_ptr(), g.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                                             C.c_float(1e-5), None, status.data_ptr(), stream)
        assert rc == native.OK, native.last_error()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        if call == 1:
            assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
        kernels.raise_on_status(status)
        a = kernels.to_host(out).astype(np.float32)
        r = kernels.to_host(ref).astype(np.float32)
        assert O.max_abs_rel_err(a, r) <= TOL_BF16, f"call {call}: differs from the workspace entry point"
        assert O.max_abs_rel_err(a, expect) <= TOL_BF16, f"call {call}: differs from the CPU oracle"


def test_noalloc_entry_rejects_sizes_beyond_its_scratch(native_lib):
    import torch

    from autotune import native

    lib = native.load()
    z = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.b200_rmsnorm_matmul_noalloc(z.data_ptr(), None, z.data_ptr(), z.data_ptr(), 16, 32768 + 8, 64,
                                         C.c_float(1e-5), None, None, stream)
    assert rc == native.ERR_BAD_SHAPE and "exceeds the built-in scratch" in native.last_error()
    rc = lib.b200_rmsnorm_matmul_noalloc(z.data_ptr(), None, z.data_ptr(), z.data_ptr(), 17, 256, 64,
                                         C.c_float(1e-5), None, None, stream)
    assert rc == native.ERR_BAD_SHAPE and "rows" in native.last_error()
