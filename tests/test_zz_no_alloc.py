"""sgemkmNoAlloc -- the GeMKM entry point for callers that cannot allocate device memory.

Kept in a file that pytest collects last, so a failure here cannot hide the other tests in
a run that stops at the first failure.  The check: through the C ABI, the no-allocation
call must produce what sgemkm produces with caller-provided temporaries (same kernels,
same plan, so the results are compared exactly as well as against the usual tolerance),
on two calls in a row -- the second call finds the static scratch dirty from the first.
"""
import ctypes
import gc
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402

pytestmark = pytest.mark.gpu


def _call_noalloc(h, c, xd, fd, z, yd):
    from fastkron_b200 import lib as fk
    L = fk.get()
    n = len(c["ps"])
    rc = L.sgemkmNoAlloc(h.h, ctypes.c_uint32(c["M"]), ctypes.c_uint32(n), fk.u32arr(c["ps"]), fk.u32arr(c["qs"]),
                         ctypes.c_void_p(xd.data_ptr()), ctypes.c_int(1 if c["opx"] == "N" else 2),
                         fk.ptrarr([f.data_ptr() for f in fd]), ctypes.c_int(1 if c["opf"] == "N" else 2),
                         ctypes.c_void_p(z.data_ptr()), ctypes.c_float(c["alpha"]), ctypes.c_float(c["beta"]),
                         ctypes.c_void_p(yd.data_ptr() if yd is not None else 0))
    return rc


def test_no_alloc_matches_sgemkm_twice():
    import torch
    import fastkron_b200
    import gpu_util
    from fastkron_b200 import lib as fk
    h = fastkron_b200.FastKron()
    # two different problems back to back; both fit the static scratch
    problems = [cases.case("mkm", "f32", 16, [16] * 4, [16] * 4, "N", "N", 2.0, 1.0, seed=51),
                cases.case("mkm", "f32", 7, [8, 4, 32, 3], [8, 4, 32, 5], "N", "T", 1.0, 0.0, seed=52)]
    first = True
    for rep in range(2):
        for c in problems:
            x, fs, y = cases.operands(c)
            want = gpu_util.run_case(h, c, x=x, fs=fs, y=y)            # sgemkm, caller temporaries
            xd = torch.from_numpy(x).cuda()
            fd = [torch.from_numpy(f).cuda() for f in fs]
            yd = torch.from_numpy(y).cuda() if y is not None else None
            ye, te = h.sizes(c["M"], c["ps"], c["qs"])
            assert te <= fk.NOALLOC_MAX_TEMP_ELEMS
            z = torch.full((ye,), float("nan"), dtype=torch.float32, device="cuda")
            # nothing may be allocated by the call: neither through torch's allocator nor behind its
            # back (cudaMemGetInfo sees every allocation on the device).  Collect garbage first so
            # that tensors of earlier tests are not released in the middle of the measurement.
            gc.collect()
            torch.cuda.synchronize()
            before = torch.cuda.memory_allocated()
            free_before = torch.cuda.mem_get_info()[0]
            assert _call_noalloc(h, c, xd, fd, z, yd) == fk.SUCCESS
            torch.cuda.synchronize()
            assert torch.cuda.memory_allocated() == before
            # (the very first call on a device may make the driver load the module that holds the
            # static scratch -- CUDA loads modules lazily -- which is when those 16 MiB are mapped)
            if not first:
                assert torch.cuda.mem_get_info()[0] >= free_before
            first = False
            got = z.cpu().numpy().reshape(want.shape)
            assert cases.row_rel_err(got, want, "mkm") <= cases.TOL["f32"]
            assert np.array_equal(got, want)
    h.close()


def test_no_alloc_rejects_oversized_problem():
    import torch
    import fastkron_b200
    from fastkron_b200 import lib as fk
    h = fastkron_b200.FastKron()
    c = cases.case("mkm", "f32", 64, [16] * 4, [16] * 4)          # 64 * 65536 = 4 Mi > limit
    _, te = h.sizes(c["M"], c["ps"], c["qs"])
    assert te > fk.NOALLOC_MAX_TEMP_ELEMS
    d = torch.zeros(16, device="cuda")
    z = torch.zeros(16, device="cuda")
    rc = _call_noalloc(h, c, d, [d] * 4, z, None)                  # rejected before any launch
    assert rc == fk.INVALID_ARGUMENT
    torch.cuda.synchronize()
    h.close()
