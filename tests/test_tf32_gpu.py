"""Opt-in TF32 tensor-core path (fastKronOptionsTF32, not in the reference).

fp32 passes with 64x64 / 128x128 factors run through tcgen05.mma.kind::tf32: operands are read
with a 10-bit mantissa, sums are fp32.  The tolerance is this path's own:
max |z - ref| / max|ref row| <= 5e-3 (the default fp32 path is held to 1e-4).  Each case is
built so that the only large factor pass hits one tile mode of the kernel (contiguous
contraction index; trailing extent 32, 64, a multiple of 128; ragged last tiles), the other
factors being small ones that stay on the exact fp32 kernels; an error above 1e-6 shows that
the tensor-core kernel really ran, and its bounded barrier waits must never have given up."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu

TF32_TOL = 5e-3
OPT_USE_FUSION, OPT_TF32 = 2, 8


@pytest.fixture(scope="module")
def h():
    import fastkron_b200
    hd = fastkron_b200.FastKron()
    hd.set_options(OPT_USE_FUSION | OPT_TF32)
    yield hd
    hd.close()


TF32_CASES = [
    # contiguous contraction index (trailing extent 1), whole and ragged tiles
    cases.case("mkm", "f32", 16, [32, 64], [32, 64], seed=901),
    cases.case("mkm", "f32", 3, [32, 64], [32, 64], seed=902),
    cases.case("mkm", "f32", 5, [16, 128], [16, 128], seed=903),
    # trailing extent 32 and 64: four / two chunks per tile, ragged
    cases.case("mkm", "f32", 6, [64, 32], [64, 32], seed=904),
    cases.case("mkm", "f32", 5, [64, 64], [64, 64], seed=905),
    cases.case("mkm", "f32", 3, [128, 32], [128, 32], seed=906),
    # trailing extent a multiple of 128
    cases.case("mkm", "f32", 4, [64, 16, 8], [64, 16, 8], seed=907),
    cases.case("mkm", "f32", 4, [64, 64, 64], [64, 64, 64], seed=908),
    cases.case("mkm", "f32", 3, [128, 128], [128, 128], seed=909),
    cases.case("mkm", "f32", 2, [128, 16, 16], [128, 16, 16], seed=910),
    # epilogue on a tensor-core pass, transposed factors, KMM
    cases.case("mkm", "f32", 8, [64, 64], [64, 64], "N", "T", 2.0, 0.5, seed=911),
    cases.case("kmm", "f32", 128, [64, 64], [64, 64], "N", "N", 1.5, 1.0, seed=912),
    cases.case("mkm", "f32", 32, [64, 64, 64], [64, 64, 64], seed=913),
]


@pytest.mark.parametrize("c", TF32_CASES, ids=cases.case_id)
def test_tf32_option_within_its_tolerance(h, c):
    import gpu_util
    from fastkron_b200 import lib as fk
    x, fs, y = cases.operands(c)
    z = gpu_util.run_case(h, c, x=x, fs=fs, y=y)
    want = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    err = cases.row_rel_err(z, want, c["mm"])
    assert fk.get().fkbGemmTcTimeouts() == 0
    assert err <= TF32_TOL, err
    assert err > 1e-6, "result is fp32-exact: the tensor-core kernel did not run"


def test_tf32_is_off_by_default():
    import fastkron_b200
    import gpu_util
    hd = fastkron_b200.FastKron()
    try:
        c = cases.case("mkm", "f32", 8, [64, 64], [64, 64], seed=920)
        x, fs, y = cases.operands(c)
        z = gpu_util.run_case(hd, c, x=x, fs=fs, y=y)
        want = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
        assert cases.row_rel_err(z, want, c["mm"]) <= cases.TOL["f32"]
    finally:
        hd.close()


# ---- split TF32 (fastKronOptionsTF32x3): three tensor-core products per fp32 product -----------

TF32X3_TOL = 1e-5      # of the row maximum; observed a few 1e-7 to 2e-6
OPT_TF32X3 = 16

X3_CASES = [
    cases.case("mkm", "f32", 16, [32, 64], [32, 64], seed=931),                  # contraction index contiguous
    cases.case("mkm", "f32", 3, [32, 64], [32, 64], seed=932),                   # ragged tile
    cases.case("mkm", "f32", 6, [64, 32], [64, 32], seed=933),                   # trailing extent 32
    cases.case("mkm", "f32", 5, [64, 64], [64, 64], seed=934),                   # trailing extent 64 and 1
    cases.case("mkm", "f32", 4, [64, 16, 8], [64, 16, 8], seed=935),             # trailing extent 128
    cases.case("mkm", "f32", 4, [64, 64, 64], [64, 64, 64], seed=936),
    cases.case("mkm", "f32", 8, [64, 64], [64, 64], "N", "T", 2.0, 0.5, seed=937),
    cases.case("kmm", "f32", 128, [64, 64], [64, 64], "N", "N", 1.5, 1.0, seed=938),
    cases.case("mkm", "f32", 40, [64, 64, 64], [64, 64, 64], seed=939),          # several tiles per CTA: ring wraps
]


@pytest.mark.parametrize("c", X3_CASES, ids=cases.case_id)
def test_split_tf32_option_matches_fp32(c):
    import fastkron_b200
    import gpu_util
    from fastkron_b200 import lib as fk
    hd = fastkron_b200.FastKron()
    hd.set_options(OPT_USE_FUSION | OPT_TF32X3)
    try:
        before = fk.get().fkbGemmTcLaunches(1)
        x, fs, y = cases.operands(c)
        z = gpu_util.run_case(hd, c, x=x, fs=fs, y=y)
        want = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
        err = cases.row_rel_err(z, want, c["mm"])
        assert fk.get().fkbGemmTcTimeouts() == 0
        assert fk.get().fkbGemmTcLaunches(1) > before, "the split tensor-core kernel did not run"
        assert err <= TF32X3_TOL, err
    finally:
        hd.close()
