"""CPU tests of the oracles: the C restatement against the committed golden vectors
(produced by the unmodified reference x86 backend), against a float64 numpy statement of
the definition, and -- where it is present -- against the reference library itself."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402
import oracle  # noqa: E402
from golden.make_golden import golden_cases, SAMPLE_STRIDE  # noqa: E402

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))

pytestmark = pytest.mark.skipif(not oracle.port_available(), reason="oracle/libkron_oracle.so not built")


def check_against_golden(cid, z, mm, dt):
    flat = np.asarray(z).reshape(-1)
    if cid + "/full" in GOLDEN:
        ref = GOLDEN[cid + "/full"]
        got = flat
    else:
        ref = GOLDEN[cid + "/sample"]
        got = flat[::SAMPLE_STRIDE]
    scale = max(float(np.abs(ref).max()), 1e-30)
    err = float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()) / scale
    assert err <= cases.TOL[dt], (cid, err)
    s = GOLDEN[cid + "/sum"]
    assert abs(flat.astype(np.float64).sum() - s[0]) <= cases.TOL[dt] * max(s[1], 1.0), cid


def test_golden_file_lists_every_case():
    names = set(GOLDEN["names"].tolist())
    assert names == {cases.case_id(c) for c in golden_cases()}


@pytest.mark.parametrize("c", golden_cases(), ids=cases.case_id)
def test_port_matches_reference_golden(c):
    x, fs, y = cases.operands(c)
    z = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    check_against_golden(cases.case_id(c), z, c["mm"], c["dt"])


SMALL = [c for c in cases.sweep_cases() if np.prod(c["ps"], dtype=object) * c["M"] <= 1 << 16][::2]


@pytest.mark.parametrize("c", SMALL, ids=cases.case_id)
def test_port_matches_definition(c):
    x, fs, y = cases.operands(c)
    z = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    zd = oracle.numpy_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    assert cases.row_rel_err(z, zd, c["mm"]) <= cases.TOL[c["dt"]] * 0.1


def test_port_intermediates_chain():
    """Forward intermediates: applying the remaining factors to intermediate i reproduces Z."""
    c = cases.case("mkm", "f64", 3, [4, 3, 5], [2, 6, 3], seed=7)
    x, fs, _ = cases.operands(c)
    z, inter = oracle.port_gekmm("mkm", x, fs, c["ps"], c["qs"], 3, want_intermediates=True)
    # intermediate 1 = after factor 2 only; rotate-layout: applying [F0,F1] to it as a 2-factor
    # problem whose leading "identity" columns are the already produced q's is not a plain
    # GeMKM, so check sizes and the last step instead: Z = step(inter[0], F0)
    assert inter[0].shape == (3, 4 * 6 * 3) and inter[1].shape == (3, 4 * 3 * 3)
    P, Q = 4, 2
    S = inter[0].shape[1] // P
    F0 = fs[0].reshape(P, Q)
    want = np.einsum("msp,pq->mqs", inter[0].reshape(3, S, P), F0).reshape(3, -1)
    assert np.allclose(want, z, rtol=0, atol=1e-12)


@pytest.mark.skipif(not oracle.ref_available(), reason="oracle/_ref/libFastKron.so not built here")
@pytest.mark.parametrize("c", cases.MINI_CONFIGS, ids=cases.case_id)
def test_port_matches_live_reference(c):
    x, fs, y = cases.operands(c)
    z = oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    zr = oracle.ref_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
    assert cases.row_rel_err(z, zr, c["mm"]) <= cases.TOL[c["dt"]] * 0.1
