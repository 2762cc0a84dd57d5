"""Generate tests/golden/golden.npz from the UNMODIFIED reference x86 backend.

Run in the build container (needs oracle/_ref/libFastKron.so, see oracle/build_ref.sh):
    python tests/golden/make_golden.py
Inputs are not stored: they are pure functions of each case's seed (tests/cases.py).
Stored per case: the reference's full result for small cases, or a strided sample of it
plus its float64 checksum for larger ones.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from oracle import ref_gekmm, port_gekmm  # noqa: E402

SAMPLE_STRIDE = 389


def golden_cases():
    sweep = cases.sweep_cases()
    picked = [c for i, c in enumerate(sweep) if i % 3 == 0]
    return cases.MINI_CONFIGS + picked


def main():
    out = {}
    names = []
    for c in golden_cases():
        x, fs, y = cases.operands(c)
        z = ref_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
        zp = port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)
        err = cases.row_rel_err(zp, z, c["mm"])
        assert err <= cases.TOL[c["dt"]] * 0.1, (cases.case_id(c), err)
        cid = cases.case_id(c)
        flat = z.reshape(-1)
        names.append(cid)
        if flat.size <= 4096:
            out[cid + "/full"] = flat
        else:
            out[cid + "/sample"] = flat[::SAMPLE_STRIDE].copy()
        out[cid + "/sum"] = np.array([flat.astype(np.float64).sum(), np.abs(flat.astype(np.float64)).sum()])
        assert np.isfinite(flat).all(), cid
    out["names"] = np.array(names)
    path = os.path.join(HERE, "golden.npz")
    np.savez_compressed(path, **out)
    print("wrote %s: %d cases, %.1f KB" % (path, len(names), os.path.getsize(path) / 1024))


if __name__ == "__main__":
    main()
