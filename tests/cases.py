"""Shared case lists and operand builders for the parity tests.

A case is a dict: mm ("mkm"/"kmm"), dt ("f32"/"f64"), M, ps, qs, opx, opf, alpha, beta, seed.
Operands are pure functions of the seed (fastkron_b200.synth), so the CPU oracles, the
golden fixtures and the GPU tests all see identical inputs without shipping them.
"""
import numpy as np

from fastkron_b200 import synth

NP_DT = {"f32": np.float32, "f64": np.float64}


def case(mm, dt, M, ps, qs, opx="N", opf="N", alpha=1.0, beta=0.0, seed=0, dist="uniform"):
    return dict(mm=mm, dt=dt, M=M, ps=list(ps), qs=list(qs), opx=opx, opf=opf, alpha=alpha, beta=beta,
                seed=seed, dist=dist)


def case_id(c):
    shape = "x".join("%dx%d" % (p, q) for p, q in zip(c["ps"], c["qs"]))
    return "%s-%s-M%d-%s-%s%s-a%g-b%g-s%d" % (c["mm"], c["dt"], c["M"], shape, c["opx"], c["opf"],
                                               c["alpha"], c["beta"], c["seed"])


def operands(c):
    """Stored buffers (flat numpy arrays) x, [f_i], y for a case.  Stream layout: X from
    stream `seed`, Y from `seed+1000`, factor i from `seed+2000+i`, each filled in the
    order of the stored buffer."""
    dt = NP_DT[c["dt"]]
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    gen = synth.normal if c.get("dist") == "normal" else synth.uniform
    x = gen(c["seed"], c["M"] * K, dt)
    y = gen(c["seed"] + 1000, c["M"] * L, dt) if c["beta"] != 0 else None
    fs = [synth.uniform(c["seed"] + 2000 + i, p * q, dt) for i, (p, q) in enumerate(zip(c["ps"], c["qs"]))]
    return x, fs, y


def row_rel_err(z, ref, mm):
    """max |z - ref| / max_l |ref[row, l]|  (row = m: axis 1 for MKM, axis 0 for KMM) --
    the parity metric of the benchmark definition."""
    z = np.asarray(z, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    axis = 1 if mm == "mkm" else 0
    den = np.abs(ref).max(axis=axis, keepdims=True)
    den = np.where(den == 0, 1.0, den)
    return float((np.abs(z - ref) / den).max())


TOL = {"f32": 1e-4, "f64": 1e-12}

# ---- miniature versions of the five benchmark configurations -------------------
MINI_CONFIGS = [
    case("mkm", "f32", 8, [16] * 4, [16] * 4, seed=0),                                   # C1
    case("mkm", "f64", 4, [8] * 6, [8] * 6, seed=1),                                     # C2 (8^6)
    case("kmm", "f32", 16, [32] * 3, [32] * 3, opx="T", opf="N", alpha=2.0, beta=1.0, seed=2,
         dist="normal"),                                                                  # C3
    case("mkm", "f32", 4, [128, 128, 16], [128, 128, 16], seed=4),                        # C4
    case("mkm", "f32", 2, [64] * 3, [64] * 3, seed=5),                                    # C5 (64^3)
]

# ---- the reference's own functional sweep, condensed ----------------------------
# (tests/src/general-tests-NN.cpp:34-166 and general-tests-TT.cpp:26-83 of the reference:
#  square and non-square factors, distinct shapes, M in {1,3,13,16,17,20}, alpha=2/beta=1)
def sweep_cases():
    out = []
    seed = 100
    square = [(2, 9), (3, 5), (4, 6), (5, 4), (6, 3), (8, 5), (12, 3), (16, 3), (24, 2), (31, 2), (32, 3),
              (50, 2), (55, 2), (64, 2), (127, 2), (128, 2), (129, 1), (255, 1), (297, 1)]
    for p, n in square:
        for mm, M in (("mkm", 16), ("kmm", 3)):
            for ops in ("NN", "TT"):
                seed += 1
                out.append(case(mm, "f32" if seed % 2 else "f64", M, [p] * n, [p] * n, ops[0], ops[1],
                                2.0, 1.0, seed))
    nonsq = [([1], [4]), ([5], [1]), ([2, 2, 2], [4, 4, 4]), ([31, 31], [63, 63]), ([63, 63], [31, 31]),
             ([297], [127]), ([127], [297]), ([2, 5, 6], [3, 2, 4]), ([14, 19], [15, 13]),
             ([14, 19, 34, 21], [15, 13, 23, 34]), ([8, 32, 16, 32], [16, 8, 8, 8])]
    for ps, qs in nonsq:
        for mm, M in (("mkm", 13), ("kmm", 17), ("kmm", 1), ("mkm", 1)):
            for ops in ("NN", "TT", "NT", "TN"):
                seed += 1
                out.append(case(mm, "f32" if seed % 2 else "f64", M, ps, qs, ops[0], ops[1], 2.0, 1.0, seed))
    return out
