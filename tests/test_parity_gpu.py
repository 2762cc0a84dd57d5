"""GPU parity tests: every call goes through the C ABI (ctypes -> libFastKron.so) on
device buffers and is compared with the CPU oracle on identical seeded inputs.

Tolerance (the benchmark definition's): max |z - ref| / max|ref row| <= 1e-4 for fp32,
<= 1e-12 for fp64 (cases.TOL)."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz"))


@pytest.fixture(scope="module")
def h():
    import fastkron_b200
    hd = fastkron_b200.FastKron()
    yield hd
    hd.close()


def oracle_z(c, x, fs, y):
    return oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], c["M"], c["opx"], c["opf"], c["alpha"], c["beta"], y)


@pytest.mark.parametrize("c", cases.MINI_CONFIGS, ids=cases.case_id)
@pytest.mark.parametrize("use_t2", [True, False])
def test_mini_benchmark_configs(h, c, use_t2):
    import gpu_util
    x, fs, y = cases.operands(c)
    z = gpu_util.run_case(h, c, use_temp2=use_t2, x=x, fs=fs, y=y)
    assert cases.row_rel_err(z, oracle_z(c, x, fs, y), c["mm"]) <= cases.TOL[c["dt"]]


@pytest.mark.parametrize("c", cases.sweep_cases(), ids=cases.case_id)
def test_reference_sweep(h, c):
    """The reference's functional sweep (square / non-square / distinct factors, NN TT NT TN,
    MKM and KMM, alpha=2 beta=1), against the C restatement."""
    import gpu_util
    x, fs, y = cases.operands(c)
    z = gpu_util.run_case(h, c, x=x, fs=fs, y=y)
    assert cases.row_rel_err(z, oracle_z(c, x, fs, y), c["mm"]) <= cases.TOL[c["dt"]]


def test_golden_vectors_from_reference(h):
    """Results against the committed outputs of the unmodified reference x86 backend."""
    import gpu_util
    from golden.make_golden import golden_cases, SAMPLE_STRIDE
    worst = 0.0
    for c in golden_cases():
        cid = cases.case_id(c)
        z = gpu_util.run_case(h, c, guard=False).reshape(-1)
        if cid + "/full" in GOLDEN:
            ref, got = GOLDEN[cid + "/full"], z
        else:
            ref, got = GOLDEN[cid + "/sample"], z[::SAMPLE_STRIDE]
        scale = max(float(np.abs(ref).max()), 1e-30)
        err = float(np.abs(got.astype(np.float64) - ref.astype(np.float64)).max()) / scale
        assert err <= cases.TOL[c["dt"]], (cid, err)
        worst = max(worst, err / cases.TOL[c["dt"]])
    assert worst <= 1.0


TILE_CASES = []
for _dt in ("f32", "f64"):
    for _p, _n in ((2, 9), (2, 5), (4, 7), (4, 3), (8, 5), (8, 2), (16, 4), (16, 2), (32, 3), (32, 1)):
        for _mm, _M in (("mkm", 5), ("mkm", 64), ("kmm", 8), ("kmm", 32)):
            TILE_CASES.append(cases.case(_mm, _dt, _M, [_p] * _n, [_p] * _n, "N", "N", 1.5, 0.5, 900 + len(TILE_CASES)))
            TILE_CASES.append(cases.case(_mm, _dt, _M, [_p] * _n, [_p] * _n, "T", "T", 1.0, 0.0, 900 + len(TILE_CASES)))


@pytest.mark.parametrize("c", TILE_CASES, ids=cases.case_id)
def test_fused_tile_kernels(h, c):
    """Power-of-two square factors: the fused shared-memory kernels, all fusion depths."""
    import gpu_util
    x, fs, y = cases.operands(c)
    z = gpu_util.run_case(h, c, x=x, fs=fs, y=y)
    assert cases.row_rel_err(z, oracle_z(c, x, fs, y), c["mm"]) <= cases.TOL[c["dt"]]


GEMM_CASES = [
    cases.case("mkm", "f32", 1, [64] * 3, [64] * 3, seed=700),
    cases.case("mkm", "f32", 5, [64] * 3, [64] * 3, "N", "N", 2.0, 1.0, seed=701),
    cases.case("mkm", "f32", 37, [64], [64], seed=702),
    cases.case("mkm", "f32", 3, [64, 64], [64, 64], "N", "T", 1.0, 0.0, seed=703),
    cases.case("mkm", "f32", 300, [64, 64], [64, 64], seed=704),
    cases.case("mkm", "f32", 3, [128, 128], [128, 128], "N", "N", 2.0, 1.0, seed=705),
    cases.case("mkm", "f32", 2, [128, 128, 16], [128, 128, 16], seed=706),
    cases.case("mkm", "f32", 9, [128], [128], "N", "T", 1.0, 0.0, seed=707),
    cases.case("mkm", "f64", 5, [64, 64], [64, 64], "N", "N", 2.0, 1.0, seed=708),
    cases.case("mkm", "f64", 1, [64] * 3, [64] * 3, seed=709),
    cases.case("kmm", "f32", 8, [64, 64], [64, 64], "N", "N", 2.0, 1.0, seed=710),
    cases.case("kmm", "f32", 64, [64, 64], [64, 64], "N", "T", 1.0, 0.0, seed=711),
    cases.case("kmm", "f32", 4, [128, 128], [128, 128], seed=712),
    cases.case("kmm", "f64", 2, [64, 64], [64, 64], "T", "N", 1.0, 0.0, seed=713),
    cases.case("mkm", "f32", 2, [16, 64, 8, 64], [16, 64, 8, 64], seed=714),
    cases.case("mkm", "f32", 4, [64, 16, 64], [64, 16, 64], "T", "N", 1.0, 0.0, seed=715),
]


@pytest.mark.parametrize("c", GEMM_CASES, ids=cases.case_id)
def test_large_factor_kernels(h, c):
    """64x64 / 128x128 factors: the register-blocked kernels in all three tile modes
    (contiguous contraction index, short and long trailing extents, ragged last tile)."""
    import gpu_util
    x, fs, y = cases.operands(c)
    z = gpu_util.run_case(h, c, x=x, fs=fs, y=y)
    assert cases.row_rel_err(z, oracle_z(c, x, fs, y), c["mm"]) <= cases.TOL[c["dt"]]
    # the TMA-staged tile mode waits on its stage barriers with a time limit; it must never trip
    from fastkron_b200 import lib as fk
    assert fk.get().fkbGemmTmaTimeouts() == 0


def test_fusion_off_matches_fusion_on(h):
    import gpu_util
    from fastkron_b200 import lib as fk
    c = cases.case("mkm", "f32", 16, [8] * 5, [8] * 5, seed=41)
    z1 = gpu_util.run_case(h, c)
    h.set_options(fk.OPT_NONE)
    try:
        z2 = gpu_util.run_case(h, c)
    finally:
        h.set_options(fk.OPT_USE_FUSION)
    assert cases.row_rel_err(z1, z2, "mkm") <= 1e-5


@pytest.mark.parametrize("mm", ["mkm", "kmm"])
@pytest.mark.parametrize("dt", ["f32", "f64"])
@pytest.mark.parametrize("ps,qs,M", [([4, 3, 8, 2], [2, 5, 8, 3], 6), ([16, 12, 8], [16, 10, 24], 37),
                                     ([32, 16], [32, 16], 64), ([16, 3, 8], [16, 5, 8], 5), ([8] * 4, [8] * 4, 33)],
                         ids=["tiny", "narrow-tiles", "pow2", "pow2-ragged", "pow2-many-rows"])
def test_forward_intermediates(h, mm, dt, ps, qs, M):
    """{s,d}{mkm,kmm}Forward: Z and each of the N-1 intermediates in the reference's layout
    (tiny factors: one thread per output; the others: the any-shape kernel's 16- and 32-wide tiles)."""
    import torch
    import gpu_util
    c = cases.case(mm, dt, M, ps, qs, seed=77)
    x, fs, _ = cases.operands(c)
    zo, inter_o = oracle.port_gekmm(mm, x, fs, c["ps"], c["qs"], c["M"], want_intermediates=True)
    ye, ies = h.sizes_forward(c["M"], c["ps"], c["qs"])
    assert [a.size for a in inter_o] == ies and ye == zo.size
    tdt = gpu_util.torch_dt(dt)
    xd = torch.from_numpy(x).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fs]
    z = torch.empty(ye, dtype=tdt, device="cuda")
    inter = [torch.empty(n, dtype=tdt, device="cuda") for n in ies]
    h.raw_forward(mm, "s" if dt == "f32" else "d", c["M"], c["ps"], c["qs"], xd.data_ptr(), 1,
                  [f.data_ptr() for f in fd], 1, z.data_ptr(), [t.data_ptr() for t in inter])
    torch.cuda.synchronize()
    assert cases.row_rel_err(z.cpu().numpy().reshape(zo.shape), zo, mm) <= cases.TOL[dt]
    for got, want in zip(inter, inter_o):
        assert cases.row_rel_err(got.cpu().numpy().reshape(want.shape), want, mm) <= cases.TOL[dt]


@pytest.mark.parametrize("mm", ["mkm", "kmm"])
@pytest.mark.parametrize("share", ["none", "x", "f"])
def test_strided_batched(h, mm, share):
    """*StridedBatched with X-only, F-only and fully batched operands (stride 0 = shared)."""
    import torch
    import gpu_util
    B, M, ps, qs = 3, 8, [8, 8, 4], [8, 8, 6]
    dt = "f32"
    K, Lc = 256, 384
    rng = np.random.default_rng(5)
    nx = 1 if share == "x" else B
    nf = 1 if share == "f" else B
    xs = rng.uniform(-1, 1, size=(nx, M * K)).astype(np.float32)
    fss = [rng.uniform(-1, 1, size=(nf, p * q)).astype(np.float32) for p, q in zip(ps, qs)]
    ys = rng.uniform(-1, 1, size=(B, M * Lc)).astype(np.float32)
    xd = torch.from_numpy(xs).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fss]
    yd = torch.from_numpy(ys).cuda()
    ye, te = h.sizes(M, ps, qs)
    z = torch.empty((B, ye), dtype=torch.float32, device="cuda")
    t1 = torch.empty(B * te, dtype=torch.float32, device="cuda")
    t2 = torch.empty(B * te, dtype=torch.float32, device="cuda")
    h.raw_gemm_strided_batched(mm, "s", M, ps, qs, xd.data_ptr(), 1, 0 if share == "x" else M * K,
                               [f.data_ptr() for f in fd], 1, [0 if share == "f" else p * q for p, q in zip(ps, qs)],
                               z.data_ptr(), ye, 2.0, 1.0, B, yd.data_ptr(), ye, t1.data_ptr(), t2.data_ptr())
    torch.cuda.synchronize()
    zc = z.cpu().numpy()
    for b in range(B):
        want = oracle.port_gekmm(mm, xs[0 if share == "x" else b], [f[0 if share == "f" else b] for f in fss],
                                 ps, qs, M, "N", "N", 2.0, 1.0, ys[b])
        assert cases.row_rel_err(zc[b].reshape(want.shape), want, mm) <= cases.TOL[dt]


BATCH_SHAPES = [
    # dt, M, ps, qs: tile kernels (narrow + wide, TMA ring), any-shape kernel, generic kernel, fp64 DMMA
    ("f32", 8, [16, 16, 16, 16], [16, 16, 16, 16]),
    ("f32", 5, [12, 31], [12, 63]),
    ("f64", 4, [8, 8, 8, 8], [8, 8, 8, 8]),
    ("f32", 6, [3, 5, 32, 32], [3, 5, 32, 32]),
    ("f64", 3, [24, 9], [10, 24]),
]


@pytest.mark.parametrize("mm", ["mkm", "kmm"])
@pytest.mark.parametrize("share", ["none", "x", "f"])
@pytest.mark.parametrize("dt,M,ps,qs", BATCH_SHAPES, ids=lambda v: str(v).replace(" ", ""))
def test_strided_batch_is_one_launch_per_pass(h, dt, M, ps, qs, mm, share):
    """A strided batch whose passes all run on batch-capable kernels is enqueued as one launch per
    pass (the batch is a grid dimension, as in the reference's src/kernels/gpu_kmmkernel.h:124-144),
    with non-contiguous entries (padding between them), shared or per-entry operands."""
    import ctypes
    import torch
    from fastkron_b200 import lib as fk
    B = 4
    ndt = cases.NP_DT[dt]
    tdt = torch.float32 if dt == "f32" else torch.float64
    K, Lc = int(np.prod(ps)), int(np.prod(qs))
    pad = 64                                            # elements between entries: strides != sizes
    rng = np.random.default_rng(17)
    nx = 1 if share == "x" else B
    nf = 1 if share == "f" else B
    xs = rng.uniform(-1, 1, size=(nx, M * K + pad)).astype(ndt)
    fss = [rng.uniform(-1, 1, size=(nf, p * q + pad)).astype(ndt) for p, q in zip(ps, qs)]
    ys = rng.uniform(-1, 1, size=(B, M * Lc + pad)).astype(ndt)
    xd = torch.from_numpy(xs).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fss]
    yd = torch.from_numpy(ys).cuda()
    ye, te = h.sizes(M, ps, qs)
    z = torch.full((B, ye + pad), float("nan"), dtype=tdt, device="cuda")
    t1 = torch.empty(B * te, dtype=tdt, device="cuda")
    t2 = torch.empty(B * te, dtype=tdt, device="cuda")
    L = fk.get()
    L.fkbLaunchCount.restype = ctypes.c_ulonglong
    n0 = L.fkbLaunchCount()
    h.raw_gemm_strided_batched(mm, "s" if dt == "f32" else "d", M, ps, qs, xd.data_ptr(), 1,
                               0 if share == "x" else M * K + pad, [f.data_ptr() for f in fd], 1,
                               [0 if share == "f" else p * q + pad for p, q in zip(ps, qs)],
                               z.data_ptr(), ye + pad, 2.0, 1.0, B, yd.data_ptr(), ye + pad, t1.data_ptr(), t2.data_ptr())
    torch.cuda.synchronize()
    launches = int(L.fkbLaunchCount() - n0)
    buf = ctypes.create_string_buffer(1 << 14)
    npass = L.fkbDescribePlan(ctypes.c_int(mm == "kmm"), ctypes.c_int(dt == "f64"), ctypes.c_uint32(M),
                              ctypes.c_uint32(len(ps)), fk.u32arr(ps), fk.u32arr(qs), 1, 1, 0, 1, 1, 16, buf,
                              ctypes.c_size_t(len(buf)))
    assert launches == npass, (launches, npass, buf.value.decode())
    zc = z.cpu().numpy()
    assert np.isnan(zc[:, ye:]).all(), "the padding between result entries was written"
    for b in range(B):
        want = oracle.port_gekmm(mm, xs[0 if share == "x" else b][:M * K],
                                 [f[0 if share == "f" else b][:p * q] for f, p, q in zip(fss, ps, qs)],
                                 ps, qs, M, "N", "N", 2.0, 1.0, ys[b][:M * Lc])
        assert cases.row_rel_err(zc[b][:ye].reshape(want.shape), want, mm) <= cases.TOL[dt]


def test_batched_shared_factors_dense_folds_into_rows(h):
    """Strided batch with shared factors and back-to-back X/Z/Y entries (the case the reference's
    Python wrapper produces for a batched X): same result as entry-by-entry calls."""
    import torch
    B, M, ps, qs = 5, 6, [16, 16, 16], [16, 16, 16]
    K = Lc = 4096
    rng = np.random.default_rng(9)
    xs = rng.uniform(-1, 1, size=(B, M * K)).astype(np.float32)
    fss = [rng.uniform(-1, 1, size=p * q).astype(np.float32) for p, q in zip(ps, qs)]
    ys = rng.uniform(-1, 1, size=(B, M * Lc)).astype(np.float32)
    xd, yd = torch.from_numpy(xs).cuda(), torch.from_numpy(ys).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fss]
    ye, te = h.sizes(M, ps, qs)
    z = torch.empty((B, ye), dtype=torch.float32, device="cuda")
    t1 = torch.empty(B * te, dtype=torch.float32, device="cuda")
    t2 = torch.empty(B * te, dtype=torch.float32, device="cuda")
    h.raw_gemm_strided_batched("mkm", "s", M, ps, qs, xd.data_ptr(), 1, M * K, [f.data_ptr() for f in fd], 1, [0, 0, 0],
                               z.data_ptr(), ye, 2.0, 1.0, B, yd.data_ptr(), ye, t1.data_ptr(), t2.data_ptr())
    torch.cuda.synchronize()
    zc = z.cpu().numpy()
    for b in range(B):
        want = oracle.port_gekmm("mkm", xs[b], fss, ps, qs, M, "N", "N", 2.0, 1.0, ys[b])
        assert cases.row_rel_err(zc[b].reshape(want.shape), want, "mkm") <= cases.TOL["f32"]


def test_tune_option_picks_a_plan_and_stays_correct(h):
    """fastKronOptionsTune: the first call times fused against unfused passes; results unchanged."""
    import gpu_util
    from fastkron_b200 import lib as fk
    c = cases.case("mkm", "f64", 12, [8] * 4, [8] * 4, alpha=2.0, beta=1.0, seed=61)
    x, fs, y = cases.operands(c)
    want = oracle_z(c, x, fs, y)
    h.set_options(fk.OPT_USE_FUSION | fk.OPT_TUNE)
    try:
        for _ in range(2):
            z = gpu_util.run_case(h, c, x=x, fs=fs, y=y)
            assert cases.row_rel_err(z, want, "mkm") <= cases.TOL["f64"]
    finally:
        h.set_options(fk.OPT_USE_FUSION)


def test_in_place_epilogue_with_both_temps(h):
    """Z may alias Y when both temporaries are given (include/fastkron.h contract)."""
    import torch
    import gpu_util
    c = cases.case("mkm", "f64", 9, [8, 8, 8], [8, 8, 8], alpha=2.0, beta=1.0, seed=31)
    x, fs, y = cases.operands(c)
    want = oracle_z(c, x, fs, y)
    xd = torch.from_numpy(x).cuda()
    fd = [torch.from_numpy(f).cuda() for f in fs]
    zy = torch.from_numpy(y.copy()).cuda()
    ye, te = h.sizes(c["M"], c["ps"], c["qs"])
    t1 = torch.empty(te, dtype=torch.float64, device="cuda")
    t2 = torch.empty(te, dtype=torch.float64, device="cuda")
    h.raw_gemm("mkm", "d", c["M"], c["ps"], c["qs"], xd.data_ptr(), 1, [f.data_ptr() for f in fd], 1,
               zy.data_ptr(), 2.0, 1.0, zy.data_ptr(), t1.data_ptr(), t2.data_ptr())
    torch.cuda.synchronize()
    assert cases.row_rel_err(zy.cpu().numpy().reshape(want.shape), want, "mkm") <= cases.TOL["f64"]


def test_argument_errors(h):
    """Error codes of the reference's argument checks (src/handle/handle.cpp:114-127)."""
    import torch
    from fastkron_b200 import lib as fk, FastKronError
    x = torch.zeros(4 * 16, device="cuda")
    f = torch.zeros(16, device="cuda")
    z = torch.zeros(4 * 16, device="cuda")
    t = torch.zeros(4 * 16, device="cuda")
    args = ("mkm", "s", 4, [4, 4], [4, 4], x.data_ptr(), 1, [f.data_ptr(), f.data_ptr()], 1)
    with pytest.raises(FastKronError) as e:
        h.raw_gemm(*args, 0, 1.0, 0.0, 0, t.data_ptr(), 0)                      # Z == NULL
    assert e.value.code == fk.INVALID_ARGUMENT
    with pytest.raises(FastKronError) as e:
        h.raw_gemm(*args, z.data_ptr(), 1.0, 0.0, 0, 0, 0)                      # temp1 == NULL
    assert e.value.code == fk.INVALID_ARGUMENT
    with pytest.raises(FastKronError) as e:
        h.raw_gemm(*args, z.data_ptr(), 1.0, 1.0, z.data_ptr(), t.data_ptr(), 0)  # Z == Y without temp2
    assert e.value.code == fk.INVALID_ARGUMENT
    h.raw_gemm(*args, z.data_ptr(), 1.0, 0.0, 0, t.data_ptr(), 0)               # valid
    torch.cuda.synchronize()


def test_torch_front_end_matches_kron(h):
    """gemkm / gekmm on torch tensors (transposed views included) against torch.kron."""
    import torch
    import fastkron_b200
    torch.manual_seed(0)
    fs = [torch.randint(0, 5, (p, q), device="cuda").double() for p, q in ((4, 3), (2, 5), (8, 8))]
    x = torch.randint(0, 5, (6, 64), device="cuda").double()
    kron = torch.kron(torch.kron(fs[0], fs[1]), fs[2])
    y = torch.randint(0, 5, (6, 120), device="cuda").double()
    assert torch.equal(fastkron_b200.gemkm(x, fs, 2.0, 1.0, y), 2.0 * x @ kron + y)
    assert torch.equal(fastkron_b200.gemkm(x.t().contiguous().t(), fs), x @ kron)
    xt = torch.randint(0, 5, (120, 7), device="cuda").double()
    fk = [f.t().contiguous().t() for f in fs]            # transposed views -> opF = T
    assert torch.equal(fastkron_b200.gekmm(fs, xt), kron @ xt)
    assert torch.equal(fastkron_b200.gemkm(x, fk), x @ kron)


# ---- full-size checks on the benchmark configurations --------------------------------

def _rowsum_weights(fs, ps, qs, mm, opf, dt):
    """w[k] = prod_i (sum_q F_i[p_i, q]) so that (X (x)F) 1 = X w exactly in real arithmetic."""
    w = np.ones(1, dtype=np.float64)
    for f, p, q in zip(fs, ps, qs):
        fd = np.asarray(f, dtype=np.float64)
        pmajor = (opf == "N") if mm == "mkm" else (opf == "T")
        F = fd.reshape(p, q) if pmajor else fd.reshape(q, p).T
        w = np.kron(w, F.sum(axis=1))
    return w


FULL = [
    ("C1", cases.case("mkm", "f32", 1024, [16] * 4, [16] * 4, seed=0)),
    ("C2", cases.case("mkm", "f64", 16, [8] * 8, [8] * 8, seed=1)),
    ("C3", cases.case("kmm", "f32", 1024, [32] * 3, [32] * 3, "T", "N", 2.0, 1.0, seed=2, dist="normal")),
    ("C4", cases.case("mkm", "f32", 2048, [128, 128, 16], [128, 128, 16], seed=4)),
    # the one configuration whose element offsets reach 2^32 (M*K = 2^32): X, Z and both
    # temporaries are 17 GB each
    ("C5", cases.case("mkm", "f32", 256, [64] * 4, [64] * 4, seed=5)),
]


@pytest.mark.parametrize("name,c", FULL, ids=[n for n, _ in FULL])
def test_full_size_rows_and_checksum(h, name, c):
    """BASELINE-size runs: (1) a few rows (MKM) / columns (KMM) compared element-wise with
    the oracle run on just those rows, (2) the size-independent checksum property
    Z 1 = alpha X (r_1 (x) ... (x) r_N) + beta Y 1 with r_i the row sums of F_i."""
    import torch
    import gpu_util
    from fastkron_b200 import synth
    tdt = gpu_util.torch_dt(c["dt"])
    M, ps, qs, mm = c["M"], c["ps"], c["qs"], c["mm"]
    K = int(np.prod(ps, dtype=object))
    Lc = int(np.prod(qs, dtype=object))
    fs = [synth.uniform(c["seed"] + 2000 + i, p * q, cases.NP_DT[c["dt"]]) for i, (p, q) in enumerate(zip(ps, qs))]
    fd = [torch.from_numpy(f).cuda() for f in fs]
    xd = torch.empty(M * K, dtype=tdt, device="cuda")
    if c.get("dist") == "normal":
        xd.copy_(torch.from_numpy(synth.normal(c["seed"], M * K, cases.NP_DT[c["dt"]])))
    else:
        synth.fill_uniform_cuda(xd, c["seed"])
    yd = None
    if c["beta"] != 0:
        yd = torch.from_numpy(synth.normal(c["seed"] + 1000, M * Lc, cases.NP_DT[c["dt"]])).cuda()
    ye, te = h.sizes(M, ps, qs)
    z = torch.empty(ye, dtype=tdt, device="cuda")
    t1 = torch.empty(te, dtype=tdt, device="cuda")
    t2 = torch.empty(te, dtype=tdt, device="cuda")
    h.raw_gemm(mm, "s" if c["dt"] == "f32" else "d", M, ps, qs, xd.data_ptr(), gpu_util.OPC[c["opx"]],
               [f.data_ptr() for f in fd], gpu_util.OPC[c["opf"]], z.data_ptr(), c["alpha"], c["beta"],
               yd.data_ptr() if yd is not None else 0, t1.data_ptr(), t2.data_ptr())
    torch.cuda.synchronize()
    # views as (M, K) / (M, L) matrices regardless of storage order
    x_rowmajor = (mm == "mkm") == (c["opx"] == "N")
    Xv = xd.view(M, K) if x_rowmajor else xd.view(K, M).t()
    Zv = z.view(M, Lc) if mm == "mkm" else z.view(Lc, M).t()
    Yv = None if yd is None else (yd.view(M, Lc) if mm == "mkm" else yd.view(Lc, M).t())
    rows = sorted({0, 1, M // 2, M - 1})
    xr = np.ascontiguousarray(Xv[rows].cpu().numpy())
    yr = None if Yv is None else np.ascontiguousarray(Yv[rows].cpu().numpy())
    # the oracle on those rows as an MKM with row-major X (rows are independent)
    opf_mkm = c["opf"] if mm == "mkm" else ("T" if c["opf"] == "N" else "N")
    want = oracle.port_gekmm("mkm", xr, fs, ps, qs, len(rows), "N", opf_mkm, c["alpha"], c["beta"], yr)
    got = Zv[rows].cpu().numpy()
    assert cases.row_rel_err(got, want, "mkm") <= cases.TOL[c["dt"]]
    # checksum over all rows, accumulated in float64 on the device, a slab of rows at a time so
    # that the float64 copies stay below 2 GB whatever the configuration
    del t1, t2
    torch.cuda.empty_cache()
    w = torch.from_numpy(_rowsum_weights(fs, ps, qs, mm, c["opf"], c["dt"])).cuda()
    slab = max(1, min(M, (1 << 28) // max(K, Lc)))
    rel = 0.0
    for r0 in range(0, M, slab):
        r1 = min(M, r0 + slab)
        zs = Zv[r0:r1].double()
        lhs = zs.sum(dim=1)
        rhs = c["alpha"] * (Xv[r0:r1].double() @ w)
        if Yv is not None:
            rhs = rhs + c["beta"] * Yv[r0:r1].double().sum(dim=1)
        scale = zs.abs().sum(dim=1)
        rel = max(rel, ((lhs - rhs).abs() / scale).max().item())
        del zs, lhs, rhs, scale
    assert rel <= cases.TOL[c["dt"]], rel


def test_host_operand_pipeline(h):
    """HostGeMKM: pinned host X/Z, row slabs with overlapped copies, ragged last slab."""
    import torch
    import fastkron_b200
    c = cases.case("mkm", "f32", 37, [16, 8, 16], [16, 8, 16], alpha=1.5, seed=88)
    x, fs, _ = cases.operands(c)
    want = oracle_z(c, x, fs, None)
    hx = torch.from_numpy(x).view(37, -1).pin_memory()
    hz = torch.empty(37, want.shape[1], dtype=torch.float32).pin_memory()
    fd = [torch.from_numpy(f).cuda().view(p, q) for f, p, q in zip(fs, c["ps"], c["qs"])]
    op = fastkron_b200.HostGeMKM(37, c["ps"], c["qs"], rows_per_slab=5)
    for _ in range(2):
        hz.zero_()
        op(hx, fd, hz, 1.5)
        torch.cuda.synchronize()
        assert cases.row_rel_err(hz.numpy(), want, "mkm") <= cases.TOL["f32"]
    op.close()
