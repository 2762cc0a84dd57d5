"""GPU tests of the reference's multi-GPU API (fastKronMgInitCUDA / AllocX / SGEMM / GatherY).

The distributed schedule is driven through the C ABI with several LOGICAL GPUs placed on the
one physical device (FASTKRON_MG_ONE_DEVICE=1): phases are ordered by stream events only,
no kernel waits on another, so this exercises the real kernels, redistribution maps and
buffer plan of the multi-GPU path on a single GPU.  Cases follow the reference's distributed
tests (tests/src/multi-cuda-*.cpp: 64^4-style square factors, non-square 8x32/64x16,
distinct shapes, GM x GK grids)."""
import ctypes
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu

MG_CASES = [
    # M, ps, qs, GM, GK
    (8, [16, 16, 16], [16, 16, 16], 1, 2),
    (8, [16, 16, 16, 16], [16, 16, 16, 16], 1, 4),
    (4, [16] * 4, [16] * 4, 2, 2),
    (8, [8, 32, 16], [16, 8, 8], 1, 8),
    (6, [8, 32], [32, 8], 1, 2),
    (4, [64, 64], [64, 64], 1, 8),
    (2, [64, 64, 64], [64, 64, 64], 1, 4),
    (4, [64, 64, 64], [64, 64, 64], 2, 2),
    (2, [128, 128], [128, 128], 1, 2),
    (4, [8, 32, 16, 32], [16, 8, 8, 8], 1, 4),
    (4, [16, 16, 16], [16, 16, 16], 4, 1),
]


def _cuda_free(ptr):
    """cudaFree through the CUDA runtime torch has loaded (fastKronMgAllocX hands out cudaMalloc blocks)."""
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaFree.argtypes = [ctypes.c_void_p]
    return rt.cudaFree(ctypes.c_void_p(ptr))


@pytest.mark.parametrize("parts", [1, 2])
@pytest.mark.parametrize("M,ps,qs,GM,GK", MG_CASES, ids=lambda v: str(v).replace(" ", ""))
def test_mg_api_on_logical_gpus(M, ps, qs, GM, GK, parts, monkeypatch):
    import torch
    from fastkron_b200 import lib as fk
    monkeypatch.setenv("FASTKRON_MG_ONE_DEVICE", "1")
    monkeypatch.setenv("FASTKRON_MG_PARTS", str(parts))     # row slices of the pipelined schedule
    L = fk.get()
    gpus = GM * GK
    n = len(ps)
    K = int(np.prod(ps))
    Lc = int(np.prod(qs))
    c = cases.case("mkm", "f32", M, ps, qs, seed=600 + gpus)
    x, fs, _ = cases.operands(c)
    want = oracle.port_gekmm("mkm", x, fs, ps, qs, M)

    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    streams = [torch.cuda.Stream() for _ in range(gpus)]
    sarr = (ctypes.c_void_p * gpus)(*[s.cuda_stream for s in streams])
    assert L.fastKronMgInitCUDA(h, sarr, gpus, GM, GK, 1) == fk.SUCCESS
    ye, te = ctypes.c_size_t(), ctypes.c_size_t()
    assert L.gekmmSizes(h, ctypes.c_uint32(M), ctypes.c_uint32(n), fk.u32arr(ps), fk.u32arr(qs),
                        ctypes.byref(ye), ctypes.byref(te)) == fk.SUCCESS
    assert ye.value == (M // GM) * (Lc // GK)

    dX = (ctypes.c_void_p * gpus)()
    xh = np.ascontiguousarray(x)
    assert L.fastKronMgAllocX(h, dX, ctypes.c_void_p(xh.ctypes.data), ctypes.c_uint32(M), ctypes.c_uint32(K)) == fk.SUCCESS
    fd = [torch.from_numpy(f).cuda() for f in fs]
    kron = (ctypes.c_void_p * (gpus * n))(*[fd[i].data_ptr() for _ in range(gpus) for i in range(n)])
    res = [torch.full((ye.value,), float("nan"), dtype=torch.float32, device="cuda") for _ in range(gpus)]
    t1 = [torch.empty(te.value, dtype=torch.float32, device="cuda") for _ in range(gpus)]
    t2 = [torch.empty(te.value, dtype=torch.float32, device="cuda") for _ in range(gpus)]
    torch.cuda.synchronize()
    P = lambda ts: (ctypes.c_void_p * gpus)(*[t.data_ptr() for t in ts])
    for rep in range(2):
        rc = L.fastKronMgSGEMM(h, ctypes.c_uint32(n), dX, kron, P(res), ctypes.c_uint32(M), ctypes.c_uint32(Lc),
                               ctypes.c_uint32(K), fk.u32arr(qs), fk.u32arr(ps), P(t1), P(t2), sarr)
        assert rc == fk.SUCCESS
    zh = np.zeros((M, Lc), dtype=np.float32)
    assert L.fastKronMgGatherY(h, P(res), ctypes.c_void_p(zh.ctypes.data), ctypes.c_uint32(M), ctypes.c_uint32(K),
                               ctypes.c_uint32(n), fk.u32arr(qs), fk.u32arr(ps)) == fk.SUCCESS
    assert cases.row_rel_err(zh, want, "mkm") <= cases.TOL["f32"]
    L.fastKronDestroy(h)
    # X blocks were allocated by the library with cudaMalloc; the caller frees them
    torch.cuda.synchronize()
    for g in range(gpus):
        assert _cuda_free(dX[g]) == 0


def test_mg_init_argument_errors():
    import torch
    from fastkron_b200 import lib as fk
    L = fk.get()
    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    s = (ctypes.c_void_p * 1)(torch.cuda.current_stream().cuda_stream)
    assert L.fastKronMgInitCUDA(h, s, 1, 2, 2, 1) == fk.INVALID_ARGUMENT          # grid != gpus
    os.environ["FASTKRON_MG_ONE_DEVICE"] = "1"
    try:
        s2 = (ctypes.c_void_p * 2)(0, 0)
        assert L.fastKronMgInitCUDA(h, s2, 2, 1, 2, 1) == fk.SUCCESS
        # a single factor cannot be column-sharded
        d = (ctypes.c_void_p * 2)(1, 1)
        rc = L.fastKronMgSGEMM(h, ctypes.c_uint32(1), d, d, d, ctypes.c_uint32(4), ctypes.c_uint32(8), ctypes.c_uint32(8),
                               fk.u32arr([8]), fk.u32arr([8]), d, d, s2)
        assert rc == fk.INVALID_KMM_PROBLEM
    finally:
        os.environ.pop("FASTKRON_MG_ONE_DEVICE", None)
    L.fastKronDestroy(h)
