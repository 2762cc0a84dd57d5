"""The multi-GPU path on REAL devices (skipped below two GPUs).

(1) fastKronMgInitCUDA / AllocX / SGEMM / GatherY from one process on two physical devices --
    what the reference's tests/src/multi-cuda-no-fusion-tests.cpp does: real devices, gather,
    compare all elements.
(2) The per-rank pipeline of fastkron_b200.mg with two NCCL ranks (tests/mg_child.py): fused and
    staged transport, one and two row slices, device and host operands, all rows against the oracle.
(3) fastkron_b200.mg at world size 1 (any number of GPUs)."""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402
import oracle  # noqa: E402

pytestmark = pytest.mark.gpu


def _ngpu():
    import torch
    return torch.cuda.device_count()


C_API_CASES = [
    (8, [64, 64, 64], [64, 64, 64], 1),
    (8, [64, 64, 64], [64, 64, 64], 2),
    (8, [16] * 4, [16] * 4, 2),
    (6, [8, 32], [32, 8], 1),
    (4, [128, 128], [128, 128], 2),
]


@pytest.mark.parametrize("M,ps,qs,parts", C_API_CASES, ids=lambda v: str(v).replace(" ", ""))
def test_mg_c_api_on_two_real_devices(M, ps, qs, parts, monkeypatch):
    import torch
    from fastkron_b200 import lib as fk
    if _ngpu() < 2:
        pytest.skip("needs two GPUs")
    monkeypatch.delenv("FASTKRON_MG_ONE_DEVICE", raising=False)
    monkeypatch.setenv("FASTKRON_MG_PARTS", str(parts))
    L = fk.get()
    gpus, n = 2, len(ps)
    K, Lc = int(np.prod(ps)), int(np.prod(qs))
    c = cases.case("mkm", "f32", M, ps, qs, seed=650 + n)
    x, fs, _ = cases.operands(c)
    want = oracle.port_gekmm("mkm", x, fs, ps, qs, M)
    torch.cuda.set_device(0)
    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    streams = []
    for d in range(gpus):
        with torch.cuda.device(d):
            streams.append(torch.cuda.Stream())
    sarr = (ctypes.c_void_p * gpus)(*[s.cuda_stream for s in streams])
    assert L.fastKronMgInitCUDA(h, sarr, gpus, 1, gpus, 1) == fk.SUCCESS
    ye, te = ctypes.c_size_t(), ctypes.c_size_t()
    assert L.gekmmSizes(h, ctypes.c_uint32(M), ctypes.c_uint32(n), fk.u32arr(ps), fk.u32arr(qs),
                        ctypes.byref(ye), ctypes.byref(te)) == fk.SUCCESS
    dX = (ctypes.c_void_p * gpus)()
    xh = np.ascontiguousarray(x)
    assert L.fastKronMgAllocX(h, dX, ctypes.c_void_p(xh.ctypes.data), ctypes.c_uint32(M), ctypes.c_uint32(K)) == fk.SUCCESS
    fd, res, t1, t2 = [], [], [], []
    for d in range(gpus):
        with torch.cuda.device(d):
            fd.append([torch.from_numpy(f).cuda() for f in fs])
            res.append(torch.full((ye.value,), float("nan"), dtype=torch.float32, device="cuda"))
            t1.append(torch.empty(te.value, dtype=torch.float32, device="cuda"))
            t2.append(torch.empty(te.value, dtype=torch.float32, device="cuda"))
            torch.cuda.synchronize()
    kron = (ctypes.c_void_p * (gpus * n))(*[fd[d][i].data_ptr() for d in range(gpus) for i in range(n)])
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
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaFree.argtypes = [ctypes.c_void_p]
    for d in range(gpus):
        with torch.cuda.device(d):
            torch.cuda.synchronize()
            assert rt.cudaFree(ctypes.c_void_p(dX[d])) == 0
    torch.cuda.set_device(0)


def test_mg_pipeline_two_nccl_ranks():
    if _ngpu() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    env.pop("FASTKRON_MG_ONE_DEVICE", None)
    env.pop("FASTKRON_MG_PARTS", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "mg_child.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + "\n" + out.stderr[-4000:]
    assert "MG-CHILD-OK" in out.stdout


def test_mg_module_world_size_one():
    """fastkron_b200.mg without a process group: the single-rank path of the same class."""
    import torch
    from fastkron_b200 import mg
    for M, ps, qs in ((8, [64, 64, 64], [64, 64, 64]), (5, [16, 8, 4], [8, 8, 6])):
        c = cases.case("mkm", "f32", M, ps, qs, seed=680)
        x, fs, _ = cases.operands(c)
        want = oracle.port_gekmm("mkm", x, fs, ps, qs, M)
        eng = mg.PipelinedRankGeMKM(M, ps, qs)
        assert eng.world == 1
        z = eng.run(torch.from_numpy(x).cuda(), [torch.from_numpy(f).cuda() for f in fs])
        torch.cuda.synchronize()
        assert cases.row_rel_err(z.cpu().numpy(), want, "mkm") <= cases.TOL["f32"]
        eng.close()
