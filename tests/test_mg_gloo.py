"""CPU test of the multi-GPU schedule's host logic with real ranks (gloo, world_size 2 and 4).

Every rank owns a column block of X, runs a numpy statement of phase 1 / phase 2
(fastkron_b200.mg.emulate_rank_phase*) and places its outputs exactly where the library's
redistribution maps (fkbMgScatterDesc, the same numbers the CUDA kernels use) say; blocks
travel between ranks through torch.distributed.  The gathered result must equal the oracle's."""
import os
import socket
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import cases  # noqa: E402


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, M, ps, qs, seed, q):
    import torch
    import torch.distributed as dist
    from fastkron_b200 import mg
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = cases.case("mkm", "f32", M, ps, qs, seed=seed)
        x, fs, _ = cases.operands(c)
        K = int(np.prod(ps))
        L = int(np.prod(qs))
        Kl, Ll = K // world, L // world
        xb = x.reshape(M, K)[:, rank * Kl:(rank + 1) * Kl]
        B = int(np.prod(qs[2:])) if len(qs) > 2 else 1

        def exchange(pieces, nelem):
            """pieces: list of (dst, offsets, values); returns this rank's received buffer."""
            buf = np.zeros(nelem, dtype=np.float64)
            for src in range(world):
                for dst in range(world):
                    if rank == src:
                        _, off, val = pieces[dst]
                        payload = [torch.from_numpy(off.astype(np.int64)), torch.from_numpy(val.copy())]
                    else:
                        payload = None
                    if src == dst:
                        if rank == src:
                            buf[payload[0].numpy()] = payload[1].numpy()
                        continue
                    if rank == src:
                        dist.send(torch.tensor([payload[0].numel()]), dst)
                        dist.send(payload[0], dst)
                        dist.send(payload[1], dst)
                    elif rank == dst:
                        n = torch.zeros(1, dtype=torch.int64)
                        dist.recv(n, src)
                        off = torch.zeros(int(n), dtype=torch.int64)
                        val = torch.zeros(int(n), dtype=torch.float64)
                        dist.recv(off, src)
                        dist.recv(val, src)
                        buf[off.numpy()] = val.numpy()
            return buf

        recv = exchange(mg.emulate_rank_phase1(rank, world, M, ps, qs, xb, fs), M * ps[0] * (qs[1] // world) * B)
        dist.barrier()
        res = exchange(mg.emulate_rank_phase2(rank, world, M, ps, qs, recv, fs[0]), M * Ll)
        parts = [torch.zeros(M * Ll, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(res))
        if rank == 0:
            z = np.concatenate([p.numpy().reshape(M, Ll) for p in parts], axis=1)
            q.put(z)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,M,ps,qs", [
    (2, 3, [4, 4, 4], [4, 4, 4]),
    (2, 2, [8, 6], [4, 2]),
    (4, 2, [4, 8, 3, 2], [8, 4, 2, 5]),
    (2, 5, [2, 5, 6], [2, 4, 4]),
])
def test_schedule_with_gloo_ranks(world, M, ps, qs):
    import torch.multiprocessing as mp
    import oracle
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, ps, qs, 11, q)) for r in range(world)]
    for p in procs:
        p.start()
    z = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    c = cases.case("mkm", "f32", M, ps, qs, seed=11)
    x, fs, _ = cases.operands(c)
    want = oracle.numpy_gekmm("mkm", x, fs, ps, qs, M)
    assert np.abs(z - want).max() <= 1e-9 * max(1.0, np.abs(want).max())


def test_scatter_desc_rejects_bad_grids():
    from fastkron_b200 import mg, FastKronError
    with pytest.raises(FastKronError):
        mg.scatter_desc(1, 0, 2, [4], [4])               # one factor cannot be column-sharded
    with pytest.raises(FastKronError):
        mg.scatter_desc(1, 0, 4, [6, 4], [4, 4])         # 4 does not divide P1
    d = mg.scatter_desc(2, 1, 2, [4, 4, 4], [4, 4, 4])
    assert d["parts"] == 2 and d["qPer"] == 2 and d["sQ"] == 16 and d["zOff"] == 8


def test_schedule_order_of_row_slices():
    """Host logic of the pipelined schedule: with R row slices a call enqueues, on a GPU's one
    compute stream, P1(0), P1(1), P2(0), ..., P2(R-1): every slice's second half comes after its
    first half and after the NEXT slice's first half (whose passes hide this slice's transfer)."""
    import ctypes
    from fastkron_b200 import lib as fk
    L = fk.get()
    for R in (1, 2, 3, 4, 8):
        out = (ctypes.c_int * (4 * R))()
        n = L.fkbMgOrder(ctypes.c_int(R), out, ctypes.c_int(2 * R))
        assert n == 2 * R
        seq = [(out[2 * i], out[2 * i + 1]) for i in range(n)]
        assert sorted(seq) == sorted([(1, s) for s in range(R)] + [(2, s) for s in range(R)])
        pos = {hs: i for i, hs in enumerate(seq)}
        for s in range(R):
            assert pos[(1, s)] < pos[(2, s)]
            if s + 1 < R:
                assert pos[(1, s + 1)] < pos[(2, s)]
                assert pos[(2, s)] < pos[(2, s + 1)]
