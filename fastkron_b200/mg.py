"""Column-sharded multi-GPU GeMKM for one-process-per-GPU hosts (torch.distributed).

The reference's multi-GPU API (include/fastkronMg.h of the reference) is one process
driving all GPUs; `libFastKron.so` implements that API (fastKronMgSGEMM).  A torchrun-style
host has one process per GPU instead, so the library exposes the same schedule per rank
(`fkbMgPipe*` in csrc/mg.cu) and this module supplies the one thing processes must do for
each other: exchanging CUDA IPC handles of the buffers the peers write into.

Rank g of G owns columns [g*K/G, (g+1)*K/G) of X and of the result, all M rows, and a
copy of every factor.  Phase 1 contracts the trailing modes locally and hands each output
row to the rank that owns its slice of the second mode; phase 2 contracts the leading mode
and hands each result row to the rank that owns it.
"""
import ctypes

import numpy as np

from . import lib as _lib


def _prod(v):
    r = 1
    for a in v:
        r *= int(a)
    return r


class _RawCuda:
    """Wraps a raw device pointer so that torch can view it as a tensor."""

    def __init__(self, ptr, nelem, typestr="<f4"):
        self.__cuda_array_interface__ = {"shape": (nelem,), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}


class PipelinedRankGeMKM:
    """One rank of a column-sharded fp32 GeMKM  Z = X (F1 (x) ... (x) FN)  in a host that runs
    one process per GPU.

    The schedule itself -- row slices out of phase, kernels, copy-engine transfers, ordering
    between ranks -- is the library's (csrc/mg.cu, the same code fastKronMgSGEMM runs).  This
    class only does what a process cannot do for its peers: it publishes CUDA IPC handles of
    the rank's receive area, result block and flag array and maps the peers'.

    parts: row slices (0 = the library's choice); mode: "staged" (copy engines), "fused"
    (peer stores from the kernels) or "auto"."""

    def __init__(self, M, ps, qs, parts=0, group=None, mode="auto"):
        import torch
        import torch.distributed as dist
        from . import FastKron
        self.torch, self.dist, self.group = torch, dist, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.M, self.ps, self.qs = int(M), [int(p) for p in ps], [int(q) for q in qs]
        G = self.world
        K, L = _prod(ps), _prod(qs)
        if G > 1 and (len(ps) < 2 or ps[0] % G or qs[0] % G or qs[1] % G):
            raise ValueError("column sharding over %d ranks needs N >= 2 and P1, Q1, Q2 divisible by it" % G)
        self.Kloc, self.Lloc = K // G, L // G
        self.h = FastKron()
        self.lib = _lib.get()
        self.pipe = None
        self._mapped = []
        if G == 1:
            _, te = self.h.sizes(self.M, self.ps, self.qs)
            self.t1 = torch.empty(te, dtype=torch.float32, device="cuda")
            self.t2 = torch.empty(te, dtype=torch.float32, device="cuda")
            self.result = torch.empty(self.M * L, dtype=torch.float32, device="cuda")
            self.parts, self.mode = 1, "single"
            return
        pipe = ctypes.c_void_p()
        _lib.check(self.lib.fkbMgPipeCreate(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(G), ctypes.c_uint32(self.M),
                                            ctypes.c_uint32(len(self.ps)), _lib.u32arr(self.ps), _lib.u32arr(self.qs),
                                            ctypes.c_int(int(parts)), ctypes.c_int({"auto": -1, "fused": 0, "staged": 1}[mode]),
                                            ctypes.byref(pipe)))
        self.pipe = pipe
        recv, result, flags = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        nparts, staged = ctypes.c_int(), ctypes.c_int()
        _lib.check(self.lib.fkbMgPipeLocalBuffers(pipe, ctypes.byref(recv), None, ctypes.byref(result), None,
                                                  ctypes.byref(flags), None, ctypes.byref(nparts), ctypes.byref(staged)))
        self.parts, self.mode = nparts.value, ("staged" if staged.value else "fused")
        self.result = torch.as_tensor(_RawCuda(result.value, self.M * self.Lloc), device="cuda")
        peers = [self._exchange(ptr.value) for ptr in (recv, result, flags)]
        _lib.check(self.lib.fkbMgPipeSetPeers(pipe, _lib.ptrarr(peers[0]), _lib.ptrarr(peers[1]), _lib.ptrarr(peers[2])))
        torch.cuda.synchronize()
        dist.barrier(group=group)

    # -- CUDA IPC plumbing -------------------------------------------------------------
    def _exchange(self, ptr):
        """All ranks learn a pointer through which they can reach every rank's buffer."""
        torch, dist = self.torch, self.dist
        hbuf = (ctypes.c_ubyte * 64)()
        rc = self.lib.fkbIpcExport(ctypes.c_void_p(ptr), hbuf)
        if rc != 0:
            raise RuntimeError("cudaIpcGetMemHandle failed (cuda error %d)" % rc)
        mine = torch.tensor(list(hbuf), dtype=torch.uint8, device="cuda")
        allh = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(allh, mine, group=self.group)
        out = []
        for r in range(self.world):
            if r == self.rank:
                out.append(ptr)
                continue
            raw = bytes(allh[r].cpu().tolist())
            hb = (ctypes.c_ubyte * 64).from_buffer_copy(raw)
            p = ctypes.c_void_p()
            rc = self.lib.fkbIpcOpen(hb, ctypes.byref(p))
            if rc != 0:
                raise RuntimeError("cudaIpcOpenMemHandle failed (cuda error %d)" % rc)
            out.append(p.value)
            self._mapped.append(p.value)
        return out

    # -- the product -------------------------------------------------------------------
    def run(self, x, fs):
        """x: this rank's [M, K/G] block (contiguous fp32 CUDA tensor); fs: the N factors.
        Enqueues the product on the handle's stream (the stream that was current when this
        object was made) and returns this rank's [M, L/G] block of the result, a view of an
        internal buffer that is complete in that stream's order."""
        if self.world == 1:
            self.h.raw_gemm("mkm", "s", self.M, self.ps, self.qs, x.data_ptr(), _lib.OP_N,
                            [f.data_ptr() for f in fs], _lib.OP_N, self.result.data_ptr(), 1.0, 0.0, 0,
                            self.t1.data_ptr(), self.t2.data_ptr())
            return self.result.view(self.M, -1)
        _lib.check(self.lib.fkbMgPipeRun(self.pipe, ctypes.c_void_p(x.data_ptr()),
                                         _lib.ptrarr([f.data_ptr() for f in fs])))
        return self.result.view(self.M, self.Lloc)

    def run_host(self, x_host, fs, z_host):
        """Same product on pinned HOST blocks x_host [M, K/G] -> z_host [M, L/G]: every row
        slice is copied in ahead of its passes and copied out as soon as it is complete.
        z_host is complete once the handle's stream has been synchronised."""
        if self.world == 1:
            raise ValueError("use fastkron_b200.HostGeMKM on a single GPU")
        _lib.check(self.lib.fkbMgPipeRunHost(self.pipe, ctypes.c_void_p(x_host.data_ptr()),
                                             _lib.ptrarr([f.data_ptr() for f in fs]),
                                             ctypes.c_void_p(z_host.data_ptr())))
        return z_host

    def close(self):
        if self.world > 1 and self.pipe is not None:
            self.torch.cuda.synchronize()
            self.dist.barrier(group=self.group)
            for p in self._mapped:
                self.lib.fkbIpcClose(ctypes.c_void_p(p))
            self._mapped = []
            self.dist.barrier(group=self.group)
            self.result = None
            self.lib.fkbMgPipeDestroy(self.pipe)
            self.pipe = None
        self.h.close()


def scatter_desc(phase, rank, world, ps, qs):
    """The redistribution map of a phase as a dict (host arithmetic only; no GPU needed):
    destination of output row (m, a, q), trailing position b is rank q // qPer at offset
    m*sM + a*sA + (q % qPer)*sQ + zOff + b, where the phase's chunk index n = m*aLoc + a."""
    out = (ctypes.c_longlong * 7)()
    rc = _lib.get().fkbMgScatterDesc(ctypes.c_int(phase), ctypes.c_int(rank), ctypes.c_int(world),
                                     ctypes.c_uint32(len(ps)), _lib.u32arr(ps), _lib.u32arr(qs), out)
    _lib.check(rc)
    keys = ("parts", "qPer", "aLoc", "sM", "sA", "sQ", "zOff")
    return {k: int(out[i]) for i, k in enumerate(keys)}


def emulate_rank_phase1(rank, world, M, ps, qs, x_block, fs):
    """numpy statement of phase 1 for one rank: returns a list of (dest_rank, flat_offsets,
    values) describing what this rank stores where.  Used by the CPU (gloo) tests."""
    G = world
    p1loc = ps[0] // G
    t = np.asarray(x_block, dtype=np.float64).reshape([M, p1loc] + [int(p) for p in ps[1:]])
    for i in range(len(ps) - 1, 0, -1):
        F = np.asarray(fs[i], dtype=np.float64).reshape(ps[i], qs[i])
        t = np.moveaxis(np.tensordot(t, F, axes=([i + 1], [0])), -1, i + 1)
    d = scatter_desc(1, rank, world, ps, qs)
    B = _prod(qs[2:])
    t = t.reshape(M, p1loc, qs[1], B)
    out = []
    for dst in range(G):
        qs_ = np.arange(dst * d["qPer"], (dst + 1) * d["qPer"])
        m, a, q, b = np.meshgrid(np.arange(M), np.arange(p1loc), qs_, np.arange(B), indexing="ij")
        off = m * d["sM"] + a * d["sA"] + (q % d["qPer"]) * d["sQ"] + d["zOff"] + b
        out.append((dst, off.reshape(-1), t[:, :, qs_, :].reshape(-1)))
    return out


def emulate_rank_phase2(rank, world, M, ps, qs, recv, f0):
    G = world
    B2 = (qs[1] // G) * _prod(qs[2:])
    t = np.asarray(recv, dtype=np.float64).reshape(M, ps[0], B2)
    F = np.asarray(f0, dtype=np.float64).reshape(ps[0], qs[0])
    t = np.einsum("mpb,pq->mqb", t, F)
    d = scatter_desc(2, rank, world, ps, qs)
    out = []
    for dst in range(G):
        qs_ = np.arange(dst * d["qPer"], (dst + 1) * d["qPer"])
        m, q, b = np.meshgrid(np.arange(M), qs_, np.arange(B2), indexing="ij")
        off = m * d["sM"] + (q % d["qPer"]) * d["sQ"] + d["zOff"] + b
        out.append((dst, off.reshape(-1), t[:, qs_, :].reshape(-1)))
    return out
