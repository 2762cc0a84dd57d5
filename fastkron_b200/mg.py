"""Column-sharded multi-GPU GeMKM for one-process-per-GPU hosts (torch.distributed).

The reference's multi-GPU API (include/fastkronMg.h of the reference) is one process
driving all GPUs; `libFastKron.so` implements that API as well.  A torchrun-style host
has one process per GPU instead, so the same two phases are exposed per rank
(`fkbMgRankPhase1/2` in csrc/mg.cu) and this module supplies what the single process
did with pointers and stream events: buffers every peer can store into (CUDA IPC) and
the barriers between the phases (a one-element all-reduce enqueued on the stream).

Rank g of G owns columns [g*K/G, (g+1)*K/G) of X and of the result, all M rows, and a
copy of every factor.  Phase 1 contracts the trailing modes locally and redistributes
with peer stores from inside the last kernel; phase 2 contracts the leading mode and
stores each result row into the rank that owns it.
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


class RankGeMKM:
    """One rank of a column-sharded fp32 GeMKM  Z = X (F1 (x) ... (x) FN)."""

    def __init__(self, M, ps, qs, group=None):
        import torch
        import torch.distributed as dist
        from . import FastKron
        self.torch, self.dist = torch, dist
        self.group = group
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
        # widest local intermediate: the global one divided by G
        cols = K
        widest = 0
        for p, q in reversed(list(zip(self.ps, self.qs))):
            cols = cols // p * q
            widest = max(widest, cols)
        if len(ps) == 1:
            widest = max(K, L)
        self.tmp_elems = self.M * (widest // G)
        dev = torch.cuda.current_device()
        self.t1 = torch.empty(self.tmp_elems, dtype=torch.float32, device="cuda")
        self.t2 = torch.empty(self.tmp_elems, dtype=torch.float32, device="cuda")
        self._raw = []
        if G == 1:
            self.result = torch.empty(self.M * L, dtype=torch.float32, device="cuda")
            self.recv = None
            return
        B = _prod(self.qs[2:])
        recv_elems = self.M * self.ps[0] * (self.qs[1] // G) * B
        self.recv_ptr = self._alloc(recv_elems * 4)
        self.result_ptr = self._alloc(self.M * self.Lloc * 4)
        self.recv = torch.as_tensor(_RawCuda(self.recv_ptr, recv_elems), device="cuda")
        self.result = torch.as_tensor(_RawCuda(self.result_ptr, self.M * self.Lloc), device="cuda")
        self.peer_recv = self._exchange(self.recv_ptr)
        self.peer_result = self._exchange(self.result_ptr)
        self._flag = torch.zeros(1, dtype=torch.float32, device="cuda")
        _ = dev

    # -- CUDA IPC plumbing -------------------------------------------------------------
    def _alloc(self, nbytes):
        p = ctypes.c_void_p()
        rc = self.lib.fkbIpcAlloc(ctypes.byref(p), ctypes.c_size_t(nbytes))
        if rc != 0:
            raise MemoryError("cudaMalloc of %d bytes failed (cuda error %d)" % (nbytes, rc))
        self._raw.append(p.value)
        return p.value

    def _exchange(self, ptr):
        """All ranks learn a pointer through which they can store into every rank's buffer."""
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
        return out

    def barrier(self):
        """Stream-ordered barrier: nothing enqueued after it starts before every rank's
        earlier work on its stream has finished."""
        self.dist.all_reduce(self._flag, group=self.group)

    # -- the product -------------------------------------------------------------------
    def run(self, x, fs):
        """x: this rank's [M, K/G] block (contiguous fp32 CUDA tensor); fs: the N factors.
        Returns this rank's [M, L/G] block of the result (a view of an internal buffer)."""
        n = len(self.ps)
        if self.world == 1:
            self.h.raw_gemm("mkm", "s", self.M, self.ps, self.qs, x.data_ptr(), _lib.OP_N,
                            [f.data_ptr() for f in fs], _lib.OP_N, self.result.data_ptr(), 1.0, 0.0, 0,
                            self.t1.data_ptr(), self.t2.data_ptr())
            return self.result.view(self.M, -1)
        L = self.lib
        P, Q = _lib.u32arr(self.ps), _lib.u32arr(self.qs)
        F = _lib.ptrarr([f.data_ptr() for f in fs])
        _lib.check(L.fkbMgRankPhase1(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                     ctypes.c_uint32(self.M), ctypes.c_uint32(n), P, Q,
                                     ctypes.c_void_p(x.data_ptr()), F, ctypes.c_void_p(self.t1.data_ptr()),
                                     ctypes.c_void_p(self.t2.data_ptr()), _lib.ptrarr(self.peer_recv)))
        self.barrier()
        _lib.check(L.fkbMgRankPhase2(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                     ctypes.c_uint32(self.M), ctypes.c_uint32(n), P, Q,
                                     ctypes.c_void_p(self.recv_ptr), ctypes.c_void_p(fs[0].data_ptr()),
                                     _lib.ptrarr(self.peer_result)))
        self.barrier()
        return self.result.view(self.M, self.Lloc)

    def close(self):
        if self.world > 1:
            self.torch.cuda.synchronize()
            self.dist.barrier(group=self.group)
            for plist in (getattr(self, "peer_recv", []), getattr(self, "peer_result", [])):
                for r, p in enumerate(plist):
                    if r != self.rank:
                        self.lib.fkbIpcClose(ctypes.c_void_p(p))
            self.dist.barrier(group=self.group)
            self.recv = self.result = None
            for p in self._raw:
                self.lib.fkbIpcFree(ctypes.c_void_p(p))
            self._raw = []
        self.h.close()


class StagedRankGeMKM(RankGeMKM):
    """Same product, other transport: the kernels write per-destination blocks into local
    staging buffers and copy engines move them (cudaMemcpyAsync / cudaMemcpy2DAsync into the
    peers' IPC-mapped buffers) on a second stream.  The NVLink traffic then costs no SM time
    and overlaps whatever else the GPU computes.  For the large-factor shapes (64, 128) only;
    RankGeMKM (stores fused into the kernels) covers everything else."""

    def __init__(self, M, ps, qs, group=None):
        super().__init__(M, ps, qs, group=group)
        torch = self.torch
        if self.world == 1:
            return
        G = self.world
        B = _prod(self.qs[2:])
        self.blk1 = self.M * (self.ps[0] // G) * (self.qs[1] // G) * B
        self.B2 = (self.qs[1] // G) * B
        self.blk2 = self.M * (self.qs[0] // G) * self.B2
        self.stage1 = torch.empty(G * self.blk1, dtype=torch.float32, device="cuda")
        self.stage2 = torch.empty(G * self.blk2, dtype=torch.float32, device="cuda")
        # copies and barriers go first whenever they are ready; the compute kernels retire
        # their CTAs every few tiles so that the barrier's small kernel finds a free slot
        self.copy_stream = torch.cuda.Stream(priority=-1)
        self.lib.fkbSetTilesPerCta(self.h.h, ctypes.c_int(int(__import__("os").environ.get("FASTKRON_MG_TILES_PER_CTA", "8"))))

    def _copies1(self, s):
        L, g, G = self.lib, self.rank, self.world
        for k in range(G):
            d = (g + k) % G
            dst = self.peer_recv[d] + 4 * g * self.blk1
            rc = L.fkbCopyAsync(ctypes.c_void_p(dst), ctypes.c_void_p(self.stage1.data_ptr() + 4 * d * self.blk1),
                                ctypes.c_size_t(4 * self.blk1), ctypes.c_void_p(s.cuda_stream))
            if rc != 0:
                raise RuntimeError("peer copy failed (cuda error %d)" % rc)

    def _copies2(self, s):
        L, g, G = self.lib, self.rank, self.world
        rows = self.M * (self.qs[0] // G)
        dpitch = 4 * self.Lloc // (self.qs[0] // G)         # bytes of one (m, q1) row of the result
        for k in range(G):
            d = (g + k) % G
            dst = self.peer_result[d] + 4 * g * self.B2
            rc = L.fkbCopy2DAsync(ctypes.c_void_p(dst), ctypes.c_size_t(dpitch),
                                  ctypes.c_void_p(self.stage2.data_ptr() + 4 * d * self.blk2),
                                  ctypes.c_size_t(4 * self.B2), ctypes.c_size_t(4 * self.B2), ctypes.c_size_t(rows),
                                  ctypes.c_void_p(s.cuda_stream))
            if rc != 0:
                raise RuntimeError("peer 2-D copy failed (cuda error %d)" % rc)

    def run(self, x, fs, after=None):
        """Enqueues the whole step; returns (result view, event that marks its completion).
        `after`: optional event the local passes wait for (used to stagger row slices)."""
        torch = self.torch
        if self.world == 1:
            return super().run(x, fs), None
        n = len(self.ps)
        L = self.lib
        sC, sX = self.h.stream, self.copy_stream
        P, Q = _lib.u32arr(self.ps), _lib.u32arr(self.qs)
        F = _lib.ptrarr([f.data_ptr() for f in fs])
        with torch.cuda.stream(sC):
            if after is not None:
                sC.wait_event(after)
            _lib.check(L.fkbMgRankPhase1Staged(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                               ctypes.c_uint32(self.M), ctypes.c_uint32(n), P, Q,
                                               ctypes.c_void_p(x.data_ptr()), F, ctypes.c_void_p(self.t1.data_ptr()),
                                               ctypes.c_void_p(self.t2.data_ptr()),
                                               ctypes.c_void_p(self.stage1.data_ptr()), ctypes.c_int(1)))
            self.local_done = sC.record_event()
            _lib.check(L.fkbMgRankPhase1Staged(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                               ctypes.c_uint32(self.M), ctypes.c_uint32(n), P, Q,
                                               ctypes.c_void_p(x.data_ptr()), F, ctypes.c_void_p(self.t1.data_ptr()),
                                               ctypes.c_void_p(self.t2.data_ptr()),
                                               ctypes.c_void_p(self.stage1.data_ptr()), ctypes.c_int(2)))
            e1 = sC.record_event()
        with torch.cuda.stream(sX):
            sX.wait_event(e1)
            self._copies1(sX)
            self.barrier()
            e2 = sX.record_event()
        with torch.cuda.stream(sC):
            sC.wait_event(e2)
            _lib.check(L.fkbMgRankPhase2Staged(self.h.h, ctypes.c_int(self.rank), ctypes.c_int(self.world),
                                               ctypes.c_uint32(self.M), ctypes.c_uint32(n), P, Q,
                                               ctypes.c_void_p(self.recv_ptr), ctypes.c_void_p(fs[0].data_ptr()),
                                               ctypes.c_void_p(self.stage2.data_ptr())))
            e3 = sC.record_event()
        with torch.cuda.stream(sX):
            sX.wait_event(e3)
            self._copies2(sX)
            self.barrier()
            e4 = sX.record_event()
        return self.result.view(self.M, self.Lloc), e4


class PipelinedRankGeMKM:
    """The same product with the rows cut into `parts` independent slices, each a rank object
    of its own with its own streams, buffers and communicator.

    Why: two of the four passes of a column-sharded step hand their output to the peers and
    are bound by NVLink, the other two by arithmetic.  Rows are independent, so one slice's
    transfers can overlap another slice's arithmetic.
      mode "staged": kernels fill local per-destination blocks, copy engines ship them
                     (large-factor shapes); compute kernels run at full width.
      mode "fused" : the producing kernels store straight into the peers (any shape); the
                     slices share the SMs (1/parts each) and start staggered."""

    def __init__(self, M, ps, qs, parts=2, group=None, mode="staged"):
        import torch
        import torch.distributed as dist
        self.torch = torch
        self.parts = parts if M % parts == 0 else 1
        self.mode = mode
        self.M, self.Mp = int(M), int(M) // self.parts
        self.streams = [torch.cuda.Stream() for _ in range(self.parts)]
        self.slices = []
        for i, s in enumerate(self.streams):
            # a communicator of its own per slice: barriers of different slices must not
            # queue behind one another on a shared collective stream
            g = group
            if dist.is_initialized() and dist.get_world_size(group) > 1 and i > 0:
                g = dist.new_group(ranks=list(range(dist.get_world_size())))
            with torch.cuda.stream(s):
                cls = StagedRankGeMKM if mode == "staged" else RankGeMKM
                r = cls(self.Mp, ps, qs, group=g)
                r.h.set_stream(s)
                if mode == "fused":
                    r.lib.fkbSetSmShare(r.h.h, ctypes.c_float(1.0 / self.parts))
                self.slices.append(r)
        self.world, self.rank = self.slices[0].world, self.slices[0].rank
        self.Lloc = self.slices[0].Lloc
        self._done = [None] * self.parts
        torch.cuda.synchronize()

    def run(self, x, fs, join=True):
        """x: this rank's [M, K/G] block.  Returns the per-slice result blocks ([M/parts, L/G]
        each, in row order).  join=False leaves the slices free-running from one call to the
        next (call join() before reading results), which keeps them out of phase."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        xs = x.view(self.M, -1)
        outs = []
        if join:
            for r, s in zip(self.slices, self.streams):
                s.wait_stream(cur)
                if self.mode == "staged" and r.world > 1:
                    r.copy_stream.wait_stream(cur)
        if self.world == 1:
            for i, (r, s) in enumerate(zip(self.slices, self.streams)):
                with torch.cuda.stream(s):
                    outs.append(RankGeMKM.run(r, xs[i * self.Mp:(i + 1) * self.Mp], fs))
            if join:
                self.join()
            return outs
        if self.mode == "staged":
            prev = None
            for i, r in enumerate(self.slices):
                z, done = r.run(xs[i * self.Mp:(i + 1) * self.Mp], fs, after=prev)
                prev = r.local_done
                self._done[i] = done
                outs.append(z)
            if join:
                self.join()
            return outs
        n = len(self.slices[0].ps)
        L = self.slices[0].lib
        F = _lib.ptrarr([f.data_ptr() for f in fs])
        prev_local_done = None
        for i, (r, s) in enumerate(zip(self.slices, self.streams)):
            with torch.cuda.stream(s):
                P, Q = _lib.u32arr(r.ps), _lib.u32arr(r.qs)
                xi = xs[i * self.Mp:(i + 1) * self.Mp]
                args = (r.h.h, ctypes.c_int(r.rank), ctypes.c_int(r.world), ctypes.c_uint32(r.M),
                        ctypes.c_uint32(n), P, Q, ctypes.c_void_p(xi.data_ptr()), F,
                        ctypes.c_void_p(r.t1.data_ptr()), ctypes.c_void_p(r.t2.data_ptr()),
                        _lib.ptrarr(r.peer_recv))
                if prev_local_done is not None:
                    s.wait_event(prev_local_done)
                _lib.check(L.fkbMgRankPhase1Stage(*args, ctypes.c_int(1)))
                prev_local_done = s.record_event()
                _lib.check(L.fkbMgRankPhase1Stage(*args, ctypes.c_int(2)))
                r.barrier()
        for i, (r, s) in enumerate(zip(self.slices, self.streams)):
            with torch.cuda.stream(s):
                P, Q = _lib.u32arr(r.ps), _lib.u32arr(r.qs)
                _lib.check(L.fkbMgRankPhase2(r.h.h, ctypes.c_int(r.rank), ctypes.c_int(r.world),
                                             ctypes.c_uint32(r.M), ctypes.c_uint32(n), P, Q,
                                             ctypes.c_void_p(r.recv_ptr), ctypes.c_void_p(fs[0].data_ptr()),
                                             _lib.ptrarr(r.peer_result)))
                r.barrier()
                outs.append(r.result.view(r.M, r.Lloc))
        if join:
            self.join()
        return outs

    def join(self):
        cur = self.torch.cuda.current_stream()
        for r, s in zip(self.slices, self.streams):
            cur.wait_stream(s)
            if self.mode == "staged" and r.world > 1:
                cur.wait_stream(r.copy_stream)

    def close(self):
        for r in self.slices:
            r.close()


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
