"""fastkron_b200 -- B200-native GeMKM / GeKMM behind the FastKron C API.

Host-side mirror of the reference's torch front-end (pyfastkron/fastkrontorch.py:
``gemkm`` :404-434, ``gekmm`` :437-466 of the reference): same function names,
argument order and meaning.  All arithmetic happens in ``libFastKron.so`` (CUDA,
sm_100a) reached through the C ABI of ``include/fastkron.h``; torch is used only
for device memory and streams.  There is no CPU path.
"""
import ctypes
from typing import List, Optional

from . import lib as _lib
from .lib import FastKronError  # noqa: F401

__all__ = ["FastKron", "gemkm", "gekmm", "gemkm_host", "gekmm_sizes", "FastKronError"]


def _torch():
    import torch
    return torch


class FastKron:
    """One library handle bound to the current CUDA device and a stream.

    Mirrors pyfastkron/fastkronhandle.py:1-88 of the reference (init, initCUDA with
    the current torch stream, gekmmSizes, x{gemkm,gekmm})."""

    def __init__(self, stream=None):
        torch = _torch()
        if not torch.cuda.is_available():
            raise RuntimeError("fastkron_b200 needs a CUDA device (no CPU fallback)")
        self.lib = _lib.get()
        self.h = ctypes.c_void_p()
        _lib.check(self.lib.fastKronInit(ctypes.byref(self.h), ctypes.c_uint32(_lib.BACKEND_CUDA)))
        self._stream_holder = None
        self._init_stream(stream)

    def _init_stream(self, stream):
        torch = _torch()
        s = stream if stream is not None else torch.cuda.current_stream()
        self._stream_holder = ctypes.c_void_p(s.cuda_stream)
        _lib.check(self.lib.fastKronInitCUDA(self.h, ctypes.byref(self._stream_holder)))
        self.stream = s

    def set_stream(self, stream):
        self._stream_holder = ctypes.c_void_p(stream.cuda_stream)
        _lib.check(self.lib.fastKronSetStream(self.h, ctypes.c_int(_lib.BACKEND_CUDA),
                                              ctypes.byref(self._stream_holder)))
        self.stream = stream

    def set_options(self, options):
        _lib.check(self.lib.fastKronSetOptions(self.h, ctypes.c_uint32(options)))

    def close(self):
        if self.h:
            self.lib.fastKronDestroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def version(self):
        return self.lib.fastKronVersion().decode()

    def sizes(self, M, ps, qs):
        ye, te = ctypes.c_size_t(), ctypes.c_size_t()
        _lib.check(self.lib.gekmmSizes(self.h, ctypes.c_uint32(M), ctypes.c_uint32(len(ps)),
                                       _lib.u32arr(ps), _lib.u32arr(qs), ctypes.byref(ye), ctypes.byref(te)))
        return ye.value, te.value

    def sizes_forward(self, M, ps, qs):
        n = len(ps)
        ye = ctypes.c_size_t()
        ie = (ctypes.c_size_t * max(n - 1, 1))()
        _lib.check(self.lib.gekmmSizesForward(self.h, ctypes.c_uint32(M), ctypes.c_uint32(n),
                                              _lib.u32arr(ps), _lib.u32arr(qs), ctypes.byref(ye), ie))
        return ye.value, [ie[i] for i in range(n - 1)]

    # -- raw calls on device pointers (ints); these are thin wrappers of the C ABI --
    def raw_gemm(self, mm, dtype_char, M, ps, qs, x_ptr, opx, f_ptrs, opf, z_ptr, alpha, beta, y_ptr,
                 t1_ptr, t2_ptr):
        """mm: "mkm" | "kmm"; dtype_char: "s" | "d"; op*: 1 (N) or 2 (T)."""
        n = len(ps)
        sc = ctypes.c_float if dtype_char == "s" else ctypes.c_double
        P, Q, F = _lib.u32arr(ps), _lib.u32arr(qs), _lib.ptrarr(f_ptrs)
        vp = ctypes.c_void_p
        if mm == "mkm":
            fn = getattr(self.lib, dtype_char + "gemkm")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(M), ctypes.c_uint32(n), P, Q,
                    vp(x_ptr), ctypes.c_int(opx), F, ctypes.c_int(opf), vp(z_ptr), sc(alpha), sc(beta),
                    vp(y_ptr), vp(t1_ptr), vp(t2_ptr))
        else:
            fn = getattr(self.lib, dtype_char + "gekmm")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(n), Q, P, ctypes.c_uint32(M),
                    F, ctypes.c_int(opf), vp(x_ptr), ctypes.c_int(opx), vp(z_ptr), sc(alpha), sc(beta),
                    vp(y_ptr), vp(t1_ptr), vp(t2_ptr))
        _lib.check(rc)

    def raw_forward(self, mm, dtype_char, M, ps, qs, x_ptr, opx, f_ptrs, opf, z_ptr, inter_ptrs):
        n = len(ps)
        P, Q, F = _lib.u32arr(ps), _lib.u32arr(qs), _lib.ptrarr(f_ptrs)
        I = _lib.ptrarr(inter_ptrs) if inter_ptrs else None
        vp = ctypes.c_void_p
        if mm == "mkm":
            fn = getattr(self.lib, dtype_char + "mkmForward")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(M), ctypes.c_uint32(n), P, Q,
                    vp(x_ptr), ctypes.c_int(opx), F, ctypes.c_int(opf), vp(z_ptr), I)
        else:
            fn = getattr(self.lib, dtype_char + "kmmForward")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(n), Q, P, ctypes.c_uint32(M),
                    F, ctypes.c_int(opf), vp(x_ptr), ctypes.c_int(opx), vp(z_ptr), I)
        _lib.check(rc)

    def raw_gemm_strided_batched(self, mm, dtype_char, M, ps, qs, x_ptr, opx, stride_x, f_ptrs, opf,
                                 stride_f, z_ptr, stride_z, alpha, beta, batch, y_ptr, stride_y,
                                 t1_ptr, t2_ptr):
        n = len(ps)
        sc = ctypes.c_float if dtype_char == "s" else ctypes.c_double
        P, Q, F = _lib.u32arr(ps), _lib.u32arr(qs), _lib.ptrarr(f_ptrs)
        SF = _lib.u64arr(stride_f)
        vp, u64 = ctypes.c_void_p, ctypes.c_uint64
        if mm == "mkm":
            fn = getattr(self.lib, dtype_char + "gemkmStridedBatched")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(M), ctypes.c_uint32(n), P, Q,
                    vp(x_ptr), ctypes.c_int(opx), u64(stride_x), F, ctypes.c_int(opf), SF,
                    vp(z_ptr), u64(stride_z), sc(alpha), sc(beta), ctypes.c_uint32(batch),
                    vp(y_ptr), u64(stride_y), vp(t1_ptr), vp(t2_ptr))
        else:
            fn = getattr(self.lib, dtype_char + "gekmmStridedBatched")
            rc = fn(self.h, ctypes.c_int(_lib.BACKEND_CUDA), ctypes.c_uint32(n), Q, P, ctypes.c_uint32(M),
                    F, ctypes.c_int(opf), SF, vp(x_ptr), ctypes.c_int(opx), u64(stride_x),
                    vp(z_ptr), u64(stride_z), sc(alpha), sc(beta), ctypes.c_uint32(batch),
                    vp(y_ptr), u64(stride_y), vp(t1_ptr), vp(t2_ptr))
        _lib.check(rc)


_default = {}


def _handle():
    torch = _torch()
    dev = torch.cuda.current_device()
    h = _default.get(dev)
    if h is None:
        h = FastKron()
        _default[dev] = h
    cur = torch.cuda.current_stream()
    if cur.cuda_stream != h.stream.cuda_stream:
        h.set_stream(cur)
    return h


def _as_op(t):
    """Return (storage tensor, is_transposed): a 2-D tensor that is the .T / .mT view
    of a contiguous tensor is passed as op = T without a copy, like
    pyfastkron/fastkronbase.py:129-137 of the reference does."""
    if t.dim() != 2:
        raise ValueError("expected a 2-D tensor")
    if t.is_contiguous():
        return t, False
    if t.t().is_contiguous():
        return t.t(), True
    return t.contiguous(), False


def gekmm_sizes(M, ps, qs):
    return _handle().sizes(M, ps, qs)


def _run(mm, x, fs, alpha, beta, y):
    torch = _torch()
    if not x.is_cuda:
        raise ValueError("fastkron_b200 computes on CUDA tensors only")
    if x.dtype not in (torch.float32, torch.float64):
        raise TypeError("only float32 and float64 are supported")
    h = _handle()
    dch = "s" if x.dtype == torch.float32 else "d"
    xs, trx = _as_op(x)
    fstore, trfs = [], []
    for f in fs:
        if f.dtype != x.dtype or f.device != x.device:
            raise TypeError("factors must match x in dtype and device")
        s, t = _as_op(f)
        fstore.append(s)
        trfs.append(t)
    # the C API has a single opFs for all factors: materialise the minority
    trf = sum(trfs) * 2 > len(trfs)
    for i, f in enumerate(fs):
        if trfs[i] != trf:
            fstore[i] = (f.t().contiguous() if trf else f.contiguous())
    if mm == "mkm":
        M, K = x.shape
        ps = [f.shape[0] for f in fs]
        qs = [f.shape[1] for f in fs]
    else:
        K, M = x.shape
        qs = [f.shape[0] for f in fs]
        ps = [f.shape[1] for f in fs]
    kk = 1
    for p in ps:
        kk *= p
    if kk != K:
        raise ValueError("product of factor sizes (%d) does not match x (%d)" % (kk, K))
    L = 1
    for q in qs:
        L *= q
    zshape = (M, L) if mm == "mkm" else (L, M)
    z = torch.empty(zshape, dtype=x.dtype, device=x.device)
    yptr = 0
    if y is not None and beta != 0:
        if tuple(y.shape) != zshape:
            raise ValueError("y has shape %s, expected %s" % (tuple(y.shape), zshape))
        y = y.contiguous()
        yptr = y.data_ptr()
    elif beta != 0:
        raise ValueError("beta != 0 needs y")
    _, te = h.sizes(M, ps, qs)
    t1 = torch.empty(te, dtype=x.dtype, device=x.device)
    t2 = torch.empty(te, dtype=x.dtype, device=x.device)
    h.raw_gemm(mm, dch, M, ps, qs, xs.data_ptr(), _lib.OP_T if trx else _lib.OP_N,
               [f.data_ptr() for f in fstore], _lib.OP_T if trf else _lib.OP_N,
               z.data_ptr(), float(alpha), float(beta), yptr, t1.data_ptr(), t2.data_ptr())
    return z


def gemkm(x, fs: List, alpha: float = 1.0, beta: float = 0.0, y: Optional[object] = None):
    """Z = alpha * X (F1 (x) ... (x) FN) + beta * Y with X of shape (M, prod P_i) and
    F_i of shape (P_i, Q_i)."""
    return _run("mkm", x, fs, alpha, beta, y)


def gekmm(fs: List, x, alpha: float = 1.0, beta: float = 0.0, y: Optional[object] = None):
    """Z = alpha * (F1 (x) ... (x) FN) X + beta * Y with F_i of shape (Q_i, P_i) and X of
    shape (prod P_i, M)."""
    return _run("kmm", x, fs, alpha, beta, y)


class HostGeMKM:
    """GeMKM on HOST operands: X and Z live in pinned host memory, the product runs on the GPU.

    Rows of a GeMKM are independent, so the call is cut into row slabs and pipelined on three
    streams: slab i+1 travels host->device while slab i is multiplied and slab i-1 travels
    device->host (PCIe is full duplex, so the two copy directions overlap as well).  Device
    memory holds two input slabs, two output slabs and one pair of temporaries, whatever the
    size of X.  The factors stay on the device.  Construct once per shape, call many times."""

    def __init__(self, M, ps, qs, dtype=None, rows_per_slab=None, device_budget_bytes=8 << 30):
        torch = _torch()
        self.torch = torch
        self.dtype = dtype or torch.float32
        self.es = 4 if self.dtype == torch.float32 else 8
        self.M, self.ps, self.qs = int(M), [int(p) for p in ps], [int(q) for q in qs]
        self.K = 1
        for p in self.ps:
            self.K *= p
        self.L = 1
        for q in self.qs:
            self.L *= q
        self.h = FastKron()
        if rows_per_slab is None:
            _, te1 = self.h.sizes(1, self.ps, self.qs)
            per_row = (2 * self.K + 2 * self.L + 2 * te1) * self.es
            rows_per_slab = max(1, min(self.M, device_budget_bytes // per_row))
            # about 32 slabs when possible, so that the un-overlapped first copy-in and last
            # copy-out are a small part of the call, but no slab below 256 MB of input (copy
            # and launch overheads stay negligible)
            floor_rows = -(-(256 << 20) // (self.K * self.es))
            rows_per_slab = max(1, min(rows_per_slab, max(-(-self.M // 32), floor_rows)))
        self.rows = int(rows_per_slab)
        _, te = self.h.sizes(self.rows, self.ps, self.qs)
        dev = "cuda"
        self.xd = [torch.empty(self.rows * self.K, dtype=self.dtype, device=dev) for _ in range(2)]
        self.zd = [torch.empty(self.rows * self.L, dtype=self.dtype, device=dev) for _ in range(2)]
        self.t1 = torch.empty(te, dtype=self.dtype, device=dev)
        self.t2 = torch.empty(te, dtype=self.dtype, device=dev)
        self.s_in, self.s_mm, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        self.h.set_stream(self.s_mm)

    def __call__(self, x_host, fs, z_host, alpha=1.0, beta=0.0, y_host=None):
        """x_host [M, K] and z_host [M, L]: pinned, contiguous host tensors; fs: device factors.
        Returns after z_host is complete.  beta*Y is not supported on this path."""
        torch = self.torch
        if beta != 0.0 or y_host is not None:
            raise ValueError("HostGeMKM computes alpha * X (F1 (x) ... (x) FN) only")
        dch = "s" if self.dtype == torch.float32 else "d"
        cur = torch.cuda.current_stream()
        for s in (self.s_in, self.s_mm, self.s_out):
            s.wait_stream(cur)
        xh, zh = x_host.view(self.M, self.K), z_host.view(self.M, self.L)
        nslab = -(-self.M // self.rows)
        in_done = [None, None]      # event: slab copied into xd[b]
        mm_done = [None, None]      # event: product of buffer b finished (xd[b] free, zd[b] full)
        out_done = [None, None]     # event: zd[b] copied out
        fptr = [f.data_ptr() for f in fs]
        for i in range(nslab):
            b = i & 1
            r0 = i * self.rows
            r = min(self.rows, self.M - r0)
            with torch.cuda.stream(self.s_in):
                if mm_done[b] is not None:
                    self.s_in.wait_event(mm_done[b])
                self.xd[b][: r * self.K].view(r, self.K).copy_(xh[r0:r0 + r], non_blocking=True)
                in_done[b] = self.s_in.record_event()
            with torch.cuda.stream(self.s_mm):
                self.s_mm.wait_event(in_done[b])
                if out_done[b] is not None:
                    self.s_mm.wait_event(out_done[b])
                self.h.raw_gemm("mkm", dch, r, self.ps, self.qs, self.xd[b].data_ptr(), _lib.OP_N, fptr, _lib.OP_N,
                                self.zd[b].data_ptr(), float(alpha), 0.0, 0, self.t1.data_ptr(), self.t2.data_ptr())
                mm_done[b] = self.s_mm.record_event()
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(mm_done[b])
                zh[r0:r0 + r].copy_(self.zd[b][: r * self.L].view(r, self.L), non_blocking=True)
                out_done[b] = self.s_out.record_event()
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_mm)
        # z_host is host memory the caller reads with the CPU: block until the last slab landed
        for ev in out_done:
            if ev is not None:
                ev.synchronize()
        return z_host

    def close(self):
        self.h.close()


def gemkm_host(x_host, fs, z_host, alpha=1.0):
    """One-shot form of HostGeMKM (allocates its device slabs on every call)."""
    M = x_host.shape[0]
    ps = [f.shape[0] for f in fs]
    qs = [f.shape[1] for f in fs]
    op = HostGeMKM(M, ps, qs, dtype=x_host.dtype)
    try:
        op(x_host, fs, z_host, alpha)
        _torch().cuda.synchronize()
    finally:
        op.close()
    return z_host
