"""ctypes front-ends of the two CPU oracles plus a tiny numpy restatement.

All functions take and return numpy arrays; ``mm`` is "mkm" or "kmm"; ``opx`` /
``opf`` are "N" or "T" with the meaning of the reference's fastKronOp
(include/fastkron.h:21-30 of the reference): "T" = the buffer holds the
transpose of the row-major operand.
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT_PATH = os.path.join(_HERE, "libkron_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libFastKron.so")

_OP = {"N": 1, "T": 2}
_BACKEND_X86 = 2


def port_available():
    return os.path.exists(_PORT_PATH)


def ref_available():
    return os.path.exists(_REF_PATH)


def _shapes(mm, M, ps, qs):
    K = int(np.prod([int(p) for p in ps], dtype=object))
    L = int(np.prod([int(q) for q in qs], dtype=object))
    zshape = (M, L) if mm == "mkm" else (L, M)
    return K, L, zshape


_port = None


def _port_lib():
    global _port
    if _port is None:
        _port = ctypes.CDLL(_PORT_PATH)
    return _port


def port_gekmm(mm, x, fs, ps, qs, M, opx="N", opf="N", alpha=1.0, beta=0.0, y=None,
               exact=False, want_intermediates=False):
    """Run the C restatement.  x, fs[i], y are the *stored* buffers (any shape, C order)."""
    lib = _port_lib()
    dt = x.dtype
    assert dt in (np.float32, np.float64)
    name = "oracle_gekmm_" + ("f32" if dt == np.float32 else "f64") + ("_exact" if exact else "")
    fn = getattr(lib, name)
    fn.restype = ctypes.c_int
    N = len(fs)
    K, L, zshape = _shapes(mm, M, ps, qs)
    x = np.ascontiguousarray(x)
    fs = [np.ascontiguousarray(f, dtype=dt) for f in fs]
    z = np.empty(zshape, dtype=dt)
    Ps = (ctypes.c_uint32 * N)(*[int(p) for p in ps])
    Qs = (ctypes.c_uint32 * N)(*[int(q) for q in qs])
    Fp = (ctypes.c_void_p * N)(*[f.ctypes.data for f in fs])
    inter = None
    Ip = None
    if want_intermediates and N > 1:
        inter = []
        cols = K
        sizes = {}
        for i in range(N - 1, 0, -1):
            cols = cols // int(ps[i]) * int(qs[i])
            sizes[i] = cols
        for i in range(1, N):
            shp = (M, sizes[i]) if mm == "mkm" else (sizes[i], M)
            inter.append(np.empty(shp, dtype=dt))
        Ip = (ctypes.c_void_p * (N - 1))(*[a.ctypes.data for a in inter])
    yp = None
    if y is not None:
        y = np.ascontiguousarray(y, dtype=dt)
        yp = ctypes.c_void_p(y.ctypes.data)
    rc = fn(ctypes.c_int(1 if mm == "kmm" else 0), ctypes.c_uint32(M), ctypes.c_uint32(N), Ps, Qs,
            ctypes.c_void_p(x.ctypes.data), ctypes.c_int(_OP[opx]), Fp, ctypes.c_int(_OP[opf]),
            ctypes.c_void_p(z.ctypes.data), ctypes.c_double(alpha), ctypes.c_double(beta), yp, Ip)
    if rc != 0:
        raise MemoryError("oracle allocation failed")
    return (z, inter) if want_intermediates else z


def numpy_gekmm(mm, x, fs, ps, qs, M, opx="N", opf="N", alpha=1.0, beta=0.0, y=None):
    """Definition-level check in float64: builds op(X), op(F_i) and contracts mode by
    mode with einsum (no Kronecker matrix is materialised).  Small cases only."""
    N = len(fs)
    K, L, zshape = _shapes(mm, M, ps, qs)
    xd = np.asarray(x, dtype=np.float64).reshape(-1)
    if mm == "mkm":
        X = xd.reshape(M, K) if opx == "N" else xd.reshape(K, M).T
    else:
        X = xd.reshape(K, M).T if opx == "N" else xd.reshape(M, K)      # X as M x K
    t = X.reshape([M] + [int(p) for p in ps])
    for i in range(N - 1, -1, -1):
        P, Q = int(ps[i]), int(qs[i])
        fd = np.asarray(fs[i], dtype=np.float64).reshape(-1)
        if mm == "mkm":
            F = fd.reshape(P, Q) if opf == "N" else fd.reshape(Q, P).T
        else:
            F = fd.reshape(Q, P).T if opf == "N" else fd.reshape(P, Q)  # F as P x Q
        t = np.moveaxis(np.tensordot(t, F, axes=([i + 1], [0])), -1, i + 1)
    Zm = alpha * t.reshape(M, L)
    Z = Zm if mm == "mkm" else Zm.T
    if beta != 0.0 and y is not None:
        Z = Z + beta * np.asarray(y, dtype=np.float64).reshape(zshape)
    return np.ascontiguousarray(Z)


class RefLib:
    """The unmodified reference x86 backend behind its own C API."""

    def __init__(self, threads=None):
        if threads is not None:
            os.environ["OMP_NUM_THREADS"] = str(int(threads))
        self.lib = ctypes.CDLL(_REF_PATH)
        self.lib.fastKronGetErrorString.restype = ctypes.c_char_p
        self.h = ctypes.c_void_p()
        rc = self.lib.fastKronInit(ctypes.byref(self.h), ctypes.c_uint32(_BACKEND_X86))
        if rc != 0:
            raise RuntimeError("reference fastKronInit failed: %d" % rc)
        rc = self.lib.fastKronInitX86(self.h)
        if rc != 0:
            raise RuntimeError("reference fastKronInitX86 failed: %d" % rc)

    def close(self):
        if self.h:
            self.lib.fastKronDestroy(self.h)
            self.h = None

    def sizes(self, M, ps, qs):
        N = len(ps)
        Ps = (ctypes.c_uint32 * N)(*[int(p) for p in ps])
        Qs = (ctypes.c_uint32 * N)(*[int(q) for q in qs])
        ye, te = ctypes.c_size_t(), ctypes.c_size_t()
        rc = self.lib.gekmmSizes(self.h, ctypes.c_uint32(M), ctypes.c_uint32(N), Ps, Qs,
                                 ctypes.byref(ye), ctypes.byref(te))
        if rc != 0:
            raise RuntimeError("reference gekmmSizes failed: %d" % rc)
        return ye.value, te.value

    def gekmm(self, mm, x, fs, ps, qs, M, opx="N", opf="N", alpha=1.0, beta=0.0, y=None, z=None,
              temps=None):
        dt = x.dtype
        N = len(fs)
        K, L, zshape = _shapes(mm, M, ps, qs)
        x = np.ascontiguousarray(x)
        fs = [np.ascontiguousarray(f, dtype=dt) for f in fs]
        # Z and the temporaries are zero-filled on purpose: with uninitialised
        # scratch the reference's partial-tile kernels can pick up NaN/Inf garbage
        # (observed for fp32 MKM with distinct non-square factors and mixed ops).
        if z is None:
            z = np.zeros(zshape, dtype=dt)
        _, te = self.sizes(M, ps, qs)
        if temps is None:
            temps = (np.zeros(te, dtype=dt), np.zeros(te, dtype=dt))
        Ps = (ctypes.c_uint32 * N)(*[int(p) for p in ps])
        Qs = (ctypes.c_uint32 * N)(*[int(q) for q in qs])
        Fp = (ctypes.c_void_p * N)(*[f.ctypes.data for f in fs])
        yp = None
        if y is not None:
            y = np.ascontiguousarray(y, dtype=dt)
            yp = ctypes.c_void_p(y.ctypes.data)
        sc = ctypes.c_float if dt == np.float32 else ctypes.c_double
        pre = "s" if dt == np.float32 else "d"
        if mm == "mkm":
            fn = getattr(self.lib, pre + "gemkm")
            rc = fn(self.h, ctypes.c_int(_BACKEND_X86), ctypes.c_uint32(M), ctypes.c_uint32(N), Ps, Qs,
                    ctypes.c_void_p(x.ctypes.data), ctypes.c_int(_OP[opx]), Fp, ctypes.c_int(_OP[opf]),
                    ctypes.c_void_p(z.ctypes.data), sc(alpha), sc(beta), yp,
                    ctypes.c_void_p(temps[0].ctypes.data), ctypes.c_void_p(temps[1].ctypes.data))
        else:
            fn = getattr(self.lib, pre + "gekmm")
            rc = fn(self.h, ctypes.c_int(_BACKEND_X86), ctypes.c_uint32(N), Qs, Ps, ctypes.c_uint32(M),
                    Fp, ctypes.c_int(_OP[opf]), ctypes.c_void_p(x.ctypes.data), ctypes.c_int(_OP[opx]),
                    ctypes.c_void_p(z.ctypes.data), sc(alpha), sc(beta), yp,
                    ctypes.c_void_p(temps[0].ctypes.data), ctypes.c_void_p(temps[1].ctypes.data))
        if rc != 0:
            raise RuntimeError("reference call failed: %d %s" % (rc, self.lib.fastKronGetErrorString(rc)))
        return z


def ref_gekmm(*args, **kw):
    """One reference call on a FRESH handle.  A long-lived reference handle keeps
    per-thread tile caches between calls, and after some shape sequences stale cache
    contents leak into later fp32 results as NaN (seen for 5x5^4 after other shapes and
    for the distinct 14x15,19x13,34x23,21x34 case); a new handle per call avoids that."""
    ref = RefLib()
    try:
        return ref.gekmm(*args, **kw)
    finally:
        ref.close()
