"""Seeded synthetic operands for the parity tests and the benchmark.

The reference benchmarks on synthetic matrices as well (all-ones or small random
integers, tests/benchmarks/run_benchmarks.py:217-235 and tests/testBase.h:82 of the
reference); here every value is a pure function of (seed, index), so the same
operand can be produced on the host (numpy) and in HBM (CUDA kernel in
csrc/synth.cu) bit for bit, in any chunking.

uniform:  u(seed, i) = SplitMix64(seed*C + i) -> top 53 bits -> [-1, 1)
normal:   Box-Muller on two uniform streams (host only)
"""
import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SYNTH_PATH = os.path.join(_HERE, "libfkb_synth.so")
_slib = None

_C = np.uint64(0xD1342543DE82EF95)
_G = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def _splitmix64(z):
    with np.errstate(over="ignore"):
        z = z + _G
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def _unit(seed, n, offset):
    """float64 values in [0, 1) for indices offset .. offset+n-1."""
    with np.errstate(over="ignore"):
        idx = np.arange(offset, offset + n, dtype=np.uint64)
        h = _splitmix64(np.uint64(seed) * _C + idx)
    return (h >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def _helper():
    """The helper library (csrc/synth.cu), or None when it has not been built."""
    global _slib
    if _slib is None and os.path.exists(_SYNTH_PATH):
        _slib = ctypes.CDLL(_SYNTH_PATH)
    return _slib


def uniform(seed, n, dtype=np.float32, offset=0, chunk=1 << 24, force_numpy=False):
    """n values uniform in [-1, 1) as a 1-D numpy array.  Large requests go through the
    multi-threaded C generator of the helper library when it is there (same bits)."""
    out = np.empty(n, dtype=dtype)
    lib = None if (force_numpy or n < (1 << 20)) else _helper()
    if lib is not None and hasattr(lib, "fkbFillUniformHostF32") and np.dtype(dtype) in (np.float32, np.float64):
        fn = lib.fkbFillUniformHostF32 if np.dtype(dtype) == np.float32 else lib.fkbFillUniformHostF64
        fn.restype = None
        fn(ctypes.c_void_p(out.ctypes.data), ctypes.c_uint64(n), ctypes.c_uint64(seed), ctypes.c_uint64(offset))
        return out
    for s in range(0, n, chunk):
        m = min(chunk, n - s)
        out[s:s + m] = (_unit(seed, m, offset + s) * 2.0 - 1.0).astype(dtype)
    return out


def normal(seed, n, dtype=np.float32, offset=0, chunk=1 << 23):
    """n standard-normal values (Box-Muller over the streams seed and seed+2^32)."""
    out = np.empty(n, dtype=dtype)
    for s in range(0, n, chunk):
        m = min(chunk, n - s)
        u1 = 1.0 - _unit(seed, m, offset + s)                 # (0, 1]
        u2 = _unit(seed + (1 << 32), m, offset + s)
        out[s:s + m] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(dtype)
    return out



def fill_uniform_cuda(t, seed, offset=0):
    """Fill the contiguous CUDA tensor t (float32/float64) with uniform(seed) values,
    element i of the flattened tensor getting stream index offset+i."""
    import torch
    if _helper() is None:
        raise ImportError("%s is missing -- run `make -C fastkron_b200/csrc`" % _SYNTH_PATH)
    assert t.is_cuda and t.is_contiguous()
    fn = _slib.fkbFillUniformF32 if t.dtype == torch.float32 else _slib.fkbFillUniformF64
    rc = fn(ctypes.c_void_p(t.data_ptr()), ctypes.c_uint64(t.numel()), ctypes.c_uint64(seed),
            ctypes.c_uint64(offset), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError("fill kernel launch failed: cuda error %d" % rc)
    return t
