"""ctypes binding of the C ABI in include/fastkron.h / include/fastkronMg.h.

This is the raw boundary: every function takes plain integers and pointers,
exactly as the reference's pybind shim passes them (pyfastkron/pywrapper.cpp:90-98
of the reference passes device pointers as uint64).  There is no CPU fallback: if
the shared library is missing the import fails.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libFastKron.so")

# enum values of include/fastkron.h
OP_N, OP_T = 1, 2
BACKEND_NONE, BACKEND_X86, BACKEND_ARM, BACKEND_CUDA, BACKEND_HIP = 1, 2, 4, 8, 16
OPT_NONE, OPT_USE_FUSION, OPT_TUNE = 1, 2, 4
OPT_TF32, OPT_TF32X3 = 8, 16          # not in the reference: tensor-core opt-ins for fp32 large factors
(SUCCESS, BACKEND_NOT_AVAILABLE, INVALID_MEMORY_ACCESS, KERNEL_NOT_FOUND, INVALID_ARGUMENT,
 INVALID_KMM_PROBLEM, OTHER_ERROR) = range(7)

# every symbol the headers declare; tests check that the library exports all of them
API_SYMBOLS = [
    "fastKronVersion", "fastKronCUDAArchs", "fastKronGetErrorString", "fastKronGetBackends",
    "fastKronInit", "fastKronInitAllBackends", "fastKronSetOptions", "fastKronDestroy",
    "fastKronInitCUDA", "fastKronInitHIP", "fastKronInitX86", "fastKronSetStream",
    "gekmmSizes", "gekmmSizesForward",
    "sgemkm", "dgemkm", "sgekmm", "dgekmm",
    "sgemkmStridedBatched", "dgemkmStridedBatched", "sgekmmStridedBatched", "dgekmmStridedBatched",
    "smkmForward", "dmkmForward", "skmmForward", "dkmmForward",
    "smkmForwardStridedBatched", "dmkmForwardStridedBatched",
    "skmmForwardStridedBatched", "dkmmForwardStridedBatched",
    "fastKronMgInitCUDA", "fastKronMgSGEMM", "fastKronMgAllocX", "fastKronMgGatherY",
    "sgemkmNoAlloc",
]
NOALLOC_MAX_TEMP_ELEMS = 2 << 20


class FastKronError(RuntimeError):
    def __init__(self, code, text):
        super().__init__("fastKron error %d: %s" % (code, text))
        self.code = code


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "fastkron_b200: %s is missing -- build it with `make -C fastkron_b200/csrc` "
            "(or __graft_entry__.build()); there is no CPU fallback" % LIB_PATH)
    lib = ctypes.CDLL(LIB_PATH)
    lib.fastKronVersion.restype = ctypes.c_char_p
    lib.fastKronCUDAArchs.restype = ctypes.c_char_p
    lib.fastKronGetErrorString.restype = ctypes.c_char_p
    lib.fastKronGetBackends.restype = ctypes.c_uint32
    lib.fastKronDestroy.restype = None
    lib.fkbGemmTcLaunches.restype = ctypes.c_ulonglong
    return lib


_lib = None


def get():
    global _lib
    if _lib is None:
        _lib = load()
    return _lib


def check(rc):
    if rc != SUCCESS:
        txt = get().fastKronGetErrorString(ctypes.c_int(rc))
        raise FastKronError(rc, txt.decode() if txt else "?")


def u32arr(vals):
    return (ctypes.c_uint32 * len(vals))(*[int(v) for v in vals])


def u64arr(vals):
    return (ctypes.c_uint64 * len(vals))(*[int(v) for v in vals])


def ptrarr(vals):
    return (ctypes.c_void_p * len(vals))(*[int(v) for v in vals])
