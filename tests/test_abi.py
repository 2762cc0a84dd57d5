"""CPU tests of the drop-in boundary: the shared library loads without a GPU, exports
every symbol include/fastkron.h and include/fastkronMg.h declare, answers the
device-independent calls like the reference does, and plans the benchmark shapes as
documented.  No compute call is made here."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from fastkron_b200 import lib as fk  # noqa: E402
import oracle  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    return fk.get()


def declared_symbols():
    names = set()
    for h in ("fastkron.h", "fastkronMg.h"):
        txt = open(os.path.join(ROOT, "include", h)).read()
        txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
        for m in re.finditer(r"^\s*(?:const char\*|uint32_t|void|fastKronError)\s+(\w+)\s*\(", txt, re.M):
            names.add(m.group(1))
    return names


def test_every_declared_symbol_is_exported(L):
    decl = declared_symbols()
    assert decl == set(fk.API_SYMBOLS), decl ^ set(fk.API_SYMBOLS)
    for s in decl:
        assert hasattr(L, s), s


def test_header_compiles_as_cxx_and_c(tmp_path):
    src = tmp_path / "t.cpp"
    src.write_text('#include "fastkronMg.h"\nint main(){return (int)fastKronBackend_CUDA - 8;}\n')
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                           str(tmp_path / "t.o")])


def test_option_bits_keep_reference_values_and_tf32_is_an_extra_bit(tmp_path):
    """Reference option values (include/fastkron.h:57-61) are ABI; the TF32 opt-in takes the next free bit."""
    src = tmp_path / "o.cpp"
    src.write_text('#include "fastkron.h"\n'
                   'static_assert(fastKronOptionsNone == 1 && fastKronOptionsUseFusion == 2 && fastKronOptionsTune == 4, "reference values");\n'
                   'static_assert(fastKronOptionsTF32 == 8, "extension bit");\nint main(){return 0;}\n')
    subprocess.check_call(["g++", "-std=c++17", "-I", os.path.join(ROOT, "include"), "-c", str(src), "-o",
                           str(tmp_path / "o.o")])
    Lh = fk.get()
    assert hasattr(Lh, "fkbGemmTcTimeouts") and hasattr(Lh, "fkbGemmTmaTimeouts")


def test_enum_values_and_strings(L):
    assert (fk.OP_N, fk.OP_T) == (1, 2)
    assert fk.BACKEND_CUDA == 8 and fk.BACKEND_X86 == 2
    assert L.fastKronGetBackends() == fk.BACKEND_CUDA
    assert L.fastKronGetErrorString(0) == b"Operation successfull"
    assert L.fastKronGetErrorString(4) == b"An argument to the function is invalid"
    assert b"CUDA" in L.fastKronVersion()


def test_init_rejects_backends_not_in_library(L):
    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_X86)) == fk.INVALID_ARGUMENT
    assert h.value  # handle is still written, as in the reference (src/fastkron.cpp:78-89)
    assert L.fastKronInitX86(h) == fk.BACKEND_NOT_AVAILABLE
    assert L.fastKronInitHIP(h, None) == fk.BACKEND_NOT_AVAILABLE
    L.fastKronDestroy(h)
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    assert L.fastKronSetOptions(h, ctypes.c_uint32(fk.OPT_USE_FUSION)) == fk.SUCCESS
    assert L.fastKronSetStream(h, ctypes.c_int(fk.BACKEND_CUDA), None) == fk.INVALID_ARGUMENT
    L.fastKronDestroy(h)


def sizes(L, h, M, ps, qs):
    ye, te = ctypes.c_size_t(), ctypes.c_size_t()
    rc = L.gekmmSizes(h, ctypes.c_uint32(M), ctypes.c_uint32(len(ps)), fk.u32arr(ps), fk.u32arr(qs),
                      ctypes.byref(ye), ctypes.byref(te))
    assert rc == fk.SUCCESS
    return ye.value, te.value


SIZE_CASES = [(16, [8] * 4, [8] * 4), (3, [2, 5, 6], [3, 2, 4]), (7, [31, 31], [63, 63]), (5, [63, 63], [31, 31]),
              (2, [4], [9]), (2, [9], [4]), (13, [14, 19, 34, 21], [15, 13, 23, 34]), (1024, [16] * 4, [16] * 4)]


@pytest.mark.parametrize("M,ps,qs", SIZE_CASES)
def test_gekmm_sizes(L, M, ps, qs):
    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    ye, te = sizes(L, h, M, ps, qs)
    L.fastKronDestroy(h)
    K = 1
    for p in ps:
        K *= p
    Lc = 1
    for q in qs:
        Lc *= q
    assert ye == M * Lc
    widest = 0
    cols = K
    for p, q in reversed(list(zip(ps, qs))):
        cols = cols // p * q
        widest = max(widest, cols)
    if len(ps) == 1:
        widest = max(K, Lc)
    assert te == M * widest
    if oracle.ref_available():
        r = oracle.RefLib()
        assert r.sizes(M, ps, qs) == (ye, te)   # same answer as the reference library
        r.close()


def test_sizes_64bit(L):
    """The reference's 32-bit element counts wrap for M*K >= 2^32 (src/kmm/matrix.h:112);
    this library counts in 64 bits."""
    h = ctypes.c_void_p()
    assert L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)) == fk.SUCCESS
    ye, te = sizes(L, h, 256, [64] * 4, [64] * 4)
    L.fastKronDestroy(h)
    assert ye == te == 256 * 64 ** 4 == 1 << 32


def describe(L, mm, dt, M, ps, qs, opx="N", opf="N", forward=0, t2=1, fusion=1, align=16):
    buf = ctypes.create_string_buffer(1 << 14)
    n = L.fkbDescribePlan(ctypes.c_int(mm == "kmm"), ctypes.c_int(dt == "f64"), ctypes.c_uint32(M),
                          ctypes.c_uint32(len(ps)), fk.u32arr(ps), fk.u32arr(qs), ctypes.c_int(fk.OP_N if opx == "N" else fk.OP_T),
                          ctypes.c_int(fk.OP_N if opf == "N" else fk.OP_T), ctypes.c_int(forward), ctypes.c_int(t2),
                          ctypes.c_int(fusion), ctypes.c_int(align), buf, ctypes.c_size_t(len(buf)))
    assert n > 0, n
    return n, buf.value.decode().strip().split("\n")


def test_plan_buffers_follow_reference_rules(L):
    # without temp2 the result buffer doubles as scratch and the last pass lands in Z
    # (reference: src/kmm/kmmalgo.cpp:82-92)
    for nfac in (1, 2, 3, 4, 5):
        n, lines = describe(L, "mkm", "f32", 4, [7] * nfac, [7] * nfac, t2=0)
        assert n == nfac
        assert lines[0].split()[-2 if lines[0].endswith("epi") else -1].startswith("X->")
        assert "->Z" in lines[-1] and lines[-1].endswith("epi")
        prev = None
        for ln in lines:
            arrow = [t for t in ln.split() if "->" in t][0]
            src, dst = arrow.split("->")
            assert src != dst and dst != "X"
            if prev is not None:
                assert src == prev
            prev = dst
        assert all("T2" not in ln for ln in lines)


def test_plan_fuses_benchmark_shapes(L):
    n, lines = describe(L, "mkm", "f32", 1024, [16] * 4, [16] * 4)
    assert n == 2 and all(" tile " in ln for ln in lines), lines
    n, lines = describe(L, "mkm", "f64", 16, [8] * 8, [8] * 8)
    assert n == 3 and all(" tile " in ln for ln in lines), lines
    n, lines = describe(L, "mkm", "f32", 16, [8] * 8, [8] * 8, fusion=0)
    assert n == 8
    # unaligned operands cannot use the shared-memory tile kernels; the any-shape large-factor
    # kernel takes them (single-element accesses)
    n, lines = describe(L, "mkm", "f32", 16, [8] * 3, [8] * 3, align=4)
    assert n == 3 and all(" gemm " in ln for ln in lines)
    n, lines = describe(L, "mkm", "f32", 16, [4] * 3, [4] * 3, align=4)
    assert n == 3 and all(" generic " in ln for ln in lines)
    # factors from 5x5 on go to the any-shape kernel (narrow tiles); smaller ones and factors with a
    # side below 5 and fewer than 64 elements stay with the one-thread-per-output kernel
    for p, q, kind in ((5, 5, "gemm"), (7, 6, "gemm"), (3, 3, "generic"), (2, 12, "generic"), (12, 2, "generic"),
                       (2, 32, "gemm"), (4, 16, "gemm"), (6, 4, "generic")):
        n, lines = describe(L, "mkm", "f64", 8, [p, p], [q, q])
        assert n == 2 and all(" %s " % kind in ln for ln in lines), (p, q, lines)


def test_no_large_factor_pass_is_left_to_the_one_thread_per_output_kernel(L):
    """Over the reference's functional shape matrix (tests/src/general-tests-NN.cpp:34-166 of the
    reference: 12, 24, 31, 50, 55, 127, 129, 255, 297, 31x63, 297x127, mixed shapes, all op
    combinations, aligned or not, forward variants included) every pass whose factor has at
    least 64 elements gets a tiled kernel."""
    import re
    import cases
    seen = 0
    for c in cases.sweep_cases():
        for align in (16, 4):
            for forward in (0, 1):
                _, lines = describe(L, c["mm"], c["dt"], c["M"], c["ps"], c["qs"], c["opx"], c["opf"], forward=forward,
                                    align=align)
                for ln in lines:
                    m = re.match(r"pass\d+ (\w+) f\[(\d+)\.\.(\d+)\] P=(\d+) Q=(\d+)", ln)
                    kind, f0, f1 = m.group(1), int(m.group(2)), int(m.group(3))
                    if kind == "generic":
                        assert f0 == f1
                        # KMM with one column runs as MKM: factor order is unchanged
                        assert c["ps"][f0] * c["qs"][f0] < 64, (cases.case_id(c), ln)
                    seen += 1
    assert seen > 1000


def test_plan_forward_keeps_every_intermediate(L):
    n, lines = describe(L, "mkm", "f32", 4, [4, 3, 5], [2, 6, 3], forward=1)
    assert n == 3
    assert "X->I1" in lines[0] and "I1->I0" in lines[1] and "I0->Z" in lines[2]


def test_emulated_tile_kernels_match_direct_contraction(tmp_path):
    """Runs the tile kernels' contraction steps on the host, thread id by thread id
    (fastkron_b200/csrc/emu_tile.cu), against a direct contraction."""
    exe = tmp_path / "emu_tile"
    csrc = os.path.join(ROOT, "fastkron_b200", "csrc")
    subprocess.check_call(["nvcc", "-O1", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
                           "-I", os.path.join(ROOT, "include"), "-I", csrc, "-o", str(exe),
                           os.path.join(csrc, "emu_tile.cu")])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout[-2000:]
    assert "PASSED" in out.stdout


def test_tuned_tables_name_only_instantiated_kernels():
    """csrc/tile_db.inc / tile_fuse.inc (written by fastkron_b200/tune.py): every row names an
    existing tile kernel and an instantiated (ring depth, CTAs per SM) pair."""
    import re
    csrc = os.path.join(ROOT, "fastkron_b200", "csrc")
    table = open(os.path.join(csrc, "tile_table.h")).read()
    narrow = set(re.findall(r"X\((\d+), (\d+)\)", table.split("#define FKB_TILE_WIDE")[0]))
    wide = set(re.findall(r"X\((\d+), (\d+)\)", table.split("#define FKB_TILE_WIDE")[1].split("inline")[0]))
    rows = re.findall(r"\{DType::(F32|F64), (\d+), (\d+), (true|false), \{(\d+), (\d+), (\d+), (\d+)\}\}",
                      open(os.path.join(csrc, "tile_db.inc")).read())
    assert len(rows) >= 20
    for dt, P, nf, w, kb, nbuf, minb, tma in rows:
        assert (P, nf) in (wide if w == "true" else narrow), (P, nf, w)
        assert (int(nbuf), int(minb)) in ((2, 3), (2, 4), (1, 4), (1, 6)) and int(kb) in (16, 32, 64)
        assert tma == "0" or (dt == "F32" and w == "true" and nbuf == "2")
    fuse = re.findall(r"\{DType::(F32|F64), (\d+), (true|false), (\d+), (\d+)\}", open(os.path.join(csrc, "tile_fuse.inc")).read())
    for dt, P, w, left, nf in fuse:
        assert int(nf) <= int(left) and (P, nf) in (wide if w == "true" else narrow)
    import fastkron_b200.tune as tune
    assert len(tune.CANDIDATES) == 24 and len(tune.PROBES) >= 16


def test_bench_host_logic():
    """bench.py's workload description, operation counts and CPU-arm slab rule (no GPU needed)."""
    sys.path.insert(0, ROOT)
    import bench
    c5 = dict(bench.CONFIGS["C5"], name="C5")
    assert "factors=4x(64x64)" in bench.workload_desc(c5, 1)["workload"]
    c4 = dict(bench.CONFIGS["C4"], name="C4")
    assert "factors=2x(128x128),16x16" in bench.workload_desc(c4, 1)["workload"]
    # library flop count of src/kmm/kmmalgo.h:174-184: 2*M*sum_i K_out,i * P_i
    assert bench.flops_library(c5) == 2 * 256 * 4 * (64 ** 4) * 64
    assert bench.flops_harness(c5) == bench.flops_library(c5) + 2 * 256 * 64 ** 4
    # the reference counts elements in 32 bits: C5 goes to the CPU arm in slabs of 64 rows, the rest whole
    assert bench.cpu_slab_rows(c5) == 64
    for name in ("C1", "C2", "C3", "C4"):
        assert bench.cpu_slab_rows(bench.CONFIGS[name]) == bench.CONFIGS[name]["M"]
    t, src = bench.carried_traffic("gemm", 100e6 * 172, 100e6 * 172)
    assert src.startswith("profiles/") and os.path.exists(os.path.join(ROOT, src.split(",")[0]))
    assert 2 * 100e6 * 172 - 60e6 < t < 2 * 100e6 * 172 + 10e6
