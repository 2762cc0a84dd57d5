#!/usr/bin/env python
"""Benchmark of the GeMKM/GeKMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config C5]

One step = one complete GeMKM/GeKMM call (all passes) on one synthetic operand set.
The default workload is the distributed benchmark configuration C5 (fp32 GeMKM,
M=256, four 64x64 factors, K = 64^4 = 16.8M columns, 17 GB of X): it fits one B200,
so the same problem is measured at 1, 2, 4 and 8 GPUs (strong scaling; at N > 1 the
columns of X are sharded over the ranks).  With N = 1 the line also carries the
single-GPU configurations C1-C4 under "configs".

Metric: GFLOP/s with the reference library's operation count
2*M*sum_i(K_out,i * P_i) (src/kmm/kmmalgo.h:174-184 of the reference); the count of the
reference's test harness, which adds the epilogue (tests/testBase.h:994-1003), is
reported as "value_harness_count".

Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: mm, dtype, M, Ps, Qs, opX, opF, alpha, beta, seed, distribution of X/Y
    "C1": dict(mm="mkm", dt="f32", M=1024, ps=[16] * 4, qs=[16] * 4, opx="N", opf="N", alpha=1.0, beta=0.0, seed=0, dist="uniform"),
    "C2": dict(mm="mkm", dt="f64", M=16, ps=[8] * 8, qs=[8] * 8, opx="N", opf="N", alpha=1.0, beta=0.0, seed=1, dist="uniform"),
    "C3": dict(mm="kmm", dt="f32", M=1024, ps=[32] * 3, qs=[32] * 3, opx="T", opf="N", alpha=2.0, beta=1.0, seed=2, dist="normal"),
    # C4: "opF = T on F1 only" cannot be said through the C API's single opFs; as in the
    # reference's own Python wrapper the transposed factor is materialised and opFs = N.
    "C4": dict(mm="mkm", dt="f32", M=2048, ps=[128, 128, 16], qs=[128, 128, 16], opx="N", opf="N", alpha=1.0, beta=0.0, seed=4, dist="uniform"),
    "C5": dict(mm="mkm", dt="f32", M=256, ps=[64] * 4, qs=[64] * 4, opx="N", opf="N", alpha=1.0, beta=0.0, seed=5, dist="uniform"),
}
# reduced copies for quick functional runs of this script (--config C5s etc.)
CONFIGS["C5s"] = dict(CONFIGS["C5"], M=16, ps=[64] * 3, qs=[64] * 3)
CONFIGS["C1s"] = dict(CONFIGS["C1"], M=64)
# profiling sizes: operands larger than L2, a few hundred MB each
CONFIGS["C5m"] = dict(CONFIGS["C5"], M=256, ps=[64] * 3, qs=[64] * 3)
CONFIGS["C2p"] = dict(CONFIGS["C2"], M=4)
CONFIGS["C4p"] = dict(CONFIGS["C4"], M=256)
# the any-shape large-factor kernel on a shape outside the fixed-shape kernels (profiling / side table)
CONFIGS["A127"] = dict(CONFIGS["C1"], M=4096, ps=[127, 127], qs=[127, 127], seed=9)


def flops_library(c, M=None):
    M = c["M"] if M is None else M
    cols = int(np.prod(c["ps"], dtype=object))
    tot = 0
    for p, q in reversed(list(zip(c["ps"], c["qs"]))):
        cols = cols // p * q
        tot += cols * p
    return 2 * M * tot


def flops_harness(c, M=None):
    M = c["M"] if M is None else M
    L = int(np.prod(c["qs"], dtype=object))
    return flops_library(c, M) + 2 * M * (L + (2 * L if c["beta"] != 0 else 0))


def algorithmic_bytes(c, M=None):
    """X read once + Z written once (+ Y read when beta != 0) + factors."""
    M = c["M"] if M is None else M
    es = 4 if c["dt"] == "f32" else 8
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    b = M * K + M * L + (M * L if c["beta"] != 0 else 0) + sum(p * q for p, q in zip(c["ps"], c["qs"]))
    return b * es


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for ln in open(self.path):
                f = [t.strip() for t in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def make_device_operands(c, M=None, col_shard=None):
    """Seeded operands in HBM.  Uniform operands are generated on the device by the same
    counter-based generator the CPU oracle inputs use; normal ones come from the host."""
    import torch
    from fastkron_b200 import synth
    M = c["M"] if M is None else M
    tdt = torch.float32 if c["dt"] == "f32" else torch.float64
    ndt = np.float32 if c["dt"] == "f32" else np.float64
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    x = torch.empty(M * K, dtype=tdt, device="cuda")
    if c["dist"] == "normal":
        x.copy_(torch.from_numpy(synth.normal(c["seed"], M * K, ndt)))
    else:
        synth.fill_uniform_cuda(x, c["seed"])
    y = None
    if c["beta"] != 0:
        gen = synth.normal if c["dist"] == "normal" else synth.uniform
        y = torch.from_numpy(gen(c["seed"] + 1000, M * L, ndt)).cuda()
    fs = [torch.from_numpy(synth.uniform(c["seed"] + 2000 + i, p * q, ndt)).cuda()
          for i, (p, q) in enumerate(zip(c["ps"], c["qs"]))]
    return x, fs, y


OPC = {"N": 1, "T": 2}


def call(h, c, M, x, fs, z, y, t1, t2):
    h.raw_gemm(c["mm"], "s" if c["dt"] == "f32" else "d", M, c["ps"], c["qs"], x.data_ptr(), OPC[c["opx"]],
               [f.data_ptr() for f in fs], OPC[c["opf"]], z.data_ptr(), c["alpha"], c["beta"],
               y.data_ptr() if y is not None else 0, t1.data_ptr(), t2.data_ptr())


def time_config(h, c, steps, warmup, profile=False):
    """Device-resident timing of one configuration on one GPU.  Returns a dict."""
    import torch
    from fastkron_b200 import lib as fk
    M = c["M"]
    tdt = torch.float32 if c["dt"] == "f32" else torch.float64
    x, fs, y = make_device_operands(c)
    ye, te = h.sizes(M, c["ps"], c["qs"])
    z = torch.empty(ye, dtype=tdt, device="cuda")
    t1 = torch.empty(te, dtype=tdt, device="cuda")
    t2 = torch.empty(te, dtype=tdt, device="cuda")
    L = fk.get()
    L.fkbLaunchCount.restype = ctypes.c_ulonglong
    for _ in range(warmup):
        call(h, c, M, x, fs, z, y, t1, t2)
    torch.cuda.synchronize()
    if profile:
        L.fkbSetProfiling(h.h, 1)
    n0 = L.fkbLaunchCount()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        a.record()
        call(h, c, M, x, fs, z, y, t1, t2)
        b.record()
    torch.cuda.synchronize()
    launches = L.fkbLaunchCount() - n0
    times = [a.elapsed_time(b) for a, b in ev]
    passes = None
    if profile:
        ms = (ctypes.c_float * 4096)()
        kinds = (ctypes.c_int * 4096)()
        n = L.fkbGetPassTimes(h.h, ms, kinds, 4096)
        L.fkbSetProfiling(h.h, 0)
        per = n // steps if steps else 0
        passes = []
        for p in range(per):
            vals = [ms[s * per + p] for s in range(steps)]
            passes.append({"kind": ["generic", "tile", "gemm"][kinds[p]], "ms": float(np.mean(vals))})
    total_ms = float(sum(times))
    return {"ms_per_step": total_ms / steps, "ms_min": float(min(times)), "launches": int(launches),
            "passes": passes, "buffers": (x, fs, y, z, t1, t2)}


def measure_fma_peak(dt):
    """FFMA / DFMA issue peak of this GPU from a register-only FMA chain kernel (TFLOP/s)."""
    import torch
    from fastkron_b200 import synth
    synth.fill_uniform_cuda(torch.empty(16, device="cuda"), 0)     # loads the helper library
    lib = synth._slib
    fn = lib.fkbFmaPeakF32 if dt == "f32" else lib.fkbFmaPeakF64
    fn.restype = ctypes.c_ulonglong
    blocks = 148 * 8
    out = torch.empty(blocks * 256, dtype=torch.float32 if dt == "f32" else torch.float64, device="cuda")
    iters = 20000 if dt == "f32" else 8000
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    best = 0.0
    for i in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        n = fn(ctypes.c_void_p(out.data_ptr()), ctypes.c_int(blocks), ctypes.c_int(iters), st)
        b.record()
        torch.cuda.synchronize()
        if n and i >= 1:
            best = max(best, 2.0 * n / (a.elapsed_time(b) * 1e-3) / 1e12)
    return best


def read_measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return json.load(open(p)), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0}, "fallback"


def cpu_slab_rows(c):
    """Rows per reference call: the whole configuration when its matrices stay below 2^31
    elements, otherwise the largest power-of-two row slab that does (at most 128 rows; the
    reference counts elements in 32 bits, src/kmm/matrix.h:112).  Rows of an MKM are
    independent, so a call is the sum of its slabs."""
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    width = max(K, L)
    if c["M"] * width < (1 << 31):
        return c["M"]
    rows = 128
    while rows > 1 and rows * width >= (1 << 31):
        rows //= 2
    return rows


def cpu_whole(c, reps, warm=1, threads=None):
    """Time the reference x86 backend (oracle/_ref) -- or, where that library is absent, the
    C restatement -- on the WHOLE configuration with all host threads.  A configuration too
    large for one reference call runs as row slabs with their true seeded rows; a step is the
    sum of its slab times.  Returns per-step seconds (list) and a description."""
    import oracle
    from fastkron_b200 import synth
    ndt = np.float32 if c["dt"] == "f32" else np.float64
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    M = c["M"]
    rows = cpu_slab_rows(c)
    if rows < M and (c["mm"] != "mkm" or c["opx"] != "N" or c["beta"] != 0):
        raise SystemExit("row slabs are implemented for row-major MKM without Y")
    gen = synth.normal if c["dist"] == "normal" else synth.uniform
    fs = [synth.uniform(c["seed"] + 2000 + i, p * q, ndt) for i, (p, q) in enumerate(zip(c["ps"], c["qs"]))]
    cores = threads or os.cpu_count() or 1
    nslab = -(-M // rows)
    step = [0.0] * reps
    use_ref = oracle.ref_available()
    kind = "reference" if use_ref else "port"
    ref = oracle.RefLib(threads=cores) if use_ref else None
    if not use_ref:
        os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    z = temps = None
    for sl in range(nslab):
        r0 = sl * rows
        r = min(rows, M - r0)
        x = gen(c["seed"], r * K, ndt, offset=r0 * K)
        y = gen(c["seed"] + 1000, r * L, ndt, offset=r0 * L) if c["beta"] != 0 else None
        if use_ref and (z is None or z.size != r * L):
            z = np.zeros(r * L, dtype=ndt)
            _, te = ref.sizes(r, c["ps"], c["qs"])
            temps = (np.zeros(te, dtype=ndt), np.zeros(te, dtype=ndt))
        for i in range(warm + reps):
            t0 = time.perf_counter()
            if use_ref:
                ref.gekmm(c["mm"], x, fs, c["ps"], c["qs"], r, c["opx"], c["opf"], c["alpha"], c["beta"], y, z=z, temps=temps)
            else:
                oracle.port_gekmm(c["mm"], x, fs, c["ps"], c["qs"], r, c["opx"], c["opf"], c["alpha"], c["beta"], y)
            dt = time.perf_counter() - t0
            if i >= warm:
                step[i - warm] += dt
        del x, y
    if ref is not None:
        ref.close()
    best = min(step)
    return {"value": flops_library(c) / best / 1e9, "unit": "GFLOP/s", "cores": cores, "kind": kind,
            "sample": "whole %s (%d rows) as %d slab(s) of %d rows, slab times summed; best of %d steps after %d warm-up "
                      "call(s) per slab: %.3f s per step (mean %.3f s)" % (c["name"], M, nslab, rows, reps, warm, best,
                                                                          float(np.mean(step))),
            "seconds": best, "seconds_mean": float(np.mean(step)), "slabs": nslab, "slab_rows": rows}


def run_reference(args):
    c = dict(CONFIGS[args.config], name=args.config)
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    # a step is the whole configuration; warm-up calls are per slab and capped so that the
    # run stays within a few minutes on any host
    res = cpu_whole(c, reps=max(1, min(args.steps, 10)), warm=max(1, min(args.warmup, 2)))
    out = {
        "impl": "reference", "metric": "GeMKM/GeKMM GFLOP/s", "value": res["value"], "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["seconds"] * 1e3,
        "ms_per_step_mean": res["seconds_mean"] * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": c["dt"], "data": "synthetic",
        "config": workload_desc(c, args.gpus),
        "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": res["value"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(out))


def factor_desc(c):
    """Factor list with runs of equal shapes folded: 4x(64x64), 2x(128x128),16x16."""
    out, shapes = [], list(zip(c["ps"], c["qs"]))
    k = 0
    while k < len(shapes):
        n = 1
        while k + n < len(shapes) and shapes[k + n] == shapes[k]:
            n += 1
        one = "%dx%d" % shapes[k]
        out.append(one if n == 1 else "%dx(%s)" % (n, one))
        k += n
    return ",".join(out)


def workload_desc(c, gpus):
    return {"workload": "%s: %s %s M=%d factors=%s opX=%s opF=%s alpha=%g beta=%g seed=%d" % (
        c["name"], "sge" if c["dt"] == "f32" else "dge", c["mm"], c["M"],
        factor_desc(c), c["opx"], c["opf"], c["alpha"], c["beta"], c["seed"]),
        "gpus": gpus, "sharding": "none" if gpus == 1 else "X columns over %d ranks" % gpus,
        "l2": "operands exceed L2 (no flush needed)" if algorithmic_bytes(c) > 2 * 126e6 else "operands fit L2; not flushed"}


# DRAM traffic per launch, measured with ncu (dram__bytes_read.sum, dram__bytes_write.sum) on
# smaller operands of the same kernels and carried to a full launch: reads scale with the
# matrix (ratio to the algorithmic bytes read), writes are the algorithmic bytes minus what
# is still dirty in the 126 MB L2 when the kernel ends (an absolute amount, not a ratio).
NCU_TRAFFIC = {
    "gemm": {"read_ratio": 1.0003, "dirty_l2_bytes": 52.8e6,
             "source": "profiles/gemm_kernel_c4_c5.md, C5m passes 2-3: 268.5 MB read, 215.6 MB written for 268.4 MB each way"},
    "tile": {"read_ratio": 1.0002, "dirty_l2_bytes": 50.4e6,
             "source": "profiles/tile_kernels_c1_c3.md, C1 pass 2: 268.5 MB read, 218.1 MB written for 268.4 MB each way"},
}


def carried_traffic(kind, read_bytes, write_bytes):
    t = NCU_TRAFFIC.get(kind)
    if t is None:
        return None, None
    return t["read_ratio"] * read_bytes + max(0.0, write_bytes - t["dirty_l2_bytes"]), t["source"]


def simt_peak_from_props(dt):
    """SMs x lanes x 2 x maximum SM clock of device 0 (TFLOP/s), from the device properties."""
    from fastkron_b200 import synth
    lib = synth._helper()
    if lib is None or not hasattr(lib, "fkbSimtPeakFromProps"):
        return 0.0
    lib.fkbSimtPeakFromProps.restype = ctypes.c_double
    return float(lib.fkbSimtPeakFromProps(ctypes.c_int(0), ctypes.c_int(0 if dt == "f32" else 1)))


def matrix_views(c, x, z, y):
    """(M, K) / (M, L) views of the stored operands whatever their storage order."""
    M, mm = c["M"], c["mm"]
    K = int(np.prod(c["ps"], dtype=object))
    L = int(np.prod(c["qs"], dtype=object))
    x_rowmajor = (mm == "mkm") == (c["opx"] == "N")
    Xv = x.view(M, K) if x_rowmajor else x.view(K, M).t()
    Zv = z.view(M, L) if mm == "mkm" else z.view(L, M).t()
    Yv = None if y is None else (y.view(M, L) if mm == "mkm" else y.view(L, M).t())
    return Xv, Zv, Yv


def parity_rows(c, x, fs, y, z, rows=None):
    """Rows of the device result against the CPU oracle run on those rows (outside any timed
    region): max |z - ref| / max |ref row|."""
    import oracle
    Xv, Zv, Yv = matrix_views(c, x, z, y)
    M = c["M"]
    rows = sorted(set(rows or [0, M - 1]))
    xr = np.ascontiguousarray(Xv[rows].cpu().numpy())
    yr = None if Yv is None else np.ascontiguousarray(Yv[rows].cpu().numpy())
    fh = [f.cpu().numpy() for f in fs]
    opf = c["opf"] if c["mm"] == "mkm" else ("T" if c["opf"] == "N" else "N")
    want = oracle.port_gekmm("mkm", xr, fh, c["ps"], c["qs"], len(rows), "N", opf, c["alpha"], c["beta"], yr)
    got = Zv[rows].cpu().numpy().astype(np.float64)
    den = np.abs(want).max(axis=1, keepdims=True)
    return float((np.abs(got - want) / den).max())


def time_e2e(h, c, bufs, steps):
    """The same call with HOST operands: X (and Y) start in pinned host memory, Z ends there;
    every step pays its copies.  Row-major MKM without Y goes through the public pipelined
    host-operand call (fastkron_b200.HostGeMKM: row slabs, copies overlapped with the
    product); everything else is copy in, one C-ABI call, copy out."""
    import torch
    import fastkron_b200
    x, fs, y, z, t1, t2 = bufs
    es = x.element_size()
    hx = torch.empty(x.numel(), dtype=x.dtype, pin_memory=True)
    hz = torch.empty(z.numel(), dtype=z.dtype, pin_memory=True)
    hy = None
    hx.copy_(x)
    if y is not None:
        hy = torch.empty(y.numel(), dtype=y.dtype, pin_memory=True)
        hy.copy_(y)
    torch.cuda.synchronize()
    tt = []
    if c["mm"] == "mkm" and c["beta"] == 0 and c["opx"] == "N":
        op = fastkron_b200.HostGeMKM(c["M"], c["ps"], c["qs"], dtype=x.dtype)
        mode = "row slabs of %d, copies overlapped with the product" % op.rows
        for it in range(1 + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            op(hx.view(c["M"], -1), fs, hz.view(c["M"], -1), c["alpha"])
            b.record()
            torch.cuda.synchronize()
            if it > 0:
                tt.append(a.elapsed_time(b))
        op.close()
    else:
        mode = "one copy in, one call, one copy out"
        for it in range(1 + steps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            x.copy_(hx, non_blocking=True)
            if hy is not None:
                y.copy_(hy, non_blocking=True)
            call(h, c, c["M"], x, fs, z, y, t1, t2)
            hz.copy_(z, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            if it > 0:
                tt.append(a.elapsed_time(b))
    ms = float(np.mean(tt))
    n = min(1 << 20, z.numel())
    same = bool(torch.equal(hz[:n], z[:n].cpu()) and torch.equal(hz[-n:], z[-n:].cpu()))
    h2d = x.numel() * es + (y.numel() * es if y is not None else 0)
    return {"value": flops_library(c) / (ms * 1e-3) / 1e9, "unit": "GFLOP/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": z.numel() * es, "ms_per_step": ms, "steps": steps, "how": mode,
            "matches_device_result": same}


def dominant_roofline(c, passes, flops, peaks, peak_src, fma_probe, fma_props):
    """Roofline entry of the kernel family with the largest share of a step.  Its launch
    duration is the average over its launches in a step (CUDA events the engine records
    around each launch on the launching stream).  Per launch: algorithmic bytes = the matrix
    read once and written once (2*M*K*sizeof(T)); algorithmic flops = 2*M*K*P."""
    if not passes:
        return None
    share = {}
    for q in passes:
        share[q["kind"]] = share.get(q["kind"], 0.0) + q["ms"]
    kind = max(share, key=share.get)
    idxs = [i for i, q in enumerate(passes) if q["kind"] == kind]
    ms = share[kind] / len(idxs)
    es = 4 if c["dt"] == "f32" else 8
    K = int(np.prod(c["ps"], dtype=object))
    mat = c["M"] * K * es
    pass_bytes = 2 * mat
    hbm_ach = pass_bytes / (ms * 1e-3) / 1e9
    traffic, tsrc = carried_traffic(kind, mat, mat)
    common = {"kernel": kind, "pass_indices": idxs, "launch_ms": ms,
              "launch_ms_min": min(passes[i]["ms"] for i in idxs), "launch_ms_max": max(passes[i]["ms"] for i in idxs),
              "launches_per_step": len(idxs), "algorithmic_bytes": pass_bytes, "traffic": traffic, "traffic_source": tsrc}
    roof_hbm = dict({"bound": "hbm", "achieved": hbm_ach, "peak": peaks.get("hbm_gbs"), "unit": "GB/s",
                     "frac": hbm_ach / peaks.get("hbm_gbs"), "peak_source": peak_src + " copy bandwidth"}, **common)
    dom_flops = flops / len(passes) if len(set(c["ps"])) == 1 and len(idxs) == len(passes) else None
    fp_peak = max(fma_probe or 0.0, fma_props or 0.0)
    if dom_flops is None or fp_peak <= 0:
        return roof_hbm
    fp_ach = dom_flops / (ms * 1e-3) / 1e12
    roof_fp = dict({"bound": "fp32_simt" if c["dt"] == "f32" else "fp64_simt", "achieved": fp_ach, "peak": fp_peak,
                    "unit": "TFLOP/s", "frac": fp_ach / fp_peak,
                    "peak_source": "larger of the FMA-chain probe of this run (%.1f) and SMs x lanes x 2 x max SM clock "
                                   "from the device properties (%.1f)" % (fma_probe or 0.0, fma_props or 0.0)}, **common)
    return dict(roof_fp, other=roof_hbm) if roof_fp["frac"] > roof_hbm["frac"] else dict(roof_hbm, other=roof_fp)


def run_single(args):
    import torch
    import fastkron_b200
    from fastkron_b200 import lib as fk
    c = dict(CONFIGS[args.config], name=args.config)
    torch.cuda.set_device(0)
    h = fastkron_b200.FastKron()
    peaks, peak_src = read_measured_peaks()

    sampler = ClockSampler(0)
    sampler.start()
    r = time_config(h, c, args.steps, args.warmup, profile=True)
    clocks = sampler.stop()
    flops = flops_library(c)
    value = flops / (r["ms_per_step"] * 1e-3) / 1e9

    fma_probe = measure_fma_peak(c["dt"])
    fma_props = simt_peak_from_props(c["dt"])
    passes = r["passes"] or []
    roof = dominant_roofline(c, passes, flops, peaks, peak_src, fma_probe, fma_props)

    # ---- parity of the timed result, outside the timed region -----------------------------
    x, fs, y, z, t1, t2 = r["buffers"]
    parity = None
    if not args.no_cpu:
        parity = parity_rows(c, x, fs, y, z)

    # ---- end to end with host buffers ------------------------------------------------------
    e2e_steps = max(1, min(args.steps, 3))
    try:
        if c["mm"] == "mkm" and c["beta"] == 0 and c["opx"] == "N":
            t1 = t2 = None
            r["buffers"] = (x, fs, y, z, None, None)
            torch.cuda.empty_cache()
        e2e = time_e2e(h, c, (x, fs, y, z, t1, t2), e2e_steps)
    except RuntimeError as ex:      # pinned allocation failed
        e2e = {"value": None, "unit": "GFLOP/s", "error": str(ex)[:200]}
    del x, fs, y, z, t1, t2, r["buffers"]
    torch.cuda.empty_cache()

    # ---- the other single-GPU configurations ---------------------------------------------
    extra = {}
    if not args.no_extra and args.config == "C5":
        for name in ("C1", "C2", "C3", "C4"):
            cc = dict(CONFIGS[name], name=name)
            st = max(3, args.steps)
            rr = time_config(h, cc, st, max(3, args.warmup), profile=True)
            fl = flops_library(cc)
            sec = rr["ms_per_step"] * 1e-3
            bx, bf, by, bz, bt1, bt2 = rr["buffers"]
            ent = {"gflops": fl / sec / 1e9, "gflops_harness_count": flops_harness(cc) / sec / 1e9,
                   "ms_per_step": rr["ms_per_step"], "ms_min": rr["ms_min"],
                   "algorithmic_gbs": algorithmic_bytes(cc) / sec / 1e9,
                   "hbm_frac_algorithmic": algorithmic_bytes(cc) / sec / 1e9 / peaks.get("hbm_gbs"),
                   "passes": rr["passes"], "launches_per_step": rr["launches"] // st,
                   "roofline": dominant_roofline(cc, rr["passes"] or [], fl, peaks, peak_src,
                                                 fma_probe if cc["dt"] == c["dt"] else measure_fma_peak(cc["dt"]),
                                                 simt_peak_from_props(cc["dt"]))}
            if not args.no_cpu:
                ent["parity_rows_max_rel_err"] = parity_rows(cc, bx, bf, by, bz)
            try:
                ent["e2e"] = time_e2e(h, cc, rr["buffers"], 3)
            except RuntimeError as ex:
                ent["e2e"] = {"value": None, "unit": "GFLOP/s", "error": str(ex)[:200]}
            del bx, bf, by, bz, bt1, bt2, rr["buffers"]
            torch.cuda.empty_cache()
            extra[name] = ent

    # ---- opt-in TF32 tensor-core path on the same workload (reported beside, never the headline) ----
    tf32 = None
    if not args.no_extra and c["dt"] == "f32" and c["mm"] == "mkm":
        h32 = fastkron_b200.FastKron()
        h32.set_options(2 | 8)                          # fastKronOptionsUseFusion | fastKronOptionsTF32
        rr = time_config(h32, c, max(3, min(args.steps, 5)), 3, profile=True)
        del rr["buffers"]
        torch.cuda.empty_cache()
        h32.close()
        sec = rr["ms_per_step"] * 1e-3
        slow = max(rr["passes"], key=lambda q: q["ms"]) if rr["passes"] else None
        es = 4
        pass_bytes = 2 * c["M"] * int(np.prod(c["ps"], dtype=object)) * es
        tf32 = {"gflops": flops / sec / 1e9, "ms_per_step": rr["ms_per_step"], "passes": rr["passes"],
                "hbm_frac_slowest_pass": (pass_bytes / (slow["ms"] * 1e-3) / 1e9 / peaks.get("hbm_gbs")) if slow else None,
                "tolerance": "5e-3 of the row maximum (TF32 operands, fp32 accumulation)",
                "timeouts": int(fk.get().fkbGemmTcTimeouts())}

    # ---- opt-in split TF32 (three tensor-core products per fp32 product; fp32-level results) ----
    tf32x3 = None
    if not args.no_extra and c["dt"] == "f32" and c["mm"] == "mkm":
        h3 = fastkron_b200.FastKron()
        h3.set_options(2 | 16)                          # fastKronOptionsUseFusion | fastKronOptionsTF32x3
        before = int(fk.get().fkbGemmTcLaunches(1))
        rr = time_config(h3, c, max(3, min(args.steps, 5)), 3, profile=True)
        bx, bf, by, bz, bt1, bt2 = rr["buffers"]
        par3 = parity_rows(c, bx, bf, by, bz) if not args.no_cpu else None
        del bx, bf, by, bz, bt1, bt2, rr["buffers"]
        torch.cuda.empty_cache()
        h3.close()
        sec = rr["ms_per_step"] * 1e-3
        slow = max(rr["passes"], key=lambda q: q["ms"]) if rr["passes"] else None
        pass_bytes = 2 * c["M"] * int(np.prod(c["ps"], dtype=object)) * 4
        tf32x3 = {"gflops": flops / sec / 1e9, "ms_per_step": rr["ms_per_step"], "passes": rr["passes"],
                  "hbm_frac_slowest_pass": (pass_bytes / (slow["ms"] * 1e-3) / 1e9 / peaks.get("hbm_gbs")) if slow else None,
                  "parity_rows_max_rel_err": par3,
                  "tolerance": "1e-5 of the row maximum (operands split into two TF32 numbers, three products, fp32 accumulation)",
                  "split_kernel_launches": int(fk.get().fkbGemmTcLaunches(1)) - before,
                  "timeouts": int(fk.get().fkbGemmTcTimeouts())}

    # ---- shapes outside the fixed-shape kernels: the any-shape tiled kernel against the
    # one-thread-per-output kernel it replaced (same library, same call, plan forced) --------
    any_table = None
    if not args.no_extra:
        any_table = {}
        L = fk.get()
        for name, M, ps, qs in (("31x63^2", 4096, [31, 31], [63, 63]), ("127^2", 4096, [127, 127], [127, 127]),
                                ("297x127", 65536, [297], [127]), ("12^4", 2048, [12] * 4, [12] * 4),
                                ("f64 128^2", 1024, [128, 128], [128, 128])):
            cc = dict(mm="mkm", dt="f64" if name.startswith("f64") else "f32", M=M, ps=ps, qs=qs, opx="N", opf="N",
                      alpha=1.0, beta=0.0, seed=9, dist="uniform", name=name)
            ent = {}
            for label, force in (("generic", 1), ("tiled", 0)):
                L.fkbSetForceGeneric(ctypes.c_int(force))
                hh = fastkron_b200.FastKron()
                rr = time_config(hh, cc, 5, 3, profile=True)
                if label == "tiled" and not args.no_cpu:
                    bx, bf, by, bz, bt1, bt2 = rr["buffers"]
                    ent["parity_rows_max_rel_err"] = parity_rows(cc, bx, bf, by, bz)
                    del bx, bf, by, bz, bt1, bt2
                del rr["buffers"]
                hh.close()
                torch.cuda.empty_cache()
                ent[label + "_gflops"] = flops_library(cc) / (rr["ms_per_step"] * 1e-3) / 1e9
                ent[label + "_ms"] = rr["ms_per_step"]
                ent[label + "_kernels"] = [q["kind"] for q in rr["passes"]]
            L.fkbSetForceGeneric(ctypes.c_int(0))
            ent["speedup"] = ent["generic_ms"] / ent["tiled_ms"]
            any_table[name] = ent

    cpu = None
    if not args.no_cpu:
        cpu = cpu_whole(c, reps=2, warm=1)
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}

    out = {
        "metric": "GeMKM/GeKMM GFLOP/s", "value": value, "unit": "GFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": c["dt"], "data": "synthetic", "config": workload_desc(c, 1),
        "value_harness_count": flops_harness(c) / (r["ms_per_step"] * 1e-3) / 1e9,
        "gpu_launches": r["launches"], "passes": passes, "clocks": clocks, "roofline": roof, "e2e": e2e,
        "cpu_baseline": cpu, "parity_rows_max_rel_err": parity,
        "fma_peak_tflops": {"probe": fma_probe, "device_props": fma_props}, "configs": extra, "any_shape_kernel": any_table, "tf32_optin": tf32, "tf32x3_optin": tf32x3,
        "gemm_timeouts": int(fk.get().fkbGemmTmaTimeouts()),
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="C5", choices=sorted(CONFIGS))
    ap.add_argument("--no-extra", action="store_true", help="skip the C1-C4 side measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        import bench_mg
        return bench_mg.run(args, CONFIGS, globals())
    return run_single(args)


if __name__ == "__main__":
    main()
