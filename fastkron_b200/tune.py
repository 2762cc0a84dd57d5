"""Offline tuner of the shared-memory tile kernels and of the fusion depth (B200).

    python -m fastkron_b200.tune [--emit] [--quick]

For every (element type, P, fused factors, narrow/wide layout) kernel reached by the probe
problems below, every candidate (tile KB, ring depth, CTAs per SM, TMA staging) is forced on
the library through fkbSetTileTuning, the problem is run through the ordinary C ABI, and the
per-pass device times (CUDA events the engine records around each launch) are collected.
The fastest candidate per kernel becomes a row of csrc/tile_db.inc (--emit rewrites that
file; rebuild the library afterwards).  The second table printed compares fusion splits of a
run of equal factors (e.g. 8 factors of 8x8 as 4+2+2, 3+3+2, 2+2+2+2) by capping the depth
with fkbSetMaxFuse; the planner's per-(type, P) depth caps in csrc/plan.cpp come from it.

This is the role of the reference's autotuner (src/autotuner/autotuner.cpp:24-328) and of its
shipped per-architecture kernel lists (src/kernels/best-kernels/): measure once per machine
type, keep the table.
"""
import argparse
import ctypes
import os
import re
import sys

import numpy as np

CANDIDATES = [(kb, nbuf, minb, tma)
              for kb in (16, 32, 64)
              for (nbuf, minb) in ((2, 3), (2, 4), (1, 4), (1, 6))
              for tma in (1, 0)]

# (dtype, M, factors[, "kmm"]): chosen so that the plan visits narrow and wide kernels of every
# table shape; "kmm" probes run Z = 2 (F (x) ...) X + Y with X stored transposed, which reaches the
# wide kernels with m folded into the trailing index and with the beta*Y epilogue
PROBES = [
    ("f32", 1024, [32] * 3, "kmm"), ("f32", 1024, [16] * 4, "kmm"), ("f64", 256, [8] * 6, "kmm"),
    ("f32", 1024, [16] * 4), ("f32", 4096, [16] * 3), ("f32", 2048, [32] * 3), ("f32", 512, [8] * 6),
    ("f32", 256, [4] * 9), ("f32", 256, [2] * 18), ("f32", 8192, [16] * 2 + [64]), ("f32", 256, [128, 128, 16]),
    ("f32", 2048, [64, 64, 32]), ("f32", 4096, [64, 64, 8]),
    ("f64", 16, [8] * 8), ("f64", 512, [16] * 4), ("f64", 1024, [32] * 3), ("f64", 128, [4] * 9),
    ("f64", 128, [2] * 18), ("f64", 64, [8] * 6),
]


def _plan_passes(L, dt, M, ps, kmm=False):
    buf = ctypes.create_string_buffer(1 << 16)
    from . import lib as fk
    n = L.fkbDescribePlan(1 if kmm else 0, 1 if dt == "f64" else 0, ctypes.c_uint32(M), ctypes.c_uint32(len(ps)),
                          fk.u32arr(ps), fk.u32arr(ps), 2 if kmm else 1, 1, 0, 1, 1, 16, buf, ctypes.c_size_t(len(buf)))
    out = []
    for ln in buf.value.decode().splitlines()[:max(n, 0)]:
        m = re.match(r"pass\d+ (\w+) f\[(\d+)\.\.(\d+)\] P=(\d+) Q=\d+ M=\d+ A=\d+ B=(\d+)", ln)
        var = int(re.search(r" var=(\d+)", ln).group(1))
        # transposing first passes (var 1/2) are a kernel family of their own: not in this table
        out.append((m.group(1) if var == 0 else "tile-transpose", int(m.group(4)),
                    int(m.group(3)) - int(m.group(2)) + 1, int(m.group(5)) > 1))
    return out


def _time_passes(h, L, dt, M, ps, steps=8, kmm=False):
    import torch
    from . import synth
    tdt = torch.float32 if dt == "f32" else torch.float64
    ndt = np.float32 if dt == "f32" else np.float64
    K = int(np.prod(ps, dtype=object))
    x = torch.empty(M * K, dtype=tdt, device="cuda")
    synth.fill_uniform_cuda(x, 7)
    fs = [torch.from_numpy(synth.uniform(100 + i, p * p, ndt)).cuda() for i, p in enumerate(ps)]
    ye, te = h.sizes(M, ps, ps)
    z = torch.empty(ye, dtype=tdt, device="cuda")
    t1 = torch.empty(te, dtype=tdt, device="cuda")
    t2 = torch.empty(te, dtype=tdt, device="cuda")
    y = torch.zeros(ye, dtype=tdt, device="cuda") if kmm else None

    def call():
        if kmm:
            h.raw_gemm("kmm", "s" if dt == "f32" else "d", M, ps, ps, x.data_ptr(), 2, [f.data_ptr() for f in fs], 1,
                       z.data_ptr(), 2.0, 1.0, y.data_ptr(), t1.data_ptr(), t2.data_ptr())
        else:
            h.raw_gemm("mkm", "s" if dt == "f32" else "d", M, ps, ps, x.data_ptr(), 1, [f.data_ptr() for f in fs], 1,
                       z.data_ptr(), 1.0, 0.0, 0, t1.data_ptr(), t2.data_ptr())
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    L.fkbSetProfiling(h.h, 1)
    for _ in range(steps):
        call()
    torch.cuda.synchronize()
    ms = (ctypes.c_float * 4096)()
    kinds = (ctypes.c_int * 4096)()
    n = L.fkbGetPassTimes(h.h, ms, kinds, 4096)
    L.fkbSetProfiling(h.h, 0)
    per = n // steps
    return [float(np.min([ms[s * per + p] for s in range(steps)])) for p in range(per)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--emit", action="store_true", help="rewrite csrc/tile_db.inc with the winners")
    ap.add_argument("--quick", action="store_true", help="fewer probes and candidates")
    args = ap.parse_args()
    import fastkron_b200
    from . import lib as fk
    L = fk.get()
    probes = PROBES[:4] if args.quick else PROBES
    cands = [c for c in CANDIDATES if c[0] == 32] if args.quick else CANDIDATES
    samples = {}                     # (kernel key) -> {(probe id, pass index): {candidate: ms}}
    for pi, probe in enumerate(probes):
        dt, M, ps = probe[:3]
        kmm = len(probe) > 3 and probe[3] == "kmm"
        for cand in cands:
            L.fkbSetTileTuning(*[ctypes.c_int(v) for v in cand])
            h = fastkron_b200.FastKron()            # a fresh handle: plans are cached per handle
            passes = _plan_passes(L, dt, M, ps, kmm)
            try:
                times = _time_passes(h, L, dt, M, ps, kmm=kmm)
            except fk.FastKronError:
                h.close()
                continue
            h.close()
            for k, ((kind, P, nf, wide), t) in enumerate(zip(passes, times)):
                if kind != "tile":
                    continue
                if cand[3] == 1 and not (wide and dt == "f32" and cand[1] == 2):
                    continue                          # TMA staging exists for wide fp32 rings only
                samples.setdefault((dt, P, nf, wide), {}).setdefault((pi, k), {})[cand] = t
                print("%s M=%d %s%s  %s P=%d NF=%d %s  kb=%d nbuf=%d minb=%d tma=%d  %.4f ms" % (
                    dt, M, "x".join(map(str, ps)), " kmm" if kmm else "", kind, P, nf, "wide" if wide else "narrow",
                    *cand, t), flush=True)
    L.fkbSetTileTuning(0, 0, 0, 1)
    rows = []
    print("\n== winners (score = mean over the probe passes that use the kernel of time / best time there)")
    for key in sorted(samples):
        dt, P, nf, wide = key
        score = {}
        for per_pass in samples[key].values():
            lo = min(per_pass.values())
            for cand, t in per_pass.items():
                score.setdefault(cand, []).append(t / lo)
        full = {c: float(np.mean(v)) for c, v in score.items() if len(v) == len(samples[key])}
        cand = min(full, key=full.get)
        print("%s P=%d NF=%d %-6s -> kb=%d nbuf=%d minb=%d tma=%d  (score %.3f over %d probe passes; default 32/2/3 scores %s)" % (
            dt, P, nf, "wide" if wide else "narrow", *cand, full[cand], len(samples[key]),
            "%.3f" % full[(32, 2, 3, 0)] if (32, 2, 3, 0) in full else "n/a"))
        rows.append("{DType::%s, %d, %d, %s, {%d, %d, %d, %d}}," % (
            "F32" if dt == "f32" else "F64", P, nf, "true" if wide else "false", *cand))
    if args.emit:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "tile_db.inc")
        with open(path, "w") as f:
            f.write("// dtype, P, NF, wide, {kb, nbuf, minb, tma}   -- written by fastkron_b200/tune.py --emit\n")
            f.write("\n".join(rows) + "\n")
        print("wrote", path)

    # ---- fusion splits of a run of equal factors -----------------------------------------
    print("\n== fusion depth caps (whole-call ms)")
    for dt, M, ps in ([("f32", 1024, [16] * 4), ("f64", 16, [8] * 8), ("f32", 512, [8] * 6), ("f32", 2048, [32] * 3)]
                      if not args.quick else [("f32", 1024, [16] * 4)]):
        for cap in range(1, 9):
            L.fkbSetMaxFuse(ctypes.c_int(cap))
            h = fastkron_b200.FastKron()
            passes = _plan_passes(L, dt, M, ps)
            times = _time_passes(h, L, dt, M, ps)
            h.close()
            print("%s M=%d %s cap=%d split=%s  %.4f ms" % (dt, M, "x".join(map(str, ps)), cap,
                                                            "+".join(str(p[2]) for p in passes), sum(times)), flush=True)
            if len(passes) == 1 or cap >= max(p[2] for p in passes) + 1:
                break
    L.fkbSetMaxFuse(0)


if __name__ == "__main__":
    sys.exit(main())
