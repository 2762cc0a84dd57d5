"""bench.py's N > 1 leg: the column-sharded GeMKM with one process per GPU (torchrun).

Strong scaling: the same problem as at N = 1, X's columns split over the ranks.  A step is one
complete product: every rank's result block is complete (in device order) before the next
step's first exchange touches a buffer.  Timing is on the device (CUDA events on the compute
stream), bracketed by a barrier and a device synchronisation on both sides, maximum over
ranks; rank 0 prints the JSON line."""
import ctypes
import json
import os
import time

import numpy as np


def _fill_block(x, c, M, K, Kl, rank):
    """Local [M, Kl] block of the seeded global X: element (m, j) is stream index m*K + rank*Kl + j."""
    from fastkron_b200 import synth
    xv = x.view(M, Kl)
    for m in range(M):
        synth.fill_uniform_cuda(xv[m], c["seed"], offset=m * K + rank * Kl)


def _c_api_blocking_ms(c, world, fs_host, reps=3):
    """Rank 0 alone: the reference's own entry point fastKronMgSGEMM (one process driving all
    GPUs, blocking) on the same problem; wall-clock milliseconds per call."""
    import torch
    from fastkron_b200 import lib as fk
    L = fk.get()
    M, ps, qs = c["M"], c["ps"], c["qs"]
    n = len(ps)
    K = int(np.prod(ps, dtype=object))
    Lc = int(np.prod(qs, dtype=object))
    Kl = K // world
    h = ctypes.c_void_p()
    fk.check(L.fastKronInit(ctypes.byref(h), ctypes.c_uint32(fk.BACKEND_CUDA)))
    streams, xs, res, t1, t2, fd = [], [], [], [], [], []
    try:
        for d in range(world):
            with torch.cuda.device(d):
                streams.append(torch.cuda.Stream())
        sarr = (ctypes.c_void_p * world)(*[s.cuda_stream for s in streams])
        fk.check(L.fastKronMgInitCUDA(h, sarr, world, 1, world, 1))
        ye, te = ctypes.c_size_t(), ctypes.c_size_t()
        fk.check(L.gekmmSizes(h, ctypes.c_uint32(M), ctypes.c_uint32(n), fk.u32arr(ps), fk.u32arr(qs),
                              ctypes.byref(ye), ctypes.byref(te)))
        for d in range(world):
            with torch.cuda.device(d):
                x = torch.empty(M * Kl, dtype=torch.float32, device="cuda")
                _fill_block(x, c, M, K, Kl, d)
                xs.append(x)
                res.append(torch.empty(ye.value, dtype=torch.float32, device="cuda"))
                t1.append(torch.empty(te.value, dtype=torch.float32, device="cuda"))
                t2.append(torch.empty(te.value, dtype=torch.float32, device="cuda"))
                fd.append([torch.from_numpy(f).cuda() for f in fs_host])
                torch.cuda.synchronize()
        P = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])
        kron = (ctypes.c_void_p * (world * n))(*[fd[d][i].data_ptr() for d in range(world) for i in range(n)])
        times = []
        for it in range(1 + reps):
            t0 = time.perf_counter()
            fk.check(L.fastKronMgSGEMM(h, ctypes.c_uint32(n), P(xs), kron, P(res), ctypes.c_uint32(M),
                                       ctypes.c_uint32(Lc), ctypes.c_uint32(K), fk.u32arr(qs), fk.u32arr(ps),
                                       P(t1), P(t2), sarr))
            if it > 0:
                times.append((time.perf_counter() - t0) * 1e3)
        row0 = torch.cat([r.view(M, Lc // world)[0].to("cuda:0") for r in res]).cpu().numpy()
        return float(np.mean(times)), float(min(times)), row0
    finally:
        L.fastKronDestroy(h)
        del xs, res, t1, t2, fd
        torch.cuda.set_device(0)


def run(args, CONFIGS, B):
    import torch
    import torch.distributed as dist
    from fastkron_b200 import mg, synth
    from fastkron_b200 import lib as fk

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("bench.py --gpus %d must be launched with %d ranks (torchrun), got WORLD_SIZE=%d"
                         % (args.gpus, args.gpus, world))
    torch.cuda.set_device(local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    host_group = dist.new_group(backend="gloo")          # host-side barriers that keep the GPUs idle
    c = dict(CONFIGS[args.config], name=args.config)
    if c["mm"] != "mkm" or c["dt"] != "f32" or c["beta"] != 0:
        raise SystemExit("the multi-GPU path is fp32 GeMKM without epilogue (as in the reference)")
    M, ps, qs = c["M"], c["ps"], c["qs"]
    K = int(np.prod(ps, dtype=object))
    Lc = int(np.prod(qs, dtype=object))
    Kl, Ll = K // world, Lc // world

    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        eng = mg.PipelinedRankGeMKM(M, ps, qs, parts=0, mode="auto")
        lanes = int(fk.get().fkbMgPipeLanes(eng.pipe)) if eng.pipe is not None else 1
        x = torch.empty(M * Kl, dtype=torch.float32, device="cuda")
        _fill_block(x, c, M, K, Kl, rank)
        fs_host = [synth.uniform(c["seed"] + 2000 + i, p * q, np.float32) for i, (p, q) in enumerate(zip(ps, qs))]
        fs = [torch.from_numpy(f).cuda() for f in fs_host]
        L = fk.get()
        L.fkbLaunchCount.restype = ctypes.c_ulonglong

        for _ in range(args.warmup):
            eng.run(x, fs)
        torch.cuda.synchronize()
        dist.barrier()
        sampler = B["ClockSampler"](local) if rank == 0 else None
        if sampler:
            sampler.start()
        n0 = L.fkbLaunchCount()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for st in range(args.steps):
            eng.run(x, fs)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        launches = int(L.fkbLaunchCount() - n0)
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        clocks = sampler.stop() if sampler else None
        ms_step = float(ms.item()) / args.steps
        flops = B["flops_library"](c)
        value = flops / (ms_step * 1e-3) / 1e9

        # ---- one call at a time, host-synchronised on both sides (what a blocking caller sees) ----
        tt = []
        for it in range(1 + 5):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.run(x, fs)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it > 0:
                tt.append(float(t.item()))
        single_ms = float(np.mean(tt))

        # ---- where a step's time goes: CUDA events around every kernel of one extra step ----
        L.fkbSetProfiling(eng.h.h, 1)
        eng.run(x, fs)
        torch.cuda.synchronize()
        pm = (ctypes.c_float * 4096)()
        pk = (ctypes.c_int * 4096)()
        npass = L.fkbGetPassTimes(eng.h.h, pm, pk, 4096)
        L.fkbSetProfiling(eng.h.h, 0)
        kernel_ms = [float(pm[i]) for i in range(npass)]
        # ... and how long the exchanges take from the moment their data is ready (staged transport)
        exch = None
        if eng.pipe is not None:
            L.fkbMgPipeTrace(eng.pipe, 1)
            eng.run(x, fs)
            torch.cuda.synchronize()
            tb = (ctypes.c_double * 256)()
            ne = L.fkbMgPipeTraceGet(eng.pipe, tb, 128)
            L.fkbMgPipeTrace(eng.pipe, 0)
            if ne > 0:
                ms_e = [tb[2 * i] for i in range(ne)]
                by_e = [tb[2 * i + 1] for i in range(ne)]
                exch = {"exchanges": ne, "ms_each": [round(v, 3) for v in ms_e], "ms_sum": float(np.sum(ms_e)),
                        "bytes_sent_each": by_e[0], "gbs_per_exchange_mean": float(np.mean([b / (m * 1e-3) / 1e9 for b, m in zip(by_e, ms_e) if m > 0])),
                        "note": "rank 0; from 'data ready' to the last outgoing copy's end, while the other slices compute"}
        dist.barrier()

        # ---- end to end: host block -> device, product, device -> host, every step ---------
        hx = torch.empty(M * Kl, dtype=torch.float32, pin_memory=True)
        hz = torch.empty(M * Ll, dtype=torch.float32, pin_memory=True)
        hx.copy_(x)
        torch.cuda.synchronize()
        e2e_steps = max(1, min(args.steps, 3))
        tt, copy_tt = [], []
        # host operands want row slices whatever the transport: a slice's copies overlap the other
        # slices' passes (the device-resident run above may use one slice, e.g. with two GPUs)
        eng_h = eng if eng.parts >= 8 or M % 8 else mg.PipelinedRankGeMKM(M, ps, qs, parts=8, mode="auto")
        for it in range(1 + e2e_steps):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng_h.run_host(hx, fs, hz)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it > 0:
                tt.append(float(t.item()))
        e2e_ms = float(np.mean(tt))
        e2e_parts = eng_h.parts
        hz_rows = hz.view(M, Ll)[[0, M - 1]].clone()      # (the copy tests further down reuse hz)
        if eng_h is not eng:
            eng_h.close()
        # the copies alone, all ranks at once (what the host's memory system and the PCIe links give)
        xd2 = torch.empty_like(x)
        for it in range(3):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            xd2.copy_(hx, non_blocking=True)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it > 0:
                copy_tt.append(float(t.item()))
        h2d_alone_ms = float(np.mean(copy_tt))
        # both directions at once, all ranks at once: the ceiling of any end-to-end schedule
        zd2 = torch.empty(M * Ll, dtype=torch.float32, device="cuda")
        s_a, s_b = torch.cuda.Stream(), torch.cuda.Stream()
        copy_tt = []
        for it in range(3):
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            s_a.wait_stream(stream)
            s_b.wait_stream(stream)
            with torch.cuda.stream(s_a):
                xd2.copy_(hx, non_blocking=True)
            with torch.cuda.stream(s_b):
                hz.copy_(zd2, non_blocking=True)
            stream.wait_stream(s_a)
            stream.wait_stream(s_b)
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            if it > 0:
                copy_tt.append(float(t.item()))
        duplex_alone_ms = float(np.mean(copy_tt))
        del xd2, zd2

        # ---- parity spot check outside the timed region: two full rows against the oracle ----
        z = eng.run(x, fs).clone()
        torch.cuda.synchronize()
        e2e_same = bool(torch.equal(hz_rows[1].cuda(), z.view(M, Ll)[M - 1]) and
                        torch.equal(hz_rows[0].cuda(), z.view(M, Ll)[0]))
        check = None
        rows = [0, M - 1]
        xr = [torch.empty(len(rows) * Kl, dtype=torch.float32, device="cuda") for _ in range(world)]
        zr = [torch.empty(len(rows) * Ll, dtype=torch.float32, device="cuda") for _ in range(world)]
        dist.all_gather(xr, x.view(M, Kl)[rows].contiguous().view(-1))
        dist.all_gather(zr, z.view(M, Ll)[rows].contiguous().view(-1))
        zfull = None
        if rank == 0 and not args.no_cpu:
            import oracle
            xfull = np.concatenate([t.cpu().numpy().reshape(len(rows), Kl) for t in xr], axis=1)
            zfull = np.concatenate([t.cpu().numpy().reshape(len(rows), Ll) for t in zr], axis=1)
            want = oracle.port_gekmm("mkm", xfull, fs_host, ps, qs, len(rows))
            den = np.abs(want).max(axis=1, keepdims=True)
            check = float((np.abs(zfull.astype(np.float64) - want) / den).max())
        parts, mode = eng.parts, eng.mode
        eng.close()
        del x, z, xr, zr
        torch.cuda.empty_cache()

    # ---- the reference's own entry point, one process driving all GPUs (rank 0, others idle) ----
    torch.cuda.synchronize()
    dist.barrier(group=host_group)
    c_api = None
    if rank == 0:
        try:
            mean_ms, min_ms, row0 = _c_api_blocking_ms(c, world, fs_host)
            c_api = {"ms_per_call": mean_ms, "ms_min": min_ms, "gflops": flops / (mean_ms * 1e-3) / 1e9,
                     "how": "fastKronMgSGEMM (blocking, one process, %d devices), wall clock around the call, mean of 3 after 1 warm-up" % world,
                     "row0_equals_per_rank_result": bool(zfull is not None and np.array_equal(row0, zfull[0])) if zfull is not None else None}
        except Exception as ex:          # report, do not lose the line
            c_api = {"error": str(ex)[:300]}
    dist.barrier(group=host_group)

    if rank == 0:
        peaks, peak_src = B["read_measured_peaks"]()
        fma_probe = B["measure_fma_peak"]("f32")
        fma_props = B["simt_peak_from_props"]("f32")
        fp_peak = max(fma_probe, fma_props)
        per_gpu_tflops = value / world / 1e3
        nv_bytes = 2 * (world - 1) * M * Kl * 4 // world
        roof = {"bound": "fp32_simt", "achieved": per_gpu_tflops, "peak": fp_peak, "unit": "TFLOP/s",
                "frac": per_gpu_tflops / fp_peak if fp_peak else None, "traffic": None,
                "peak_source": "larger of the FMA-chain probe of this run (%.1f) and SMs x lanes x 2 x max SM clock (%.1f)" % (fma_probe, fma_props),
                "kernel": "gemm",
                "note": "whole-step rate per GPU (4 passes + 2 exchanges)",
                "nvlink": {"bytes_per_gpu_per_step": nv_bytes,
                           "gbs_per_direction": nv_bytes / (ms_step * 1e-3) / 1e9,
                           "measured_peer_copy_gbs": 770.0}}
        out = {
            "metric": "GeMKM/GeKMM GFLOP/s", "value": value, "unit": "GFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": B["workload_desc"](c, world),
            "value_harness_count": B["flops_harness"](c) / (ms_step * 1e-3) / 1e9,
            "gpu_launches": launches * world, "clocks": clocks, "roofline": roof,
            "single_call_ms": single_ms,
            "kernel_ms_one_step_rank0": {"sum": float(np.sum(kernel_ms)), "count": len(kernel_ms),
                                         "each": [round(v, 3) for v in kernel_ms[:64]]},
            "exchange_ms_one_step_rank0": exch,
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                    "h2d_bytes_per_step": M * Kl * 4 * world, "d2h_bytes_per_step": M * Ll * 4 * world,
                    "ms_per_step": e2e_ms, "steps": e2e_steps, "row_slices": e2e_parts,
                    "how": "each rank's pinned block: a row slice is copied in ahead of its passes and copied out when complete",
                    "h2d_alone_ms_all_ranks": h2d_alone_ms,
                    "h2d_alone_gbs_aggregate": M * Kl * 4 * world / (h2d_alone_ms * 1e-3) / 1e9,
                    "copies_alone_both_directions_ms_all_ranks": duplex_alone_ms,
                    "copies_alone_gbs_aggregate_per_direction": M * Kl * 4 * world / (duplex_alone_ms * 1e-3) / 1e9,
                    "matches_device_result": e2e_same},
            "cpu_baseline": None, "parity_rows_max_rel_err": check,
            "row_slices": parts, "exchange_mode": mode, "compute_lanes": lanes,
            "c_api_single_process": c_api,
            "exchange": ("2 all-to-alls per step; staged: kernels fill local per-destination blocks, copy engines ship "
                         "them over NVLink; fused: the producing kernels store into the peers; ranks are ordered by "
                         "32-bit sequence flags in device memory (stream memory operations), no collective library "
                         "in the timed region"),
        }
        print(json.dumps(out), flush=True)
    dist.barrier(group=host_group)
    dist.destroy_process_group()
