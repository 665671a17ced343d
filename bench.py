#!/usr/bin/env python
"""Benchmark of the fused tensor-core / CUDA-core hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = a batch of PAIRS_PER_STEP fused GEMM + stencil pairs of the headline configuration (the graph of
one pair replayed that many times, so that the timed region is long enough to average): tzgemm
M = N = 4096, K = 1024 (fp16 in, fp32 out) together with 10 ping-pong Jacobi sweeps of the 7-point
stencil on a 512 x 512 x 64 fp32 grid.  The GEMM's 4096 tiles are fused with the first 10, 2 or 1 of
the sweeps (each fused launch = one sweep + an equal share of the tiles), the remaining sweeps run
alone; the three schedules are timed briefly and the best one is the timed step.  The same work
run unfused (1 tzgemm launch + 10 stencil launches) gives `fused_vs_sequential`; `ratio_sweep` holds
single fused launches at tensor : CUDA-core tile ratios 1:1 ... 1:8, `pairs` the other two pairs.  Multi-GPU = independent replicas, one process per GPU, no collective on
the data path (co-location is per GPU).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the same pair on
the host cores instead, one whole pair per step (the reference project has no CPU implementation and its
CUDA kernels are timed separately, see `ref_gpu` in the default arm's line).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M, N, K = 4096, 4096, 1024
NX, NY, NZ, SWEEPS = 512, 512, 64, 10
C0, C1 = 1.0 / 6.0, -1.0 / 6.0
PAIRS_PER_STEP = 50     # pairs per timed step (graph replays)
CD_THREADS = 448        # CUDA-core threads of the fused CTA (14 warps next to the 6 tensor-role warps)
SOLO_CD_THREADS = 256   # solo stencil: 2 CTAs of 8 warps per SM
TILES = (M // 64) * (N // 64)
CD_BLOCKS = (NX // 64) * (NY // 4)
WORKLOAD = (f"config 2: fused tzgemm {M}x{N}x{K} fp16->fp32 + {SWEEPS} Jacobi sweeps of the 7-point stencil on "
            f"{NX}x{NY}x{NZ} fp32 (c0=1/6, c1=-1/6, zero boundary)")
METRIC = "fused GEMM+stencil pairs per second (fused vs sequential kernel time in fused_vs_sequential)"

# algorithmic bytes of one fused launch: one sweep (one fp32 read + one fp32 write per cell) plus
# one tenth of the GEMM's minimum traffic (A and B read once, C written once)
SWEEP_BYTES = 8 * NX * NY * NZ
GEMM_BYTES = 2 * (M * K + N * K) + 4 * M * N
LAUNCH_BYTES = SWEEP_BYTES + GEMM_BYTES / SWEEPS
# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from ncu captures of these two kernels on this
# workload (caches flushed by ncu before the launch; part of the output is still dirty in L2 when the kernel ends)
# mix_stencil_kernel: the launch with a tenth of the tiles; mix_stencil2_kernel: the CTA-pair launch with half of them
NCU_TRAFFIC_BYTES = {"stencil_tma_kernel": 94.05e6, "mix_stencil_kernel": 108.3e6, "mix_stencil2_kernel": 138.0e6}


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class ClockSampler(threading.Thread):
    """Reads (never sets) SM clock and throttle reasons through NVML while the GPU is under load."""

    def __init__(self, index: int, period_s: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.active = threading.Event()
        self.ok = False

    def run(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {
                pynvml.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                pynvml.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                pynvml.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
                pynvml.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
            }
            self.ok = True
            while not self._stop_evt.is_set():
                if self.active.is_set():
                    self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                    r = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                    for bit, name in names.items():
                        if r & bit:
                            self.reasons.add(name)
                time.sleep(self.period)
        except Exception as e:  # NVML missing: report that, do not invent numbers
            self.error = repr(e)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples),
                "how": "NVML, 20 ms period, sampled during the timed loops and a continuation of the same loop"}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------------------------------------
# CPU arm: the restatement of the same pair on the host cores (bounded sample, extrapolated)
# ------------------------------------------------------------------------------------------------
def cpu_pair_setup():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import tacker_oracle as oracle

    _, a = oracle.uniform_f16(M * K, 11, -1.0, 1.0)
    _, b = oracle.uniform_f16(N * K, 12, -1.0, 1.0)
    grid = oracle.uniform_f32(NX * NY * NZ, 100, 0.0, 1.0).reshape(NZ, NY, NX)
    return oracle, np, a.reshape(M, K), b.reshape(N, K), grid


def cpu_pair(state):
    """One whole pair (all 4096 GEMM tiles, all 10 sweeps) on the host cores; returns seconds."""
    oracle, np, a, b, grid = state
    out = np.zeros((M, N), dtype=np.float32)
    x, y = grid.copy(), grid.copy()
    t0 = time.perf_counter()
    oracle.tzgemm_f32(a, b, alpha=1.0, start=0, end=TILES, out=out)
    oracle.stencil_jacobi_f32(np.float32(C0), np.float32(C1), x, y, SWEEPS, contract=1)
    return time.perf_counter() - t0


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    state = cpu_pair_setup()
    oracle = state[0]
    cores = oracle.set_threads(os.cpu_count() or 1)
    for _ in range(args.warmup):
        cpu_pair(state)
    t = [cpu_pair(state) for _ in range(args.steps)]
    sec = sum(t) / len(t)
    sample = ("per step: ONE whole pair (all 4096 GEMM tiles + all 10 sweeps), measured, nothing scaled; the GPU arm's "
              f"step is a batch of {PAIRS_PER_STEP} such pairs, so compare `value` (pairs/s), not ms_per_step")
    line = {
        "impl": "reference", "metric": METRIC, "value": 1.0 / sec, "unit": "pairs/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 inputs, f32 accumulate / f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "pairs_per_step": 1,
                   "arm": "CPU restatement of the pair (the reference has no CPU code; oracle/tacker_oracle.c, OpenMP, "
                          "scalar binary32)"},
        "cpu_baseline": {"value": 1.0 / sec, "unit": "pairs/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": 1.0 / sec, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels are sm_100a only and there is no CPU fallback")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    from tacker_b200 import ops
    from tacker_b200.replicas import Replicas

    rep = Replicas(backend="nccl", device=torch.device("cuda", local))
    rank, world = rep.rank, rep.world
    sms = ops.sm_count()
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    stream = torch.cuda.Stream()
    st = stream.cuda_stream

    def make_graph(fn):
        if args.no_graph:
            return fn
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()  # everything lazy (symbol addresses, attributes) happens before capture
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
        return g.replay

    def timed(fn, steps, warmup):
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            rep.barrier()
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            rep.barrier()
        return rep.max(e0.elapsed_time(e1)) / steps  # ms per step, max over ranks

    def t_of(kernels, reps=None):
        """us per pass over `kernels`; `reps` passes back to back in one graph so launch overhead cannot starve the GPU"""
        reps = reps or (2 if args.quick else 20)

        def fn():
            for _ in range(reps):
                for k in kernels:
                    k.execute(st)
        return timed(make_graph(fn), 3, 2) / reps * 1e3

    if args.profile_gemm:  # a few launches of the solo tzgemm on one shape (for profiler captures)
        m, n, k = (int(v) for v in args.profile_gemm.lower().split("x"))
        a = (torch.rand(m, k, device="cuda", generator=gen) * 2 - 1).half()
        b = (torch.rand(n, k, device="cuda", generator=gen) * 2 - 1).half()
        c = torch.zeros(m, n, device="cuda")
        for name, value in (("tzgemm_pair", args.gemm_pair), ("tzgemm_m256", args.gemm_m256)):
            ops.set_option(name, value)
        kern = ops.gptb_tzgemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, alpha=1.0, grid=sms)
        us = t_of([kern], 20)
        for _ in range(3):
            kern.execute(st)
        torch.cuda.synchronize()
        if rank == 0:
            print(json.dumps({"profile_gemm": args.profile_gemm, "tzgemm_pair": args.gemm_pair,
                              "tzgemm_m256": args.gemm_m256, "us": round(us, 2),
                              "tflops": round(2.0 * m * n * k / us / 1e6, 1), "status": ops.device_status()}), flush=True)
        rep.close()
        return

    if args.only_more:  # just sgemm, lbm, fft and cutcp with their pairs
        if rank == 0:
            print(json.dumps({"pairs": more_kernels(torch, ops, sms, gen, t_of, measured_peaks()[0])}), flush=True)
        rep.close()
        return

    if args.only_pairs or args.profile_pair:  # just the Coulomb and MRI-Q pairs (used for profiler captures of those kernels)
        if rank == 0:
            print(json.dumps({"pairs": other_pairs(torch, ops, sms, gen, t_of, st, args.profile_pair, args.profile_w,
                                                       args.profile_blocks)}),
                  flush=True)
        rep.close()
        return

    # ---------------- config 2: GEMM 4096 x 4096 x 1024 + 10 Jacobi sweeps ----------------
    A = (torch.rand(M, K, device="cuda", generator=gen) * 2 - 1).half()
    B = (torch.rand(N, K, device="cuda", generator=gen) * 2 - 1).half()
    Cm = torch.zeros(M, N, device="cuda")
    g0 = torch.rand(NZ, NY, NX, device="cuda", generator=gen)
    for sl in ((0,), (-1,), (slice(None), 0), (slice(None), -1), (slice(None), slice(None), 0),
               (slice(None), slice(None), -1)):
        g0[sl] = 0.0
    g1 = g0.clone()
    grids = (g0, g1)

    def tz_kernel(start=0, end=TILES):
        return ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cm.data_ptr(), M, N, K, alpha=1.0, start=start, end=end,
                               grid=sms)

    def cd_kernel(it):
        src, dst = grids[it & 1], grids[(it + 1) & 1]
        return ops.gptb_stencil(C0, C1, src.data_ptr(), dst.data_ptr(), NX, NY, NZ, grid=sms * 2, block=SOLO_CD_THREADS)

    def schedule(fuse_sweeps):
        """The pair as `fuse_sweeps` fused launches (sweep i + an equal share of the GEMM's tiles) followed by
        the remaining sweeps alone.  10 = every sweep fused (1 tensor tile : 2.5 CUDA-core blocks)."""
        bounds = [TILES * i // fuse_sweeps for i in range(fuse_sweeps + 1)]
        ks = [ops.mix(cd_kernel(i), tz_kernel(), cd_threads=CD_THREADS, grid=sms, tz_range=(bounds[i], bounds[i + 1]))
              for i in range(fuse_sweeps)]
        return ks + [cd_kernel(i) for i in range(fuse_sweeps, SWEEPS)]

    sequential = [tz_kernel()] + [cd_kernel(i) for i in range(SWEEPS)]

    def runner(kernels):
        def fn():
            for k in kernels:
                k.execute(st)
        return make_graph(fn)

    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    warm = max(args.warmup, 3)
    sampler.active.set()

    # pick the fused schedule (each candidate timed briefly; every rank picks the same one)
    cands = {}
    for f in (SWEEPS, 2, 1):
        cands[f] = timed(runner(schedule(f)), 50 if not args.quick else 2, 3)
    best = min(cands, key=cands.get) if args.fuse_sweeps == 0 else args.fuse_sweeps
    fused_kernels = schedule(best)
    fused_fn = runner(fused_kernels)
    seq_fn = runner(sequential)

    def batch(fn):
        def step():
            for _ in range(PAIRS_PER_STEP):
                fn()
        return step

    ms_step = timed(batch(fused_fn), args.steps, warm)          # the timed region: K steps of PAIRS_PER_STEP pairs
    ms_fused = ms_step / PAIRS_PER_STEP
    ms_seq = timed(batch(seq_fn), max(1, args.steps // 4), 1) / PAIRS_PER_STEP
    # continuation of the same fused loop, only to give the 20 ms clock sampler enough samples
    t_end = time.time() + args.sustain_ms / 1e3
    with torch.cuda.stream(stream):
        while time.time() < t_end:
            for _ in range(50):
                fused_fn()
            stream.synchronize()
    sampler.active.clear()
    status = ops.device_status()

    # ---- the kernels one by one (explain the headline) ----
    us_gemm = t_of([tz_kernel()])

    # yardstick only, never on the measured path: the vendor library's GEMM on the same operands, timed the same way
    # (fp32 output like tzgemm where this torch has `out_dtype`, else the cheaper fp16 output)
    def library_gemm_us():
        Bt = B.t()
        try:
            torch.mm(A, Bt, out_dtype=torch.float32)
            call, out = (lambda: torch.mm(A, Bt, out_dtype=torch.float32)), "fp32 out"
        except Exception:
            call, out = (lambda: torch.mm(A, Bt)), "fp16 out"
        reps = 2 if args.quick else 20

        def fn():
            for _ in range(reps):
                call()
        with torch.cuda.stream(stream):
            us = timed(make_graph(fn), 3, 2) / reps * 1e3
        return us, out
    try:
        us_lib, lib_out = library_gemm_us()
    except Exception as e:  # the yardstick must never take the benchmark down
        us_lib, lib_out = None, f"unavailable: {type(e).__name__}"
    us_sweep = t_of([cd_kernel(i) for i in range(SWEEPS)]) / SWEEPS

    # yardstick only: a plain device copy of one grid (the same 64 MiB read and 64 MiB written as one sweep), on
    # buffers of its own
    def grid_copy_us():
        scratch = (torch.empty_like(g0), torch.empty_like(g0))
        reps = 2 if args.quick else 20

        def fn():
            for i in range(reps):
                scratch[(i + 1) & 1].copy_(scratch[i & 1])
        with torch.cuda.stream(stream):
            return timed(make_graph(fn), 3, 2) / reps * 1e3
    try:
        us_copy = grid_copy_us()
    except Exception:  # the yardstick must never take the benchmark down
        us_copy = None
    us_fused_launch = {}
    for f in (SWEEPS, 2, 1):
        lo, hi = 0, TILES // f
        us_fused_launch[f] = t_of([ops.mix(cd_kernel(i), tz_kernel(), cd_threads=CD_THREADS, grid=sms, tz_range=(lo, hi))
                                   for i in range(2)]) / 2
    sweep = []
    if not args.quick:
        def point(label, nt, f, w):
            t_gs = t_of([tz_kernel(0, nt)])
            s_ = t_gs + us_sweep
            sweep.append({"tensor_to_cd_tiles": label, "gemm_tiles": nt, "cd_blocks": CD_BLOCKS, "cd_threads": w,
                          "fused_us": round(f, 2), "sequential_us": round(s_, 2), "ratio": round(f / s_, 4),
                          "attainable": round(max(t_gs, us_sweep) / s_, 4)})

        for r in (1, 2, 3, 4, 5, 6, 7, 8):
            nt = CD_BLOCKS // r  # GEMM tiles co-run with one sweep's 1024 CUDA-core blocks: 1 : r
            best_w = None
            for w in (320, 448, 576):  # the other half of the ratio: CUDA-core threads next to the 192 tensor-role ones
                f = t_of([ops.mix(cd_kernel(i), tz_kernel(), cd_threads=w, grid=sms, tz_range=(0, nt))
                          for i in range(2)]) / 2
                if best_w is None or f < best_w[0]:
                    best_w = (f, w)
            point(f"1:{r}", nt, best_w[0], best_w[1])
        for nt in (2048, 4096):
            point(f"{nt // CD_BLOCKS}:1", nt, us_fused_launch[TILES // nt], CD_THREADS)

    # ---- the other two pairs (configs 3 and 4): fused vs sequential on identical work ----
    pairs = None
    if not args.quick:
        pairs = other_pairs(torch, ops, sms, gen, t_of, st)
        pairs.update(more_kernels(torch, ops, sms, gen, t_of, measured_peaks()[0]))

    # ---- end to end through the host-buffer C-ABI call ----
    hA, hB = A.cpu().pin_memory(), B.cpu().pin_memory()
    hA0 = g0.cpu().pin_memory()
    hC = torch.empty(M, N).pin_memory()
    hOut = torch.empty(NZ, NY, NX).pin_memory()
    ws_bytes = ops.pair_tzgemm_stencil_workspace(M, N, K, NX, NY, NZ)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")

    def e2e_step():
        ops.pair_tzgemm_stencil_host(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), M, N, K, 1.0, C0, C1,
                                     hA0.data_ptr(), hOut.data_ptr(), NX, NY, NZ, SWEEPS, CD_THREADS, ws.data_ptr(),
                                     ws_bytes, st)

    e2e_pairs = 20 if not args.quick else 3
    ms_e2e = timed(e2e_step, e2e_pairs, 3)
    h2d = hA.numel() * 2 + hB.numel() * 2 + hA0.numel() * 4
    d2h = hC.numel() * 4 + hOut.numel() * 4

    # the ceiling of that call: the same bytes as plain cudaMemcpyAsync, both directions at once, no kernels
    up_stream = torch.cuda.Stream()
    dA, dB, dG, dC, dO = (torch.empty_like(t, device="cuda") for t in (hA, hB, hA0, hC, hOut))

    def copy_only():
        up_stream.wait_stream(stream)
        with torch.cuda.stream(up_stream):
            dA.copy_(hA, non_blocking=True)
            dB.copy_(hB, non_blocking=True)
            dG.copy_(hA0, non_blocking=True)
        hOut.copy_(dO, non_blocking=True)
        hC.copy_(dC, non_blocking=True)
        stream.wait_stream(up_stream)

    ms_copy = timed(copy_only, e2e_pairs, 3)
    del dA, dB, dG, dC, dO
    clocks = sampler.stop()

    # ---- the reference's own fused kernel, recompiled for sm_100 (when the test build travelled) ----
    ref_gpu = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import tacker_ref as ref

        if ref.available() and rank == 0 and world == 1 and not args.quick:
            bounds = [TILES * i // SWEEPS for i in range(SWEEPS + 1)]

            def ref_fused():
                for i in range(SWEEPS):
                    src, dst = grids[i & 1], grids[(i + 1) & 1]
                    ref.mix_stencil(C0, C1, src.data_ptr(), dst.data_ptr(), NX, NY, NZ, 0, CD_BLOCKS, A.data_ptr(),
                                    B.data_ptr(), Cm.data_ptr(), M, N, K, bounds[i], bounds[i + 1], sms * 2, st)

            def ref_seq():
                ref.tzgemm(A.data_ptr(), B.data_ptr(), Cm.data_ptr(), M, N, K, 0, TILES, sms * 2, st)
                for i in range(SWEEPS):
                    src, dst = grids[i & 1], grids[(i + 1) & 1]
                    ref.stencil(C0, C1, src.data_ptr(), dst.data_ptr(), NX, NY, NZ, 0, CD_BLOCKS, sms * 3, st)

            rf, rs = timed(ref_fused, 10, 3), timed(ref_seq, 10, 3)
            ref_gpu = {"what": "reference wmma/GPTB kernels recompiled for sm_100, same pair, same GPU",
                       "fused_ms_per_pair": round(rf, 4), "sequential_ms_per_pair": round(rs, 4),
                       "fused_vs_sequential": round(rf / rs, 4)}
    except Exception as e:  # test infrastructure absent: not an error of the product
        ref_gpu = {"unavailable": repr(e)[:120]}

    # ---- request-driven co-location on this GPU (LC VGG16 b1 at 200 q/s Poisson, BE BERT-base b8 s128) ----
    coloc = None
    if not args.quick and args.colocate_s > 0:
        try:
            from tacker_b200 import colocate

            c = colocate.run(1, args.colocate_s, 200.0, 1.5, devices=[physical_gpu_index(local)])
            coloc = {k: c[k] for k in ("be_qps_total", "lc_p99_ms_max", "lc_solo_p99_ms_max", "qos_met_all", "seconds",
                                       "lc", "be", "qps_offered_per_gpu")}
            # the same LC stream with the benchmark kernel as the best-effort job: blocks riding inside the LC layers'
            # fused kernels against plain time slicing (shorter phases: three of them)
            f = colocate.run_fused(1, min(args.colocate_s, 20.0), 200.0, 1.5, devices=[physical_gpu_index(local)])
            coloc["fused_mode"] = {k: f[k] for k in ("be_kernel", "seconds_per_phase", "fused_layers", "mixable_layers",
                                                     "blocks_per_fused_query", "timesliced_be_blocks_per_s",
                                                     "fused_be_blocks_per_s", "timesliced_lc_p99_ms_max",
                                                     "fused_lc_p99_ms_max", "qos_bound_ms_min", "qos_met_all")}
        except Exception as e:
            coloc = {"unavailable": repr(e)[:200]}
        gathered = rep.gather(coloc)
        if all(isinstance(g, dict) and "be_qps_total" in g for g in gathered):
            fm = [g.get("fused_mode") for g in gathered]
            coloc = dict(coloc, be_qps_total=sum(g["be_qps_total"] for g in gathered),
                         lc_p99_ms_max=max(g["lc_p99_ms_max"] for g in gathered),
                         qos_met_all=all(g["qos_met_all"] for g in gathered), gpus=world)
            if all(isinstance(m, dict) for m in fm):
                coloc["fused_mode"] = dict(fm[0], timesliced_be_blocks_per_s=sum(m["timesliced_be_blocks_per_s"] for m in fm),
                                           fused_be_blocks_per_s=sum(m["fused_be_blocks_per_s"] for m in fm),
                                           fused_lc_p99_ms_max=max(m["fused_lc_p99_ms_max"] for m in fm),
                                           timesliced_lc_p99_ms_max=max(m["timesliced_lc_p99_ms_max"] for m in fm),
                                           qos_met_all=all(m["qos_met_all"] for m in fm))

    cpu = None
    if rank == 0 and world == 1 and not args.quick:
        state = cpu_pair_setup()
        cores = state[0].set_threads(os.cpu_count() or 1)
        cpu_pair(state)
        secs = [cpu_pair(state) for _ in range(5)]
        sec = sum(secs) / len(secs)
        cpu = {"value": 1.0 / sec, "unit": "pairs/s", "cores": cores, "kind": "port",
               "sample": "5 whole pairs (all GEMM tiles + 10 sweeps each) after one warm-up pair, mean; nothing scaled"}

    if rank != 0:
        rep.close()
        return
    hbm, tflops, which = measured_peaks()
    # the kernel with the largest share of the step's device time
    n_solo = SWEEPS - best
    share_solo = n_solo * us_sweep / (ms_fused * 1e3)
    if share_solo >= 0.5:
        roof = {"kernel": "stencil_tma_kernel (one sweep, solo)", "launches_per_step": n_solo,
                "share_of_step": round(share_solo, 3), "bound": "hbm", "achieved": SWEEP_BYTES / (us_sweep * 1e-6) / 1e9,
                "algorithmic_bytes_per_launch": SWEEP_BYTES, "traffic": NCU_TRAFFIC_BYTES.get("stencil_tma_kernel")}
    else:
        bytes_launch = SWEEP_BYTES + GEMM_BYTES / best
        roof = {"kernel": "mix_stencil_kernel (one sweep + 1/%d of the GEMM tiles)" % best, "launches_per_step": best,
                "share_of_step": round(1.0 - share_solo, 3), "bound": "hbm",
                "achieved": bytes_launch / (us_fused_launch[best] * 1e-6) / 1e9,
                "algorithmic_bytes_per_launch": bytes_launch, "traffic": NCU_TRAFFIC_BYTES.get("mix_stencil_kernel")}
    roof.update({"peak": hbm, "unit": "GB/s", "frac": roof["achieved"] / hbm,
                 "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({which})",
                 "tensor_frac_solo_gemm": round(2.0 * M * N * K / (us_gemm * 1e-6) / 1e12 / tflops, 4)})
    line = {
        "metric": METRIC, "value": world * 1e3 / ms_fused, "unit": "pairs/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_step, "ms_per_pair": ms_fused, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 inputs, f32 accumulate (tensor role) / f32 (CUDA-core role)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "pairs_per_step": PAIRS_PER_STEP, "cd_threads": CD_THREADS, "grid": sms,
                   "replicas": world, "colocation_seconds": args.colocate_s,
                   "schedule": f"{best} fused launches (sweep + {TILES // best} GEMM tiles each) + {SWEEPS - best} solo sweeps",
                   "l2": "inputs 80 MiB (GEMM) + 128 MiB (grids) exceed the 126 MB L2; no flush between steps",
                   "launch": "CUDA graph of the step's launches" if not args.no_graph else "stream launches"},
        "fused_vs_sequential": ms_fused / ms_seq, "sequential_ms_per_pair": ms_seq,
        "attainable": max(us_gemm, SWEEPS * us_sweep) / (us_gemm + SWEEPS * us_sweep),
        "schedules_ms_per_pair": {f"{f}_fused_launches": round(v, 4) for f, v in cands.items()},
        "solo_us": {"tzgemm_4096x4096x1024": round(us_gemm, 2), "stencil_sweep": round(us_sweep, 2),
                    "tzgemm_tflops": round(2.0 * M * N * K / (us_gemm * 1e-6) / 1e12, 1),
                    "library_gemm_same_shape": {"us": None if us_lib is None else round(us_lib, 2), "output": lib_out,
                                                "tzgemm_vs_library": None if us_lib is None else round(us_lib / us_gemm, 3)},
                    "stencil_gbs": round(SWEEP_BYTES / (us_sweep * 1e-6) / 1e9, 1),
                    "device_copy_of_one_grid": None if us_copy is None else round(us_copy, 2),
                    "fused_launch_us": {f"sweep+{TILES // f}_tiles": round(v, 2) for f, v in us_fused_launch.items()}},
        "ratio_sweep": sweep, "pairs": pairs, "clocks": clocks,
        "e2e": {"value": world * 1e3 / ms_e2e, "unit": "pairs/s", "h2d_bytes_per_step": h2d * PAIRS_PER_STEP,
                "d2h_bytes_per_step": d2h * PAIRS_PER_STEP, "h2d_bytes_per_pair": h2d, "d2h_bytes_per_pair": d2h,
                "ms_per_pair": ms_e2e, "pairs_timed": e2e_pairs,
                "copy_ceiling_ms_per_pair": ms_copy, "frac_of_copy_ceiling": ms_copy / ms_e2e,
                "copy_ceiling": "the pair's 84 MB up and 134 MB down as plain cudaMemcpyAsync from/to the same pinned "
                                "buffers on two streams, no kernels, all ranks at once (max over ranks)",
                "call": "tk_pair_tzgemm_stencil_host (pinned host buffers in and out)"},
        "gpu_launches": args.steps * PAIRS_PER_STEP * len(fused_kernels),
        "roofline": roof, "cpu_baseline": cpu, "ref_gpu": ref_gpu, "colocation": coloc, "device_status": status,
    }
    print(json.dumps(line), flush=True)
    rep.close()


def balanced_quantum(t_of, make_cd, total_blocks, t_gemm, t_cd_full):
    """Blocks of CUDA-core work whose solo time is within [0.8, 1.25] of the GEMM's, found by measurement."""
    nb = max(1, min(total_blocks, int(round(total_blocks * t_gemm / t_cd_full))))
    t = t_of([make_cd(0, nb)], 10)
    for _ in range(3):
        if 0.9 <= t / t_gemm <= 1.1:
            break
        nb2 = max(1, min(total_blocks, int(round(nb * t_gemm / t))))
        if nb2 == nb:
            break
        nb = nb2
        t = t_of([make_cd(0, nb)], 10)
    return nb, t


def pair_report(ops, sms, t_of, tz, make_cd, total_blocks, cd_name, w_sweep, tz_tiles=0):
    """One GEMM + CUDA-core pair: as stated (whole kernels) and balanced in time, fused vs the two solo launches.

    `attainable` = max(a, b) / (a + b): what perfect overlap of the two solo kernels would give.  The fused launch is
    timed for every CUDA-core thread count in `w_sweep` (the other half of the tensor : CUDA-core ratio).  Where the
    whole CUDA-core kernel is shorter than the GEMM and `tz_tiles` (the GEMM's 64 x 64 tiles) is given, the balanced
    case shortens the GEMM to a tile range of the same duration instead."""
    t_g, t_c = t_of([tz()], 10), t_of([make_cd()], 5)
    full = {}
    for w in w_sweep:
        full[w] = t_of([ops.mix(make_cd(), tz(), cd_threads=w, grid=sms)], 5)
    wb = min(full, key=full.get)
    if tz_tiles and t_c < 0.9 * t_g:
        nt, t_gb = balanced_quantum(t_of, tz, tz_tiles, t_c, t_g)
        bal = {w: t_of([ops.mix(make_cd(), tz(), cd_threads=w, grid=sms, tz_range=(0, nt))], 10) for w in w_sweep}
        wbb = min(bal, key=bal.get)
        return {
            "gemm_us": round(t_g, 1), f"{cd_name}_us": round(t_c, 1), "fused_us": round(full[wb], 1), "cd_threads": wb,
            "fused_vs_sequential": round(full[wb] / (t_g + t_c), 4), "attainable": round(max(t_g, t_c) / (t_g + t_c), 4),
            "fused_us_by_cd_threads": {str(w): round(v, 1) for w, v in full.items()},
            "balanced": {"gemm_tiles": nt, "gemm_us": round(t_gb, 1), f"{cd_name}_us": round(t_c, 1),
                         "cd_over_gemm": round(t_c / t_gb, 3), "fused_us": round(bal[wbb], 1), "cd_threads": wbb,
                         "fused_vs_sequential": round(bal[wbb] / (t_gb + t_c), 4),
                         "attainable": round(max(t_gb, t_c) / (t_gb + t_c), 4),
                         "fused_us_by_cd_threads": {str(w): round(v, 1) for w, v in bal.items()}}}
    nb, t_cb = balanced_quantum(t_of, make_cd, total_blocks, t_g, t_c)
    bal = {}
    for w in w_sweep:
        bal[w] = t_of([ops.mix(make_cd(0, nb), tz(), cd_threads=w, grid=sms)], 10)
    wbb = min(bal, key=bal.get)
    return {
        "gemm_us": round(t_g, 1), f"{cd_name}_us": round(t_c, 1), "fused_us": round(full[wb], 1), "cd_threads": wb,
        "fused_vs_sequential": round(full[wb] / (t_g + t_c), 4), "attainable": round(max(t_g, t_c) / (t_g + t_c), 4),
        "fused_us_by_cd_threads": {str(w): round(v, 1) for w, v in full.items()},
        "balanced": {f"{cd_name}_blocks": nb, f"{cd_name}_us": round(t_cb, 1), "cd_over_gemm": round(t_cb / t_g, 3),
                     "fused_us": round(bal[wbb], 1), "cd_threads": wbb,
                     "fused_vs_sequential": round(bal[wbb] / (t_g + t_cb), 4),
                     "attainable": round(max(t_g, t_cb) / (t_g + t_cb), 4),
                     "fused_us_by_cd_threads": {str(w): round(v, 1) for w, v in bal.items()}}}


def other_pairs(torch, ops, sms, gen, t_of, st, profile=None, profile_w=832, profile_blocks=0):
    """Configs 3 and 4: GEMM + Coulomb (compute-bound CUDA-core pair), GEMM + MRI-Q (SFU-bound pair).

    profile = "cp" | "mriq": only find that pair's balanced quantum with solo launches, then run its fused launch
    three times with `profile_w` CUDA-core threads (the launches a profiler capture of the fused kernel wants)."""
    out = {}
    w_sweep = (448, 576, 704, 832)

    def profile_run(tz, make_cd, total_blocks):
        if profile_blocks > 0:
            nb, t_g, t_cb = profile_blocks, 0.0, 0.0
        else:
            t_g, t_c = t_of([tz()], 10), t_of([make_cd()], 5)
            nb, t_cb = balanced_quantum(t_of, make_cd, total_blocks, t_g, t_c)
        k = ops.mix(make_cd(0, nb), tz(), cd_threads=profile_w, grid=sms)
        for _ in range(3):
            k.execute(st)
        torch.cuda.synchronize()
        return {"gemm_us": round(t_g, 1), "cd_us": round(t_cb, 1), "cd_blocks": nb, "cd_threads": profile_w}

    def gemm(m, n, k):
        a = (torch.rand(m, k, device="cuda", generator=gen) * 2 - 1).half()
        b = (torch.rand(n, k, device="cuda", generator=gen) * 2 - 1).half()
        c = torch.zeros(m, n, device="cuda")
        return lambda s=0, e=None: ops.gptb_tzgemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, alpha=1.0, start=s,
                                                   end=e, grid=sms), (a, b, c)

    # config 3: GEMM 2048^3 + 8192 atoms on a 512 x 512 lattice
    tz, keep3 = gemm(2048, 2048, 2048)
    atoms = torch.rand(8192, 4, device="cuda", generator=gen) * 64
    atoms[:, 3] = torch.rand(8192, device="cuda", generator=gen) * 2 - 1
    packed = torch.empty_like(atoms)
    lat = torch.zeros(512, 512, device="cuda")
    ops.cp_pack_atoms(atoms.data_ptr(), 8192, 32.0, packed.data_ptr(), st)
    ops.set_option("cp_ppt", 8)
    cp = lambda s=0, e=None: ops.gptb_cp(8192, 0.125, lat.data_ptr(), packed.data_ptr(), 512, 512, start=s, end=e,
                                         grid=sms * 2, block=512)
    if profile == "cp":
        return {"profile_cp": profile_run(tz, cp, 256)}
    r = pair_report(ops, sms, t_of, tz, cp, 256, "coulomb", w_sweep) if profile is None else {"coulomb_us": 1.0}
    r["coulomb_gpairs_per_s"] = round(8192.0 * 512 * 512 / r["coulomb_us"] / 1e3, 1)
    r["coulomb_frac_of_rsqrt_bound"] = round(8192.0 * 512 * 512 / (sms * 16 * 1.965e9) / (r["coulomb_us"] * 1e-6), 3)
    out["config3_gemm2048_coulomb"] = r

    # config 4: GEMM 4096 x 4096 x 2048 + MRI-Q 2048 samples x 262144 voxels
    tz4, keep4 = gemm(4096, 4096, 2048)
    numK, numX = 2048, 262144
    kv = torch.rand(numK, 4, device="cuda", generator=gen) - 0.5
    kv[:, 3] = torch.rand(numK, device="cuda", generator=gen)
    xyz = [torch.rand(numX, device="cuda", generator=gen) * 64 - 32 for _ in range(3)]
    qr, qi = torch.zeros(numX, device="cuda"), torch.zeros(numX, device="cuda")
    mq = lambda s=0, e=None: ops.gptb_mriq(numK, xyz[0].data_ptr(), xyz[1].data_ptr(), xyz[2].data_ptr(), qr.data_ptr(),
                                           qi.data_ptr(), kv.data_ptr(), numX, start=s, end=e, grid=sms * 2, block=512)
    if profile == "mriq":
        return {"profile_mriq": profile_run(tz4, mq, 1024)}
    r = pair_report(ops, sms, t_of, tz4, mq, 1024, "mriq", w_sweep)
    r["mriq_gpairs_per_s"] = round(numK * numX / r["mriq_us"] / 1e3, 1)
    r["mriq_frac_of_sfu_bound"] = round(2.0 * numK * numX / (sms * 16 * 1.965e9) / (r["mriq_us"] * 1e-6), 3)
    out["config4_gemm4096x2048_mriq"] = r

    # the same GEMM with MRI-FHd, the best-effort kernel of the shipped schedule (2048 samples x 262144 voxels)
    fkv = torch.rand(5 * numK, device="cuda", generator=gen) - 0.5
    fr, fi = torch.zeros(numX, device="cuda"), torch.zeros(numX, device="cuda")
    mf = lambda s=0, e=None: ops.gptb_mrif(numK, xyz[0].data_ptr(), xyz[1].data_ptr(), xyz[2].data_ptr(), fr.data_ptr(),
                                           fi.data_ptr(), fkv.data_ptr(), numX, start=s, end=e, grid=sms * 2, block=512)
    r = pair_report(ops, sms, t_of, tz4, mf, 1024, "mrif", w_sweep)
    r["mrif_frac_of_sfu_bound"] = round(2.0 * numK * numX / (sms * 16 * 1.965e9) / (r["mrif_us"] * 1e-6), 3)
    out["gemm4096x2048_mrif"] = r
    del keep3, keep4
    return out


def more_kernels(torch, ops, sms, gen, t_of, hbm_gbs):
    """sgemm, lbm, fft and cutcp at the reference's sizes: solo time with the bound that applies, and each fused with the
    GEMM 4096 x 4096 x 2048 (as stated and balanced in time)."""
    import numpy as np

    from tacker_b200.profile_ratios import cutcp_problem

    a = (torch.rand(4096, 2048, device="cuda", generator=gen) * 2 - 1).half()
    b = (torch.rand(4096, 2048, device="cuda", generator=gen) * 2 - 1).half()
    c = torch.zeros(4096, 4096, device="cuda")
    tz = lambda s=0, e=None: ops.gptb_tzgemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), 4096, 4096, 2048, alpha=1.0, start=s,
                                             end=e, grid=sms)
    out = {}
    fp32_peak = sms * 128 * 2 * 1.965e9  # fused multiply-adds of the CUDA cores at the maximum clock

    M, N, K = 4096, 4128, 4064           # src/ori_kernel/sgemm_kernel.cu:85-87
    sa, sb = torch.rand(K, M, device="cuda", generator=gen), torch.rand(K, N, device="cuda", generator=gen)
    sc = torch.zeros(N, M, device="cuda")
    sg = lambda s=0, e=None: ops.gptb_sgemm(sa.data_ptr(), sb.data_ptr(), sc.data_ptr(), M, N, K, start=s, end=e,
                                            grid=sms * 2, block=256)
    r = pair_report(ops, sms, t_of, tz, sg, (M // 128) * (N // 16), "sgemm", (256, 384))
    r["sgemm_tflops"] = round(2.0 * M * N * K / r["sgemm_us"] / 1e6, 2)
    r["sgemm_frac_of_fp32_peak"] = round(2.0 * M * N * K / (r["sgemm_us"] * 1e-6) / fp32_peak, 3)
    out["gemm4096x2048_sgemm"] = r
    del sa, sb, sc

    nx = ny = nz = 128                    # src/header/lbm_header.h:17-19
    cells, margin = nx * ny * nz, 2 * nx * ny
    lsrc = torch.rand(20 * cells + 2 * margin, device="cuda", generator=gen)
    ldst = torch.rand(20 * cells + 2 * margin, device="cuda", generator=gen)
    lb = lambda s=0, e=None: ops.gptb_lbm(lsrc.data_ptr() + 4 * margin, ldst.data_ptr() + 4 * margin, nx, ny, nz, start=s, end=e,
                                          grid=sms * 2, block=512)
    r = pair_report(ops, sms, t_of, tz, lb, ny * nz, "lbm", (576, 832))
    r["lbm_gbs"] = round(156.0 * cells / r["lbm_us"] / 1e3, 1)   # 20 values read, 19 written per cell
    r["lbm_frac_of_hbm"] = round(156.0 * cells / (r["lbm_us"] * 1e-6) / 1e9 / hbm_gbs, 3)
    out["gemm4096x2048_lbm"] = r
    del lsrc, ldst

    nfft = 10240                          # FFT_B, src/header/fft_header.h:13
    fdata = torch.rand(nfft, 256, 2, device="cuda", generator=gen) * 2 - 1
    ff = lambda s=0, e=None: ops.gptb_fft(fdata.data_ptr(), nfft, start=s, end=e, grid=sms * 2, block=512)
    r = pair_report(ops, sms, t_of, tz, ff, nfft, "fft", (320, 576), tz_tiles=64 * 64)
    r["fft_gbs"] = round(4096.0 * nfft / r["fft_us"] / 1e3, 1)   # 2 KB in, 2 KB out per transform
    r["fft_gflops"] = round(5.0 * 256 * 8 * nfft / r["fft_us"] / 1e3, 1)
    out["gemm4096x2048_fft"] = r

    bins, nbr, cm = cutcp_problem(208, 208, 16)   # the reference's lattice, two slabs of regions in z
    dbins, dnbr = torch.from_numpy(bins).cuda(), torch.from_numpy(nbr).cuda()
    bdz, bdy, bdx = bins.shape[:3]
    zero = dbins.data_ptr() + 128 * ((cm * bdy + cm) * bdx + cm)
    regions = torch.zeros(2 * 26 * 26 * 512, device="cuda")
    inv = float(np.float32(1.0) / np.float32(144.0))
    cc = lambda s=0, e=None: ops.gptb_cutcp(bdx, bdy, zero, 0.5, 144.0, inv, regions.data_ptr(), dnbr.data_ptr(), nbr.shape[0],
                                            26, 26, 2, start=s, end=e, grid=sms * 2, block=512)
    r = pair_report(ops, sms, t_of, tz, cc, 26 * 26 * 2, "cutcp", (576, 832))
    count = (bins[..., 3] != 0).sum(axis=3).astype(np.int64)     # atoms per bin
    pairs = 0
    for dx, dy, dz, _ in nbr:                                     # every region's centre bin is the lattice bin (rx, ry, rz)
        pairs += int(count[cm + dz:cm + dz + 2, cm + dy:cm + dy + 26, cm + dx:cm + dx + 26].sum())
    r["cutcp_gpairs_per_s"] = round(512.0 * pairs / r["cutcp_us"] / 1e3, 1)   # (lattice point, atom) evaluations
    out["gemm4096x2048_cutcp"] = r
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-graph", action="store_true", help="launch the 10 kernels of a step one by one")
    ap.add_argument("--quick", action="store_true", help="skip the ratio sweep, the CPU sample and the reference kernels")
    ap.add_argument("--sustain-ms", type=float, default=400.0)
    ap.add_argument("--colocate-s", type=float, default=60.0, help="seconds of the LC/BE co-location run (0 = skip)")
    ap.add_argument("--only-pairs", action="store_true", help="run only the Coulomb and MRI-Q pairs and print them")
    ap.add_argument("--only-more", action="store_true", help="run only sgemm, lbm, fft and cutcp with their pairs and print them")
    ap.add_argument("--profile-gemm", default=None, help="MxNxK: time the solo tzgemm on that shape, launch it three more "
                                                         "times and exit")
    ap.add_argument("--gemm-pair", type=int, default=0, help="tzgemm_pair option of the --profile-gemm launches")
    ap.add_argument("--gemm-m256", type=int, default=0, help="tzgemm_m256 option of the --profile-gemm launches")
    ap.add_argument("--profile-pair", choices=("cp", "mriq"), default=None,
                    help="find that pair's balanced quantum, then launch its fused kernel three times and exit")
    ap.add_argument("--profile-w", type=int, default=832, help="CUDA-core threads of the --profile-pair launches")
    ap.add_argument("--profile-blocks", type=int, default=0,
                    help="CUDA-core blocks of the --profile-pair launches (0 = balance against the GEMM by measurement; "
                         "under a profiler that measurement is distorted, so pass the value a plain run found)")
    ap.add_argument("--fuse-sweeps", type=int, default=0, choices=(0, 1, 2, 10),
                    help="how many sweeps are fused with the GEMM (0 = time 10, 2 and 1 briefly and take the best)")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps == 40 and args.warmup == 5:
            args.steps, args.warmup = 10, 2
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
