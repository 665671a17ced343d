#!/usr/bin/env python
"""Benchmark of the fused tensor-core / CUDA-core hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One "step" = one fused GEMM + stencil pair of the headline configuration: tzgemm
M = N = 4096, K = 1024 (fp16 in, fp32 out) together with 10 ping-pong Jacobi sweeps of the 7-point
stencil on a 512 x 512 x 64 fp32 grid, executed as 10 launches of the fused persistent kernel
(sweep i co-runs with the i-th tenth of the GEMM's 4096 tiles: 1 tensor tile per 2.5 CUDA-core
blocks).  The same work run unfused (1 tzgemm launch + 10 stencil launches) gives
`fused_vs_sequential`.  Multi-GPU = independent replicas, one process per GPU, no collective on
the data path (co-location is per GPU).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU restatement of the same pair on
the host cores instead (the reference project has no CPU implementation and its CUDA kernels are
timed separately, see `ref_gpu` in the default arm's line).
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
CD_THREADS = 384        # CUDA-core threads of the fused CTA (12 warps next to the 6 tensor-role warps)
SOLO_CD_THREADS = 256   # solo stencil: 2 CTAs of 8 warps per SM
TILES = (M // 64) * (N // 64)
CD_BLOCKS = (NX // 64) * (NY // 4)
WORKLOAD = (f"config 2: fused tzgemm {M}x{N}x{K} fp16->fp32 + {SWEEPS} Jacobi sweeps of the 7-point stencil on "
            f"{NX}x{NY}x{NZ} fp32 (c0=1/6, c1=-1/6, zero boundary), {SWEEPS} fused launches per pair")
METRIC = "fused GEMM+stencil pairs per second (fused vs sequential kernel time in fused_vs_sequential)"

# algorithmic bytes of one fused launch: one sweep (one fp32 read + one fp32 write per cell) plus
# one tenth of the GEMM's minimum traffic (A and B read once, C written once)
SWEEP_BYTES = 8 * NX * NY * NZ
GEMM_BYTES = 2 * (M * K + N * K) + 4 * M * N
LAUNCH_BYTES = SWEEP_BYTES + GEMM_BYTES / SWEEPS
# dram__bytes_read.sum + dram__bytes_write.sum of one fused launch, from the ncu capture
# summarised in profiles/mix_stencil_config2_ncu.md (None until a capture exists)
NCU_TRAFFIC_BYTES = None


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


def cpu_pair_sample(state, tile_frac=4, sweeps=5):
    """Times 1/tile_frac of the GEMM's tiles and `sweeps` of the 10 sweeps; returns seconds per full pair."""
    oracle, np, a, b, grid = state
    out = np.zeros((M, N), dtype=np.float32)
    x, y = grid.copy(), grid.copy()
    t0 = time.perf_counter()
    oracle.tzgemm_f32(a, b, alpha=1.0, start=0, end=TILES // tile_frac, out=out)
    t1 = time.perf_counter()
    oracle.stencil_jacobi_f32(np.float32(C0), np.float32(C1), x, y, sweeps, contract=1)
    t2 = time.perf_counter()
    return (t1 - t0) * tile_frac + (t2 - t1) * (SWEEPS / sweeps)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    state = cpu_pair_setup()
    oracle = state[0]
    cores = oracle.set_threads(os.cpu_count() or 1)
    for _ in range(args.warmup):
        cpu_pair_sample(state)
    t = [cpu_pair_sample(state) for _ in range(args.steps)]
    sec = sum(t) / len(t)
    sample = "per step: 1/4 of the GEMM's 64x64 tiles + 5 of the 10 sweeps, time scaled to the full pair"
    line = {
        "impl": "reference", "metric": METRIC, "value": 1.0 / sec, "unit": "pairs/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 inputs, f32 accumulate / f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "arm": "CPU restatement of the pair (the reference has no CPU code; "
                                                 "oracle/tacker_oracle.c, OpenMP, scalar binary32)"},
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

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels are sm_100a only and there is no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_

        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from tacker_b200 import ops

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sms = ops.sm_count()
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    A = (torch.rand(M, K, device="cuda", generator=gen) * 2 - 1).half()
    B = (torch.rand(N, K, device="cuda", generator=gen) * 2 - 1).half()
    Cm = torch.zeros(M, N, device="cuda")
    g0 = torch.rand(NZ, NY, NX, device="cuda", generator=gen)
    for sl in ((0,), (-1,), (slice(None), 0), (slice(None), -1), (slice(None), slice(None), 0),
               (slice(None), slice(None), -1)):
        g0[sl] = 0.0
    g1 = g0.clone()
    grids = (g0, g1)
    stream = torch.cuda.Stream()
    st = stream.cuda_stream

    def tz_kernel(start, end):
        return ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cm.data_ptr(), M, N, K, alpha=1.0, start=start, end=end,
                               grid=sms)

    def cd_kernel(it, start=0, end=None, grid=None):
        src, dst = grids[it & 1], grids[(it + 1) & 1]
        return ops.gptb_stencil(C0, C1, src.data_ptr(), dst.data_ptr(), NX, NY, NZ, start=start, end=end,
                                grid=grid or sms * 2, block=SOLO_CD_THREADS)

    bounds = [TILES * i // SWEEPS for i in range(SWEEPS + 1)]
    fused = [ops.mix(cd_kernel(i), tz_kernel(0, TILES), cd_threads=CD_THREADS, grid=sms,
                     tz_range=(bounds[i], bounds[i + 1])) for i in range(SWEEPS)]
    solo_tz = tz_kernel(0, TILES)
    solo_cd = [cd_kernel(i) for i in range(SWEEPS)]

    def fused_step():
        for k in fused:
            k.execute(st)

    def sequential_step():
        solo_tz.execute(st)
        for k in solo_cd:
            k.execute(st)

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
            barrier()
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps  # ms per step, max over ranks

    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()

    fused_fn = make_graph(fused_step)
    seq_fn = make_graph(sequential_step)
    warm = max(args.warmup, 3)

    sampler.active.set()
    ms_fused = timed(fused_fn, args.steps, warm)
    ms_seq = timed(seq_fn, args.steps, warm)
    # continuation of the same fused loop, only to give the 20 ms clock sampler enough samples
    t_end = time.time() + args.sustain_ms / 1e3
    with torch.cuda.stream(stream):
        while time.time() < t_end:
            for _ in range(50):
                fused_fn()
            stream.synchronize()
    sampler.active.clear()
    status = ops.device_status()

    # ---- solo kernels and the tile-ratio sweep (explain the headline; rank 0 prints) ----
    def t_of(kernels, reps=None):
        reps = reps or (2 if args.quick else 20)
        # `reps` back-to-back repetitions in one graph, so that launch overhead cannot starve the GPU
        def fn():
            for _ in range(reps):
                for k in kernels:
                    k.execute(st)
        return timed(make_graph(fn), 3, 2) / reps

    ms_gemm = t_of([solo_tz])
    ms_sweep = t_of(solo_cd) / SWEEPS
    sweep = []
    if not args.quick:
        for r in (1, 2, 3, 4, 5, 6, 7, 8):
            nt = CD_BLOCKS // r  # GEMM tiles co-run with one sweep's 1024 CUDA-core blocks: 1 : r
            f = t_of([ops.mix(cd_kernel(0), tz_kernel(0, TILES), cd_threads=CD_THREADS, grid=sms, tz_range=(0, nt))])
            s = t_of([tz_kernel(0, nt)]) + ms_sweep
            sweep.append({"tensor_to_cd_tiles": f"1:{r}", "gemm_tiles": nt, "cd_blocks": CD_BLOCKS,
                          "fused_us": round(f * 1e3, 2), "sequential_us": round(s * 1e3, 2), "ratio": round(f / s, 4)})
        # balanced point: as many GEMM tiles as take about one sweep's time
        nt = min(TILES, max(64, int(TILES * ms_sweep / ms_gemm)))
        f = t_of([ops.mix(cd_kernel(0), tz_kernel(0, TILES), cd_threads=CD_THREADS, grid=sms, tz_range=(0, nt))])
        s = t_of([tz_kernel(0, nt)]) + ms_sweep
        sweep.append({"tensor_to_cd_tiles": f"balanced {nt}:{CD_BLOCKS}", "gemm_tiles": nt, "cd_blocks": CD_BLOCKS,
                      "fused_us": round(f * 1e3, 2), "sequential_us": round(s * 1e3, 2), "ratio": round(f / s, 4)})

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

    e2e_steps = max(3, min(args.steps, 20))
    ms_e2e = timed(e2e_step, e2e_steps, 3)
    h2d = hA.numel() * 2 + hB.numel() * 2 + hA0.numel() * 4
    d2h = hC.numel() * 4 + hOut.numel() * 4
    clocks = sampler.stop()

    # ---- the reference's own fused kernel, recompiled for sm_100 (when the test build travelled) ----
    ref_gpu = None
    try:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import tacker_ref as ref

        if ref.available() and rank == 0 and not args.quick:
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

            if dist is None:
                rf, rs = timed(ref_fused, 10, 3), timed(ref_seq, 10, 3)
                ref_gpu = {"what": "reference wmma/GPTB kernels recompiled for sm_100, same pair, same GPU",
                           "fused_ms_per_pair": round(rf, 4), "sequential_ms_per_pair": round(rs, 4),
                           "fused_vs_sequential": round(rf / rs, 4)}
    except Exception as e:  # test infrastructure absent: not an error of the product
        ref_gpu = {"unavailable": repr(e)[:120]}

    cpu = None
    if rank == 0 and world == 1 and not args.quick:
        state = cpu_pair_setup()
        cores = state[0].set_threads(os.cpu_count() or 1)
        cpu_pair_sample(state)
        sec = min(cpu_pair_sample(state) for _ in range(2))
        cpu = {"value": 1.0 / sec, "unit": "pairs/s", "cores": cores, "kind": "port",
               "sample": "1/4 of the GEMM's tiles + 5 of the 10 sweeps, scaled to one pair; best of 2"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    hbm, tflops, which = measured_peaks()
    launch_s = ms_fused / SWEEPS / 1e3
    achieved = LAUNCH_BYTES / launch_s / 1e9
    line = {
        "metric": METRIC, "value": world * 1e3 / ms_fused, "unit": "pairs/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms_fused, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 inputs, f32 accumulate (tensor role) / f32 (CUDA-core role)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "cd_threads": CD_THREADS, "grid": sms, "replicas": world,
                   "l2": "inputs 80 MiB (GEMM) + 128 MiB (grids) exceed the 126 MB L2; no flush between steps",
                   "launch": "CUDA graph of the 10 fused launches" if not args.no_graph else "10 stream launches"},
        "fused_vs_sequential": ms_fused / ms_seq, "sequential_ms_per_step": ms_seq,
        "solo_us": {"tzgemm_4096x4096x1024": round(ms_gemm * 1e3, 2), "stencil_sweep": round(ms_sweep * 1e3, 2),
                    "tzgemm_tflops": round(2.0 * M * N * K / (ms_gemm * 1e-3) / 1e12, 1),
                    "stencil_gbs": round(SWEEP_BYTES / (ms_sweep * 1e-3) / 1e9, 1)},
        "ratio_sweep": sweep,
        "clocks": clocks,
        "e2e": {"value": world * 1e3 / ms_e2e, "unit": "pairs/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "steps": e2e_steps,
                "call": "tk_pair_tzgemm_stencil_host (pinned host buffers in and out)"},
        "gpu_launches": args.steps * SWEEPS,
        "roofline": {"kernel": "mix_stencil_kernel (fused tzgemm tiles + one stencil sweep)", "bound": "hbm",
                     "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                     "traffic": NCU_TRAFFIC_BYTES, "algorithmic_bytes_per_launch": LAUNCH_BYTES,
                     "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({which})",
                     "tensor_frac_solo_gemm": round(2.0 * M * N * K / (ms_gemm * 1e-3) / 1e12 / tflops, 4)},
        "cpu_baseline": cpu,
        "ref_gpu": ref_gpu,
        "device_status": status,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-graph", action="store_true", help="launch the 10 kernels of a step one by one")
    ap.add_argument("--quick", action="store_true", help="skip the ratio sweep, the CPU sample and the reference kernels")
    ap.add_argument("--sustain-ms", type=float, default=400.0)
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 10
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
