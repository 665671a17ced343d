"""Per-GPU co-location across a node: one `aker --colocate` process per GPU, independent request streams,
no communication between them (co-location is per GPU); the result lines are summed here.

    python -m tacker_b200.colocate --gpus 8 --seconds 60 --qps 200 --qos 1.5 --lc vgg16 --be bert
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile

from . import _build

HOST = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host")


def run_fused(gpus: int, seconds: float, qps: float, qos: float, lc: str = "vgg16", be_kernel: str = "", devices=None) -> dict:
    """The co-location with a benchmark kernel as the best-effort job (`aker --colocate-fused`): time-sliced and fused
    phases under the same arrivals, one process per GPU; block rates are summed, latencies are the worst GPU's."""
    exe = os.path.join(_build.LIB_DIR, "aker")
    if not os.path.exists(exe):
        raise RuntimeError(f"{exe} is missing: build it with `python -m tacker_b200._build`")
    devices = list(range(gpus)) if devices is None else list(devices)
    workdir = tempfile.mkdtemp(prefix="aker_colocate_")
    procs = []
    for d in devices:
        cmd = [exe, "-s", "aker", "-m", lc, "-d", str(d), "-c", os.path.join(HOST, "config"), "--colocate-fused",
               str(seconds), "--qps", str(qps), "--qos", str(qos)] + (["--be-kernel", be_kernel] if be_kernel else [])
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=workdir))
    per_gpu = []
    for d, p in zip(devices, procs):
        out, err = p.communicate(timeout=seconds * 4 + 300)
        if p.returncode != 0:
            raise RuntimeError(f"aker on device {d} failed: {err[-500:]}")
        per_gpu.append(json.loads([l for l in out.splitlines() if l.startswith("{")][-1]))
    try:
        os.rmdir(workdir)
    except OSError:
        pass
    return {
        "gpus": len(devices), "lc": lc, "be_kernel": per_gpu[0]["be_kernel"], "seconds_per_phase": seconds,
        "qps_offered_per_gpu": qps, "fused_layers": per_gpu[0]["fused_layers"], "mixable_layers": per_gpu[0]["mixable_layers"],
        "blocks_per_fused_query": per_gpu[0]["blocks_per_fused_query"],
        "timesliced_be_blocks_per_s": sum(r["timesliced"]["be_blocks_per_s"] for r in per_gpu),
        "fused_be_blocks_per_s": sum(r["fused"]["be_blocks_per_s"] for r in per_gpu),
        "timesliced_lc_p99_ms_max": max(r["timesliced"]["lc_p99_ms"] for r in per_gpu),
        "fused_lc_p99_ms_max": max(r["fused"]["lc_p99_ms"] for r in per_gpu),
        "qos_bound_ms_min": min(r["qos_bound_ms"] for r in per_gpu),
        "qos_met_all": all(r["timesliced"]["qos_met"] and r["fused"]["qos_met"] for r in per_gpu),
        "per_gpu": per_gpu,
    }


def run(gpus: int, seconds: float, qps: float, qos: float, lc: str = "vgg16", be: str = "bert", devices=None) -> dict:
    exe = os.path.join(_build.LIB_DIR, "aker")
    if not os.path.exists(exe):
        raise RuntimeError(f"{exe} is missing: build it with `python -m tacker_b200._build`")
    devices = list(range(gpus)) if devices is None else list(devices)
    procs = []
    workdir = tempfile.mkdtemp(prefix="aker_colocate_")  # the children's working directory (they write nothing)
    for d in devices:
        cmd = [exe, "-s", "aker", "-m", lc, "-d", str(d), "-c", os.path.join(HOST, "config"), "--colocate",
               str(seconds), "--qps", str(qps), "--qos", str(qos), "--be", be]
        procs.append(subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, cwd=workdir))
    per_gpu = []
    for d, p in zip(devices, procs):
        out, err = p.communicate(timeout=seconds * 3 + 300)
        if p.returncode != 0:
            raise RuntimeError(f"aker on device {d} failed: {err[-500:]}")
        per_gpu.append(json.loads([l for l in out.splitlines() if l.startswith("{")][-1]))
    try:
        os.rmdir(workdir)
    except OSError:
        pass
    return {
        "gpus": len(devices), "lc": lc, "be": be, "qps_offered_per_gpu": qps, "seconds": seconds,
        "be_qps_total": sum(r["be_qps"] for r in per_gpu),
        "lc_p99_ms_max": max(r["lc_p99_ms"] for r in per_gpu),
        "lc_solo_p99_ms_max": max(r["lc_solo_p99_ms"] for r in per_gpu),
        "qos_met_all": all(r["qos_met"] for r in per_gpu),
        "per_gpu": per_gpu,
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--seconds", type=float, default=60.0)
    ap.add_argument("--qps", type=float, default=200.0)
    ap.add_argument("--qos", type=float, default=1.5)
    ap.add_argument("--lc", default="vgg16")
    ap.add_argument("--be", default="bert")
    ap.add_argument("--fused", action="store_true", help="best-effort job = the benchmark kernel of the model file, "
                                                         "time-sliced and fused (aker --colocate-fused)")
    a = ap.parse_args(argv)
    print(json.dumps(run_fused(a.gpus, a.seconds, a.qps, a.qos, a.lc) if a.fused else
                     run(a.gpus, a.seconds, a.qps, a.qos, a.lc, a.be)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
