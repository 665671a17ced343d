"""Driver of the fused-kernel generator (reference: fusion/code/gen_run.py:26-232): enumerate the candidates
of every (tzgemm, CUDA-core) pair under the SM's limits, emit the fused kernel, compile it into a loadable
module and -- when a GPU is present -- run the self-check with a time limit.

    python -m tacker_b200.fusion.gen_run [--out DIR] [--pairs stencil,cp,mriq] [--limit N] [--no-run]
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys

from .. import _build
from .data import KERNELS, fuse_kernel_info
from .gen_mix import generate_mixed_kernel

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_OUT = os.path.join(HERE, "mix_kernel")
RUN_TIMEOUT_S = 120  # the reference kills a generated binary after 5 s; a fresh CUDA context needs longer


def emit(candidate, out_dir: str) -> str:
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, candidate.name + ".cu")
    with open(path, "w") as f:
        f.write(generate_mixed_kernel(candidate))
    return path


def compile_module(cu_path: str) -> str:
    so = cu_path[:-3] + ".so"
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *_build.NVCC_FLAGS, "-shared", "-I", _build.CSRC, "-o", so, cu_path]
    subprocess.check_call(cmd)
    return so


def smoke(so: str, name: str, cd: str) -> dict:
    """Runs the self-check in a child process with a time limit (exact PID, never a pattern kill)."""
    code = ("import json,sys; from tacker_b200.fusion.gen_test import check_module; "
            f"print(json.dumps(check_module({so!r}, {name!r}, {cd!r})))")
    env = dict(os.environ, PYTHONPATH=os.path.dirname(os.path.dirname(HERE)))
    try:
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=RUN_TIMEOUT_S, env=env)
    except subprocess.TimeoutExpired:
        return {"name": name, "ok": False, "error": f"no answer within {RUN_TIMEOUT_S} s"}
    if out.returncode != 0:
        return {"name": name, "ok": False, "error": out.stderr[-500:]}
    return json.loads(out.stdout.strip().splitlines()[-1])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=DEFAULT_OUT)
    ap.add_argument("--pairs", default=",".join(KERNELS))
    ap.add_argument("--limit", type=int, default=0, help="at most N candidates per pair (0 = all)")
    ap.add_argument("--no-run", action="store_true")
    args = ap.parse_args(argv)
    _build.build_library()
    have_gpu = False
    if not args.no_run:
        try:
            import torch

            have_gpu = torch.cuda.is_available()
        except Exception:
            have_gpu = False
    report = []
    for cd in args.pairs.split(","):
        cands = fuse_kernel_info(cd)
        seen = set()
        cands = [c for c in cands if not (c.name in seen or seen.add(c.name))]  # one config per thread ratio
        if args.limit:
            cands = cands[:args.limit]
        for c in cands:
            cu = emit(c, args.out)
            so = compile_module(cu)
            entry = {"name": c.name, "threads": c.threads, "bn": c.gemm.bn, "stages": c.gemm.stages, "smem": c.smem,
                     "module": os.path.basename(so)}
            if have_gpu:
                entry.update(smoke(so, c.name, cd))
            report.append(entry)
            print(json.dumps(entry), flush=True)
    with open(os.path.join(args.out, "mix_kernel_info.json"), "w") as f:
        json.dump(report, f, indent=1)
    return 0 if all(e.get("ok", True) for e in report) else 1


if __name__ == "__main__":
    sys.exit(main())
