"""In-tree build of libtacker_b200.so (nvcc, sm_100a only) and of the `aker` host binary."""
from __future__ import annotations

import os
import shutil
import subprocess

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
HOST = os.path.join(ROOT, "host")
LIB_DIR = os.path.join(ROOT, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtacker_b200.so")
AKER_PATH = os.path.join(LIB_DIR, "aker")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libtacker_b200.so cannot be built on this machine")
    return exe


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(folder: str, exts):
    out = []
    for base, _dirs, files in os.walk(folder):
        out += [os.path.join(base, f) for f in files if f.endswith(exts)]
    return sorted(out)


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = _sources(CSRC, (".cu", ".cuh", ".h")) + [os.path.join(ROOT, "..", "include", "tacker_b200.h")]
    if not force and _newer(LIB_PATH, srcs):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    units = [s for s in srcs if s.endswith(".cu")]
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", LIB_PATH, *units]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return LIB_PATH


def build_host(force: bool = False) -> str | None:
    """The C++ host (operator surface, scheduler, `aker` CLI); links against the library."""
    if not os.path.isdir(HOST):
        return None
    srcs = _sources(HOST, (".cc", ".cpp", ".h", ".cu"))
    units = [s for s in srcs if s.endswith((".cc", ".cpp", ".cu"))]
    if not units:
        return None
    if not force and _newer(AKER_PATH, srcs + [LIB_PATH]):
        return AKER_PATH
    units = [u for u in units if os.sep + "tests" + os.sep not in u]
    cmd = [_nvcc(), "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(ROOT, "..", "include"), "-I", HOST, "-o", AKER_PATH, *units,
           "-L", LIB_DIR, "-ltacker_b200", "-ldl", "-Xlinker", "-rpath,$ORIGIN"]
    subprocess.check_call(cmd)
    return AKER_PATH


def build_host_selftest(force: bool = False) -> str:
    """Host runtime linked against a recording double of the library (no GPU, no CUDA): marshalling,
    registry, JSON, scheduling rules.  Test infrastructure."""
    out = os.path.join(LIB_DIR, "host_selftest")
    srcs = _sources(HOST, (".cc", ".h"))
    units = [s for s in srcs if s.endswith(".cc") and not s.endswith(("CudaBackend.cc", "main.cc"))]
    if not force and _newer(out, srcs):
        return out
    os.makedirs(LIB_DIR, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O1", "-g", "-std=c++17", "-Wall", "-I", os.path.join(ROOT, "..", "include"), "-I", HOST,
           "-o", out, *units, "-ldl"]
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
    print(build_host(force=True))
