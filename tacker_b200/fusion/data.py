"""Resource model and candidate enumeration (reference: fusion/code/data.py:22-69).

The reference enumerates (CTAs per SM, r1, r2) such that r1 + r2 role copies of two GPTB kernels fit an
sm_75 SM: threads <= 1024, registers <= 65536, shared memory <= 65536.  On B200 the tensor role is fixed
(one copy: 6 warps, the whole tensor memory, 147-197 KB of shared memory), exactly one CTA fits an SM, and the
free variable is the number of CUDA-core warps next to it -- the "r2" of the pair name tzgemm_<cd>_1_<r2>.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

# B200 (sm_100) per-SM limits
MAX_THREADS_PER_CTA = 1024
REGS_PER_SM = 65536
SMEM_PER_CTA = 232448          # 227 KiB opt-in maximum
TMEM_COLUMNS = 512
TENSOR_ROLE_THREADS = 192      # TMA producer, MMA issuer, 4 epilogue warps
TENSOR_ROLE_REGS = 64          # epilogue: 32 accumulator registers + addressing


@dataclass(frozen=True)
class KernelInfo:
    """Per-thread registers, shared memory per warp (bytes) and thread granularity of a CUDA-core role
    (the reference's table: fusion/code/data.py:25-35, from `nvcc --ptxas-options=-v`)."""
    name: str
    regs: int
    smem_per_warp: int
    granule: int               # threads
    bound: str


# registers from `nvcc -Xptxas -v` on the role kernels of this repository (sm_100a)
KERNELS = {
    "stencil": KernelInfo("stencil", 64, 3 * 1792 + 128, 32, "hbm"),       # >= 3 ring slots per warp
    "cp": KernelInfo("cp", 32, 0, 32, "sfu"),
    "mriq": KernelInfo("mriq", 32, 0, 32, "sfu"),
    "mrif": KernelInfo("mrif", 32, 0, 32, "sfu"),
    "sgemm": KernelInfo("sgemm", 96, 3 * 2560, 32, "fma"),                  # a ring of three slots per warp
    "lbm": KernelInfo("lbm", 64, 0, 32, "hbm"),
    "fft": KernelInfo("fft", 64, 2048 + 128, 32, "latency"),                # 2 KB per warp + its share of the 2 KB tables
    "cutcp": KernelInfo("cutcp", 64, 0, 32, "issue"),
}


@dataclass(frozen=True)
class GemmConfig:
    bn: int
    stages: int

    @property
    def smem(self) -> int:
        stage = 128 * 64 * 2 + self.bn * 64 * 2
        pipeline = self.stages * stage + (2 * self.stages + 4) * 8 + 8
        staging = 4 * 32 * 36 * 4            # epilogue transpose buffers of the four epilogue warps
        return (pipeline + 127) // 128 * 128 + staging + 1024

    @property
    def tmem(self) -> int:
        return 2 * self.bn


@dataclass(frozen=True)
class Candidate:
    pair: str
    cd: str
    r1: int                    # tensor role copies (always 1 on B200: it owns the tensor memory)
    r2: int                    # CUDA-core warps
    gemm: GemmConfig
    threads: int
    regs_per_thread: int
    smem: int

    @property
    def name(self) -> str:
        return f"tzgemm_{self.cd}_{self.r1}_{self.r2}"


def fuse_kernel_info(cd: str, gemm_configs=(GemmConfig(256, 3), GemmConfig(256, 4), GemmConfig(128, 4),
                                            GemmConfig(128, 6)), warp_choices=(4, 8, 12, 16, 20, 24)
                     ) -> List[Candidate]:
    """All (tensor role, W CUDA-core warps) combinations that fit one CTA on one SM."""
    k = KERNELS[cd]
    out = []
    for g in gemm_configs:
        if g.tmem > TMEM_COLUMNS:
            continue
        for w in warp_choices:
            threads = TENSOR_ROLE_THREADS + 32 * w
            if threads > MAX_THREADS_PER_CTA:
                continue
            regs = max(TENSOR_ROLE_REGS, k.regs)
            if threads * regs > REGS_PER_SM:
                continue
            smem = g.smem + w * k.smem_per_warp
            if smem > SMEM_PER_CTA:
                continue
            out.append(Candidate(f"tzgemm_{cd}", cd, 1, w, g, threads, REGS_PER_SM // threads // 8 * 8, smem))
    return out
