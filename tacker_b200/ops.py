"""Python mirror of the reference's operator surface over the C ABI.

Same roles and argument marshalling as the reference classes, so that a test or a benchmark
drives the kernels the way the reference runtime does:

  Kernel       src/Kernel.h:12-47         launchGridDim/launchBlockDim/kernelParams/smem
  GPTBKernel   src/GPTBKernel.h:12-124    solo kernel's params + 6 geometry ints, then at launch
                                          start, step, end, thread_base
  MixKernel    src/MixKernel.h:9-115      kernel1 params + {start, step, end} ++ kernel2 params +
                                          {start, step, end}; kernel1 = CUDA-core, kernel2 = tzgemm
                                          (src/TaskManager.cu:253-264)
  fmap         src/main.cu:108-159        key -> launcher (here: tk_lookup)

Device buffers are plain integers (device addresses, e.g. ``tensor.data_ptr()``); nothing in
this module allocates or touches device memory.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Sequence

from . import LAUNCH_FN, KernelInfo, TackerError, check, lib

def sm_count() -> int:
    n = C.c_int(0)
    check(lib().tk_sm_count(C.byref(n)), "tk_sm_count")
    return n.value


def set_option(name: str, value: int) -> None:
    check(lib().tk_set_option(name.encode(), int(value)), f"tk_set_option({name})")


def get_option(name: str) -> int:
    v = C.c_int(0)
    check(lib().tk_get_option(name.encode(), C.byref(v)), f"tk_get_option({name})")
    return v.value


def device_status() -> int:
    code = C.c_uint(0)
    check(lib().tk_device_status(C.byref(code)), "tk_device_status")
    return code.value


def query(key: str) -> KernelInfo:
    info = KernelInfo()
    check(lib().tk_query(key.encode(), C.byref(info)), f"tk_query({key})")
    return info


def lookup(key: str):
    """fmap[key]: returns a callable launcher or raises like the reference's `load kernel {key} failed`."""
    addr = lib().tk_lookup(key.encode())
    if not addr:
        raise KeyError(f"load kernel {{{key}}} failed!")
    return LAUNCH_FN(addr)


def _dim3(v) -> "C.Array":
    if isinstance(v, int):
        v = (v, 1, 1)
    v = tuple(v) + (1,) * (3 - len(v))
    return (C.c_uint * 3)(*v)


def raw_launch(key: str, params: Sequence, grid, block, smem: int = 0, stream: int = 0) -> int:
    """cudaLaunchKernel-shaped call: `params` are ctypes scalars, passed by address."""
    fn = lookup(key)
    arr = (C.c_void_p * len(params))(*[C.cast(C.pointer(p), C.c_void_p) for p in params])
    return fn(arr, len(params), _dim3(grid), _dim3(block), smem, C.c_void_p(stream))


class Kernel:
    """src/Kernel.h:12-47."""

    kernelName = ""
    funcKey = ""

    def __init__(self):
        self.kernelParams: List = []
        self.launchGridDim = (1, 1, 1)
        self.launchBlockDim = (1, 1, 1)
        self.smem = 0
        self.mixable = 0

    def execute(self, stream: int = 0) -> None:
        check(raw_launch(self.funcKey, self.kernelParams, self.launchGridDim, self.launchBlockDim, self.smem,
                         stream), self.funcKey)

    def getArgs(self) -> List[int]:
        return []


def tzgemm_dims(m: int, n: int, k: int):
    """getTZGEMMGridDim, src/tzgemm_kernel.h:30-48."""
    out = (C.c_int * 4)()
    check(lib().tk_tzgemm_dims(m, n, k, out), "tk_tzgemm_dims")
    return tuple(out)


class OriTZGEMMKernel(Kernel):
    """src/tzgemm_kernel.h:56-147; buffers are the caller's (the reference uses global scratch)."""

    kernelName = "tzgemm"
    funcKey = "gptb_tzgemm"

    def __init__(self, A: int, B: int, Cm: int, m: int, n: int, k: int, alpha: float = 1.1,
                 round_dims: bool = True):
        super().__init__()
        if round_dims:   # the reference always rounds (initParams, src/tzgemm_kernel.h:79-86)
            self.M_GLOBAL, self.N_GLOBAL, self.K_GLOBAL, self.ori_blks = tzgemm_dims(m, n, k)
        else:            # the kernel itself also takes N and K in multiples of 64
            self.M_GLOBAL, self.N_GLOBAL, self.K_GLOBAL, self.ori_blks = m, n, k, (m // 64) * (n // 64)
        self.kernelParams = [C.c_void_p(A), C.c_void_p(B), C.c_void_p(Cm), C.c_int(self.M_GLOBAL),
                             C.c_int(self.N_GLOBAL), C.c_int(self.K_GLOBAL), C.c_float(alpha)]
        self.launchGridDim = (self.ori_blks, 1, 1)
        self.launchBlockDim = (192, 1, 1)


class OriTZCONVKernel(Kernel):
    """Implicit-GEMM 3 x 3 convolution (stride 1, padding 1) on bordered NHWC fp16 images; the launch goes through
    GPTBKernel("tzconv", "gptb_tzconv", ...)."""

    kernelName = "tzconv"
    funcKey = "gptb_tzconv"

    def __init__(self, X: int, Wt: int, Y: int, H: int, W: int, Cin: int, Cout: int, bias: int = 0, act: int = 1,
                 alpha: float = 1.0):
        super().__init__()
        self.M_GLOBAL = ((H * (W + 2) + 127) // 128) * 128
        self.N_GLOBAL, self.K_GLOBAL = Cout, 9 * Cin
        self.ori_blks = (self.M_GLOBAL // 64) * (Cout // 64)
        self.kernelParams = [C.c_void_p(X), C.c_void_p(Wt), C.c_void_p(Y), C.c_int(self.M_GLOBAL), C.c_int(Cout),
                             C.c_int(9 * Cin), C.c_float(alpha), C.c_void_p(bias), C.c_int(H), C.c_int(W), C.c_int(Cin),
                             C.c_int(act)]
        self.launchGridDim = (self.ori_blks, 1, 1)
        self.launchBlockDim = (192, 1, 1)


class OriSTENCILKernel(Kernel):
    """src/ori_kernel/stencil_kernel.cu:114-204 (launch geometry :173-178)."""

    kernelName = "stencil"
    funcKey = "ori_stencil"

    def __init__(self, c0: float, c1: float, A0: int, Anext: int, nx: int, ny: int, nz: int):
        super().__init__()
        self.kernelParams = [C.c_float(c0), C.c_float(c1), C.c_void_p(A0), C.c_void_p(Anext), C.c_int(nx),
                             C.c_int(ny), C.c_int(nz)]
        self.launchGridDim = ((nx + 63) // 64, (ny + 3) // 4, 1)
        self.launchBlockDim = (32, 4, 1)


class OriCPKernel(Kernel):
    """src/ori_kernel/cp_kernel.cu:271-340; `atoms` = packed {x, y, dz^2, q} device array."""

    kernelName = "cp"
    funcKey = "ori_cp"

    def __init__(self, numatoms: int, gridspacing: float, energygrid: int, atoms: int, nx: int, ny: int):
        super().__init__()
        self.kernelParams = [C.c_int(numatoms), C.c_float(gridspacing), C.c_void_p(energygrid), C.c_void_p(atoms)]
        self.launchGridDim = (nx // 128, ny // 8, 1)
        self.launchBlockDim = (16, 8, 1)


class OriMRIQKernel(Kernel):
    """src/ori_kernel/mriq_kernel.cu:107-330; `kvals` = packed {Kx, Ky, Kz, PhiMag} device array."""

    kernelName = "mriq"
    funcKey = "ori_mriq"

    def __init__(self, numK: int, x: int, y: int, z: int, Qr: int, Qi: int, kvals: int, numX: int):
        super().__init__()
        self.kernelParams = [C.c_int(numK), C.c_int(0), C.c_void_p(x), C.c_void_p(y), C.c_void_p(z),
                             C.c_void_p(Qr), C.c_void_p(Qi), C.c_void_p(kvals)]
        self.launchGridDim = (numX // 256, 1, 1)
        self.launchBlockDim = (256, 1, 1)


class OriMRIFKernel(Kernel):
    """src/ori_kernel/mrif_kernel.cu:78-150; `kvals` = the packed table of mrif_pack_kvalues (5 * numK floats)."""

    kernelName = "mrif"
    funcKey = "ori_mrif"

    def __init__(self, numK: int, x: int, y: int, z: int, outR: int, outI: int, kvals: int, numX: int):
        super().__init__()
        self.kernelParams = [C.c_int(numK), C.c_int(0), C.c_void_p(x), C.c_void_p(y), C.c_void_p(z),
                             C.c_void_p(outR), C.c_void_p(outI), C.c_void_p(kvals)]
        self.launchGridDim = (numX // 256, 1, 1)
        self.launchBlockDim = (256, 1, 1)


class OriSGEMMKernel(Kernel):
    """src/ori_kernel/sgemm_kernel.cu:9-150: C = 2 C + 2 A B; A [K][M], B [K][N], C [N][M]."""

    kernelName = "sgemm"
    funcKey = "ori_sgemm"

    def __init__(self, A: int, B: int, Cm: int, M: int, N: int, K: int):
        super().__init__()
        self.kernelParams = [C.c_void_p(A), C.c_void_p(B), C.c_void_p(Cm), C.c_int(M), C.c_int(N), C.c_int(K)]
        self.launchGridDim = (M // 128, N // 16, 1)
        self.launchBlockDim = (16, 8, 1)


class OriLBMKernel(Kernel):
    """src/ori_kernel/lbm_kernel.cu:9-225: one time step; src / dst address cell (0, 0, 0) of element 0."""

    kernelName = "lbm"
    funcKey = "ori_lbm"

    def __init__(self, src: int, dst: int, nx: int, ny: int, nz: int):
        super().__init__()
        self.kernelParams = [C.c_void_p(src), C.c_void_p(dst)]
        self.launchGridDim = (ny, nz, 1)
        self.launchBlockDim = (nx, 1, 1)


class OriFFTKernel(Kernel):
    """src/ori_kernel/fft_kernel.cu:40-125: `nfft` transforms of 256 complex points, in place."""

    kernelName = "fft"
    funcKey = "ori_fft"

    def __init__(self, data: int, nfft: int):
        super().__init__()
        self.kernelParams = [C.c_void_p(data)]
        self.launchGridDim = (nfft, 1, 1)
        self.launchBlockDim = (128, 1, 1)


class OriCUTCPKernel(Kernel):
    """src/ori_kernel/cutcp_kernel.cu:19-330; `nbr` = the table of cutcp_pack_neighbours, `bins_zero` the bin at the
    lattice origin, `regions` gx * gy * gz regions of 512 floats."""

    kernelName = "cutcp"
    funcKey = "ori_cutcp"

    def __init__(self, binDim_x: int, binDim_y: int, bins_zero: int, h: float, cutoff2: float, inv_cutoff2: float,
                 regions: int, nbr: int, nbrlen: int, gx: int, gy: int, gz: int):
        super().__init__()
        self.kernelParams = [C.c_int(binDim_x), C.c_int(binDim_y), C.c_void_p(bins_zero), C.c_float(h),
                             C.c_float(cutoff2), C.c_float(inv_cutoff2), C.c_void_p(regions), C.c_int(gz - 1),
                             C.c_void_p(nbr), C.c_int(nbrlen)]
        self.launchGridDim = (gx, gy, gz)
        self.launchBlockDim = (8, 2, 8)


class GPTBKernel(Kernel):
    """src/GPTBKernel.h:12-124."""

    def __init__(self, kernelName: str, funcKey: str, kernel: Kernel, gridDim, blockDim, ptb_start_block_pos: int,
                 ptb_end_block_pos: int):
        super().__init__()
        lookup(funcKey)  # loadKernel(): fail at construction like the reference
        self.kernelName = kernelName
        self.funcKey = funcKey
        self.kernel_ = kernel
        self.launchGridDim = tuple(_dim3(gridDim))
        self.launchBlockDim = tuple(_dim3(blockDim))
        g, b = _dim3(kernel.launchGridDim), _dim3(kernel.launchBlockDim)
        self.gptbParams = dict(grid=(g[0], g[1], g[2]), block=(b[0], b[1], b[2]))
        self.ptb_start_block_pos = ptb_start_block_pos
        self.ptb_end_block_pos = ptb_end_block_pos
        self.smem = kernel.smem
        self.kernelParams = list(kernel.kernelParams) + [C.c_int(v) for v in (g[0], g[1], g[2], b[0], b[1], b[2])]

    @property
    def ptb_iter_block_step(self) -> int:
        g = self.launchGridDim
        return g[0] * g[1] * g[2]

    def execute(self, stream: int = 0) -> None:
        tail = [C.c_int(self.ptb_start_block_pos), C.c_int(self.ptb_iter_block_step),
                C.c_int(self.ptb_end_block_pos), C.c_int(0)]
        check(raw_launch(self.funcKey, self.kernelParams + tail, self.launchGridDim, self.launchBlockDim,
                         self.smem, stream), self.funcKey)


class MixKernel(Kernel):
    """src/MixKernel.h:9-115."""

    def __init__(self, funcKey: str, kernel1: GPTBKernel, kernel2: GPTBKernel, gridDim, blockDim,
                 ptb_start_block_pos1: int, ptb_end_block_pos1: int, ptb_start_block_pos2: int,
                 ptb_end_block_pos2: int):
        super().__init__()
        lookup(funcKey)
        self.kernelName = funcKey
        self.funcKey = funcKey
        self.launchGridDim = tuple(_dim3(gridDim))
        self.launchBlockDim = tuple(_dim3(blockDim))
        step = self.launchGridDim[0] * self.launchGridDim[1] * self.launchGridDim[2]
        self.kernelParams = (list(kernel1.kernelParams) +
                             [C.c_int(ptb_start_block_pos1), C.c_int(step), C.c_int(ptb_end_block_pos1)] +
                             list(kernel2.kernelParams) +
                             [C.c_int(ptb_start_block_pos2), C.c_int(step), C.c_int(ptb_end_block_pos2)])


# ---- input preparation -------------------------------------------------------------------------
def cp_pack_atoms(atoms_xyzq: int, count: int, zplane: float, packed: int, stream: int = 0) -> None:
    check(lib().tk_cp_pack_atoms(C.c_void_p(atoms_xyzq), count, C.c_float(zplane), C.c_void_p(packed),
                                 C.c_void_p(stream)), "tk_cp_pack_atoms")


def mriq_pack_kvalues(kx: int, ky: int, kz: int, phiR: int, phiI: int, numK: int, kvals: int,
                      stream: int = 0) -> None:
    check(lib().tk_mriq_pack_kvalues(C.c_void_p(kx), C.c_void_p(ky), C.c_void_p(kz), C.c_void_p(phiR),
                                     C.c_void_p(phiI), numK, C.c_void_p(kvals), C.c_void_p(stream)),
          "tk_mriq_pack_kvalues")


def mrif_pack_kvalues(kx: int, ky: int, kz: int, phiR: int, phiI: int, dR: int, dI: int, numK: int, kvals: int,
                      stream: int = 0) -> None:
    check(lib().tk_mrif_pack_kvalues(*[C.c_void_p(p) for p in (kx, ky, kz, phiR, phiI, dR, dI)], numK,
                                     C.c_void_p(kvals), C.c_void_p(stream)), "tk_mrif_pack_kvalues")


def im2col_f32(data_im: int, channels: int, height: int, width: int, kh: int, kw: int, pad_h: int, pad_w: int,
               stride_h: int, stride_w: int, dil_h: int, dil_w: int, data_col: int, stream: int = 0) -> None:
    check(lib().tk_im2col_f32(C.c_void_p(data_im), channels, height, width, kh, kw, pad_h, pad_w, stride_h,
                              stride_w, dil_h, dil_w, C.c_void_p(data_col), C.c_void_p(stream)), "tk_im2col_f32")


def convert_fp32_to_fp16(out_half: int, inp: int, n: int, stream: int = 0) -> None:
    check(lib().tk_convert_fp32_to_fp16(C.c_void_p(out_half), C.c_void_p(inp), C.c_longlong(n),
                                        C.c_void_p(stream)), "tk_convert_fp32_to_fp16")


def conv_mnk(args14):
    a = (C.c_int * 14)(*[int(v) for v in args14])
    out = (C.c_int * 3)()
    check(lib().tk_conv_mnk(a, out), "tk_conv_mnk")
    return tuple(out)


# ---- convenience constructors used by tests and the benchmark -------------------------------------
def gptb_tzgemm(A, B, Cm, m, n, k, alpha=1.1, start=0, end=None, grid=None, round_dims=True) -> GPTBKernel:
    ori = OriTZGEMMKernel(A, B, Cm, m, n, k, alpha, round_dims)
    return GPTBKernel("tzgemm", "gptb_tzgemm", ori, (grid or sm_count(), 1, 1), (192, 1, 1), start,
                      ori.ori_blks if end is None else end)


def gptb_tzconv(X, Wt, Y, H, W, Cin, Cout, bias=0, act=1, start=0, end=None, grid=None) -> GPTBKernel:
    ori = OriTZCONVKernel(X, Wt, Y, H, W, Cin, Cout, bias, act)
    return GPTBKernel("tzconv", "gptb_tzconv", ori, (grid or sm_count(), 1, 1), (192, 1, 1), start,
                      ori.ori_blks if end is None else end)


def gptb_stencil(c0, c1, A0, Anext, nx, ny, nz, start=0, end=None, grid=None, block=256) -> GPTBKernel:
    ori = OriSTENCILKernel(c0, c1, A0, Anext, nx, ny, nz)
    total = ori.launchGridDim[0] * ori.launchGridDim[1]
    return GPTBKernel("stencil", "gptb_stencil", ori, (grid or sm_count() * 2, 1, 1), (block, 1, 1), start,
                      total if end is None else end)


def gptb_cp(numatoms, spacing, energygrid, atoms, nx, ny, start=0, end=None, grid=None, block=256) -> GPTBKernel:
    ori = OriCPKernel(numatoms, spacing, energygrid, atoms, nx, ny)
    total = ori.launchGridDim[0] * ori.launchGridDim[1]
    return GPTBKernel("cp", "gptb_cp", ori, (grid or sm_count() * 2, 1, 1), (block, 1, 1), start,
                      total if end is None else end)


def gptb_mriq(numK, x, y, z, Qr, Qi, kvals, numX, start=0, end=None, grid=None, block=256) -> GPTBKernel:
    ori = OriMRIQKernel(numK, x, y, z, Qr, Qi, kvals, numX)
    return GPTBKernel("mriq", "gptb_mriq", ori, (grid or sm_count() * 4, 1, 1), (block, 1, 1), start,
                      ori.launchGridDim[0] if end is None else end)


def gptb_mrif(numK, x, y, z, outR, outI, kvals, numX, start=0, end=None, grid=None, block=256) -> GPTBKernel:
    ori = OriMRIFKernel(numK, x, y, z, outR, outI, kvals, numX)
    return GPTBKernel("mrif", "gptb_mrif", ori, (grid or sm_count() * 2, 1, 1), (block, 1, 1), start,
                      ori.launchGridDim[0] if end is None else end)


def _gptb_of(name: str, ori: Kernel, start, end, grid, block) -> GPTBKernel:
    g = ori.launchGridDim
    return GPTBKernel(name, "gptb_" + name, ori, (grid or sm_count() * 2, 1, 1), (block, 1, 1), start,
                      g[0] * g[1] * g[2] if end is None else end)


def gptb_sgemm(A, B, Cm, M, N, K, start=0, end=None, grid=None, block=512) -> GPTBKernel:
    return _gptb_of("sgemm", OriSGEMMKernel(A, B, Cm, M, N, K), start, end, grid or sm_count(), block)


def gptb_lbm(src, dst, nx, ny, nz, start=0, end=None, grid=None, block=512) -> GPTBKernel:
    return _gptb_of("lbm", OriLBMKernel(src, dst, nx, ny, nz), start, end, grid, block)


def gptb_fft(data, nfft, start=0, end=None, grid=None, block=512) -> GPTBKernel:
    return _gptb_of("fft", OriFFTKernel(data, nfft), start, end, grid, block)


def gptb_cutcp(binDim_x, binDim_y, bins_zero, h, cutoff2, inv_cutoff2, regions, nbr, nbrlen, gx, gy, gz, start=0,
               end=None, grid=None, block=512) -> GPTBKernel:
    ori = OriCUTCPKernel(binDim_x, binDim_y, bins_zero, h, cutoff2, inv_cutoff2, regions, nbr, nbrlen, gx, gy, gz)
    return _gptb_of("cutcp", ori, start, end, grid, block)


def cutcp_pack_neighbours(nbr_xyz, n, table, stream: int = 0) -> None:
    check(lib().tk_cutcp_pack_neighbours(C.c_void_p(nbr_xyz), n, C.c_void_p(table), C.c_void_p(stream)),
          "tk_cutcp_pack_neighbours")


def mix(cd: GPTBKernel, tz: GPTBKernel, cd_threads=256, grid=None, cd_range=None, tz_range=None) -> MixKernel:
    """tzgemm_<cd> fused kernel as TaskManager builds it (src/TaskManager.cu:253-264)."""
    cs, ce = cd_range if cd_range is not None else (cd.ptb_start_block_pos, cd.ptb_end_block_pos)
    ts, te = tz_range if tz_range is not None else (tz.ptb_start_block_pos, tz.ptb_end_block_pos)
    return MixKernel(tz.kernelName + "_" + cd.kernelName, cd, tz, (grid or sm_count(), 1, 1), (192 + cd_threads, 1, 1),
                     cs, ce, ts, te)


# ---- whole operators and the host-buffer pair ---------------------------------------------------------
def mriq_compute(kx, ky, kz, phiR, phiI, numK, x, y, z, Qr, Qi, numX, kvals_scratch, stream: int = 0) -> None:
    check(lib().tk_mriq_compute(*[C.c_void_p(p) for p in (kx, ky, kz, phiR, phiI)], numK,
                                *[C.c_void_p(p) for p in (x, y, z, Qr, Qi)], numX, C.c_void_p(kvals_scratch),
                                C.c_void_p(stream)), "tk_mriq_compute")


def mriq_compute_static(kx, ky, kz, phiR, phiI, numK, x, y, z, Qr, Qi, numX, stream: int = 0) -> None:
    """MRI-Q with the library's fixed k-space table instead of caller scratch (no allocation anywhere)."""
    check(lib().tk_mriq_compute_static(*[C.c_void_p(p) for p in (kx, ky, kz, phiR, phiI)], numK,
                                       *[C.c_void_p(p) for p in (x, y, z, Qr, Qi)], numX, C.c_void_p(stream)),
          "tk_mriq_compute_static")


def coulomb_compute(atoms_xyzq, numatoms, zplane, spacing, energygrid, nx, ny, packed_scratch,
                    stream: int = 0) -> None:
    check(lib().tk_coulomb_compute(C.c_void_p(atoms_xyzq), numatoms, C.c_float(zplane), C.c_float(spacing),
                                   C.c_void_p(energygrid), nx, ny, C.c_void_p(packed_scratch), C.c_void_p(stream)),
          "tk_coulomb_compute")


def pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz) -> int:
    n = C.c_size_t(0)
    check(lib().tk_pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz, C.byref(n)), "tk_pair_tzgemm_stencil_workspace")
    return n.value


def pair_tzgemm_stencil_host(A_host, B_host, C_host, M, N, K, alpha, c0, c1, A0_host, Aout_host, nx, ny, nz, sweeps,
                             cd_threads, workspace, workspace_bytes, stream: int = 0) -> None:
    """All five buffers are host addresses (pinned); `workspace` is a device address."""
    check(lib().tk_pair_tzgemm_stencil_host(C.c_void_p(A_host), C.c_void_p(B_host), C.c_void_p(C_host), M, N, K,
                                            C.c_float(alpha), C.c_float(c0), C.c_float(c1), C.c_void_p(A0_host),
                                            C.c_void_p(Aout_host), nx, ny, nz, sweeps, cd_threads,
                                            C.c_void_p(workspace), C.c_size_t(workspace_bytes), C.c_void_p(stream)),
          "tk_pair_tzgemm_stencil_host")


# ---- layer kernels of the DNN tasks -----------------------------------------------------------------------
def _vp(x):
    return C.c_void_p(int(x) if x else 0)


def im2col_nhwc_f16(x, H, W, Cin, kh, kw, pad, stride, A_half, M_pad, K_pad, stream: int = 0) -> None:
    check(lib().tk_im2col_nhwc_f16(_vp(x), H, W, Cin, kh, kw, pad, stride, _vp(A_half), M_pad, K_pad, _vp(stream)),
          "tk_im2col_nhwc_f16")


def bias_act_f16_bordered(x, ldx, bias, out_half, H, W, Cn, act, stream: int = 0) -> None:
    check(lib().tk_bias_act_f16_bordered(_vp(x), ldx, _vp(bias), _vp(out_half), H, W, Cn, act, _vp(stream)),
          "tk_bias_act_f16_bordered")


def maxpool2x2_f16_bordered(x_half, H, W, Cn, out_half, stream: int = 0) -> None:
    check(lib().tk_maxpool2x2_f16_bordered(_vp(x_half), H, W, Cn, _vp(out_half), _vp(stream)), "tk_maxpool2x2_f16_bordered")


def unborder_f16(x_half, H, W, Cn, row_half, stream: int = 0) -> None:
    check(lib().tk_unborder_f16(_vp(x_half), H, W, Cn, _vp(row_half), _vp(stream)), "tk_unborder_f16")


def rows_f32_to_f16(x, rows, cols, ld_in, A_half, rows_pad, cols_pad, stream: int = 0) -> None:
    check(lib().tk_rows_f32_to_f16(_vp(x), rows, cols, ld_in, _vp(A_half), rows_pad, cols_pad, _vp(stream)),
          "tk_rows_f32_to_f16")


def bias_act_f32(x, ldx, bias, out, rows, cols, ld_out, act, stream: int = 0) -> None:
    check(lib().tk_bias_act_f32(_vp(x), ldx, _vp(bias), _vp(out), rows, cols, ld_out, act, _vp(stream)),
          "tk_bias_act_f32")


def maxpool2x2_nhwc_f32(x, H, W, Cn, out, stream: int = 0) -> None:
    check(lib().tk_maxpool2x2_nhwc_f32(_vp(x), H, W, Cn, _vp(out), _vp(stream)), "tk_maxpool2x2_nhwc_f32")


def add_f32(a, b, out, n, stream: int = 0) -> None:
    check(lib().tk_add_f32(_vp(a), _vp(b), _vp(out), C.c_longlong(n), _vp(stream)), "tk_add_f32")


def softmax_rows_f32(x, out, rows, cols, scale=1.0, stream: int = 0) -> None:
    check(lib().tk_softmax_rows_f32(_vp(x), _vp(out), C.c_longlong(rows), cols, C.c_float(scale), _vp(stream)),
          "tk_softmax_rows_f32")


def layernorm_rows_f32(x, gamma, beta, out, rows, cols, eps=1e-12, stream: int = 0) -> None:
    check(lib().tk_layernorm_rows_f32(_vp(x), _vp(gamma), _vp(beta), _vp(out), C.c_longlong(rows), cols,
                                      C.c_float(eps), _vp(stream)), "tk_layernorm_rows_f32")


def add_layernorm_rows_f32(a, b, gamma, beta, out, rows, cols, eps=1e-12, stream: int = 0, out_half=0, bias=0) -> None:
    check(lib().tk_add_layernorm_rows_f32(_vp(a), _vp(bias), _vp(b), _vp(gamma), _vp(beta), _vp(out), _vp(out_half),
                                          C.c_longlong(rows), cols, C.c_float(eps), _vp(stream)),
          "tk_add_layernorm_rows_f32")


def bias_act_f32_f16(x, ldx, bias, out, ld_out, out_half, ld_half, rows, cols, act, stream: int = 0) -> None:
    check(lib().tk_bias_act_f32_f16(_vp(x), ldx, _vp(bias), _vp(out), ld_out, _vp(out_half), ld_half, rows, cols, act,
                                    _vp(stream)), "tk_bias_act_f32_f16")


def softmax_rows_f16(x, out_half, rows, cols, scale, stream: int = 0) -> None:
    check(lib().tk_softmax_rows_f16(_vp(x), _vp(out_half), C.c_longlong(rows), cols, C.c_float(scale), _vp(stream)),
          "tk_softmax_rows_f16")


def merge_heads_f16(ctx, B, S, heads, dh, out_half, stream: int = 0) -> None:
    check(lib().tk_merge_heads_f16(_vp(ctx), B, S, heads, dh, _vp(out_half), _vp(stream)), "tk_merge_heads_f16")


def split_qkv_heads_f16(x, ld, B, S, heads, dh, q_half, k_half, vt_half, stream: int = 0, bias=0) -> None:
    check(lib().tk_split_qkv_heads_f16(_vp(x), _vp(bias), ld, B, S, heads, dh, _vp(q_half), _vp(k_half), _vp(vt_half),
                                       _vp(stream)),
          "tk_split_qkv_heads_f16")


def split_heads_f16(x, ld, col0, B, S, heads, dh, transpose, out_half, stream: int = 0) -> None:
    check(lib().tk_split_heads_f16(_vp(x), ld, col0, B, S, heads, dh, transpose, _vp(out_half), _vp(stream)),
          "tk_split_heads_f16")


def merge_heads_f32(ctx, B, S, heads, dh, out, stream: int = 0) -> None:
    check(lib().tk_merge_heads_f32(_vp(ctx), B, S, heads, dh, _vp(out), _vp(stream)), "tk_merge_heads_f32")


def tzgemm_batched(A, B, Cm, M, N, K, batch, alpha=1.0, stride_a=0, stride_b=0, stride_c=0, stream: int = 0) -> None:
    check(lib().tk_tzgemm_batched(_vp(A), _vp(B), _vp(Cm), M, N, K, batch, C.c_longlong(stride_a),
                                  C.c_longlong(stride_b), C.c_longlong(stride_c), C.c_float(alpha), _vp(stream)),
          "tk_tzgemm_batched")


__all__ = [n for n in dir() if not n.startswith("_")]
