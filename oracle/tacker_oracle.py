"""numpy/ctypes front end of the CPU checker (libtacker_oracle.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The product package never imports this module.

Every function is a thin wrapper over the C restatement in tacker_oracle.c,
where the reference kernel each one follows is cited.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtacker_oracle.so")
_lib = None

_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)
_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int32)


def build(force: bool = False) -> str:
    """Compile the C restatement with the system gcc (OpenMP, no FP contraction)."""
    src = os.path.join(_HERE, "tacker_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libtacker_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.tko_max_scaled_err.restype = C.c_double
        _lib.tko_count_bit_mismatch_f32.restype = C.c_int64
    return _lib


def _p(a: np.ndarray, ty):
    return a.ctypes.data_as(ty)


def _c32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def set_threads(n: int) -> int:
    return int(lib().tko_set_threads(C.c_int(n)))


def max_threads() -> int:
    return int(lib().tko_max_threads())


# ---------------------------------------------------------------- inputs ----
def uniform_f32(n: int, seed: int, lo: float, hi: float) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().tko_fill_uniform_f32(_p(out, _f32p), C.c_int64(n), C.c_uint64(seed), C.c_float(lo), C.c_float(hi))
    return out


def uniform_f16(n: int, seed: int, lo: float, hi: float):
    """Returns (binary16 bit patterns as uint16, the same values widened to float32)."""
    bits = np.empty(n, dtype=np.uint16)
    vals = np.empty(n, dtype=np.float32)
    lib().tko_fill_uniform_f16(_p(bits, _u16p), _p(vals, _f32p), C.c_int64(n), C.c_uint64(seed),
                               C.c_float(lo), C.c_float(hi))
    return bits, vals


def normal_f32(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().tko_fill_normal_f32(_p(out, _f32p), C.c_int64(n), C.c_uint64(seed), C.c_float(mean), C.c_float(std))
    return out


def f32_to_f16_bits(a) -> np.ndarray:
    a = _c32(a).ravel()
    out = np.empty(a.size, dtype=np.uint16)
    lib().tko_f32_to_f16(_p(a, _f32p), _p(out, _u16p), C.c_int64(a.size))
    return out


def f16_bits_to_f32(a) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.uint16).ravel()
    out = np.empty(a.size, dtype=np.float32)
    lib().tko_f16_to_f32(_p(a, _u16p), _p(out, _f32p), C.c_int64(a.size))
    return out


# ---------------------------------------------------------------- tzgemm ----
def tzgemm_dims(m: int, n: int, k: int):
    out = (C.c_int * 4)()
    lib().tko_tzgemm_dims(m, n, k, out)
    return tuple(out)


def tzgemm_f32(A, B, alpha=1.0, start=0, end=None, out=None) -> np.ndarray:
    """A [M,K], B [N,K] float32 holding binary16-representable values; C [M,N] float32.
    Only the 64x64 tiles with index in [start, end) are written."""
    A, B = _c32(A), _c32(B)
    M, K = A.shape
    N = B.shape[0]
    if end is None:
        end = (M // 64) * (N // 64)
    Cm = np.zeros((M, N), dtype=np.float32) if out is None else out
    lib().tko_tzgemm_f32(_p(A, _f32p), _p(B, _f32p), _p(Cm, _f32p), M, N, K, C.c_float(alpha), start, end)
    return Cm


def tzgemm_f64(A, B, alpha=1.0, start=0, end=None) -> np.ndarray:
    A, B = _c32(A), _c32(B)
    M, K = A.shape
    N = B.shape[0]
    if end is None:
        end = (M // 64) * (N // 64)
    Cm = np.zeros((M, N), dtype=np.float64)
    lib().tko_tzgemm_f64(_p(A, _f32p), _p(B, _f32p), _p(Cm, _f64p), M, N, K, C.c_double(alpha), start, end)
    return Cm


def tzgemm_sampled(A, B, rows, cols, alpha=1.0):
    """binary64 value and magnitude sum |a||b| at sampled (row, col) outputs."""
    A, B = _c32(A), _c32(B)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    cols = np.ascontiguousarray(cols, dtype=np.int32)
    val = np.empty(rows.size, dtype=np.float64)
    mag = np.empty(rows.size, dtype=np.float64)
    lib().tko_tzgemm_sampled(_p(A, _f32p), _p(B, _f32p), B.shape[0], A.shape[1], C.c_double(alpha),
                             _p(rows, _i32p), _p(cols, _i32p), C.c_int64(rows.size), _p(val, _f64p),
                             _p(mag, _f64p))
    return val, mag


# --------------------------------------------------------------- stencil ----
def stencil_grid(nx: int, ny: int):
    return (nx + 63) // 64, (ny + 3) // 4


def stencil_sweep_f32(c0, c1, A0, Anext, start=0, end=None, contract=0) -> np.ndarray:
    """A0, Anext: [nz, ny, nx] float32.  Anext is updated in place on the interior cells of
    virtual blocks [start, end) and returned."""
    nz, ny, nx = A0.shape
    gx, gy = stencil_grid(nx, ny)
    if end is None:
        end = gx * gy
    A0 = _c32(A0)
    assert Anext.dtype == np.float32 and Anext.flags.c_contiguous
    lib().tko_stencil_sweep_f32(C.c_float(c0), C.c_float(c1), _p(A0, _f32p), _p(Anext, _f32p), nx, ny, nz,
                                gx, gy, start, end, contract)
    return Anext


def stencil_sweep_f64(c0, c1, A0, boundary=None) -> np.ndarray:
    nz, ny, nx = A0.shape
    gx, gy = stencil_grid(nx, ny)
    A0 = _c32(A0)
    out = np.array(A0 if boundary is None else boundary, dtype=np.float64)
    lib().tko_stencil_sweep_f64(C.c_double(c0), C.c_double(c1), _p(A0, _f32p), _p(out, _f64p), nx, ny, nz,
                                gx, gy, 0, gx * gy)
    return out


def stencil_jacobi_f32(c0, c1, a, b, iters, contract=0) -> np.ndarray:
    """Ping-pong sweeps a->b->a...; returns the array holding the last sweep's result."""
    nz, ny, nx = a.shape
    assert a.dtype == np.float32 and b.dtype == np.float32
    lib().tko_stencil_jacobi_f32(C.c_float(c0), C.c_float(c1), _p(a, _f32p), _p(b, _f32p), nx, ny, nz, iters,
                                 contract)
    return b if iters % 2 == 1 else a


# --------------------------------------------------------------- coulomb ----
def cp_grid(nx: int, ny: int):
    return nx // 128, ny // 8


def cp_pack_atoms(atoms_xyzq, zplane: float) -> np.ndarray:
    atoms = _c32(atoms_xyzq).reshape(-1, 4)
    out = np.empty_like(atoms)
    lib().tko_cp_pack_atoms(_p(atoms, _f32p), atoms.shape[0], C.c_float(zplane), _p(out, _f32p))
    return out


def cp_f32(packed, spacing, lattice, start=0, end=None, chunk=64) -> np.ndarray:
    """lattice [ny, nx] float32 accumulated in place (+=)."""
    ny, nx = lattice.shape
    gx, gy = cp_grid(nx, ny)
    if end is None:
        end = gx * gy
    packed = _c32(packed)
    lib().tko_cp_f32(_p(packed, _f32p), packed.shape[0], C.c_float(spacing), _p(lattice, _f32p), gx, gy,
                     start, end, chunk)
    return lattice


def cp_f64(packed, spacing, nx, ny, start=0, end=None):
    gx, gy = cp_grid(nx, ny)
    if end is None:
        end = gx * gy
    packed = _c32(packed)
    lat = np.zeros((ny, nx), dtype=np.float64)
    mag = np.zeros((ny, nx), dtype=np.float64)
    lib().tko_cp_f64(_p(packed, _f32p), packed.shape[0], C.c_float(spacing), _p(lat, _f64p), _p(mag, _f64p),
                     gx, gy, start, end)
    return lat, mag


# ----------------------------------------------------------------- mri-q ----
def mriq_phimag(phiR, phiI, mode: int = 2) -> np.ndarray:
    phiR, phiI = _c32(phiR), _c32(phiI)
    out = np.empty_like(phiR)
    lib().tko_mriq_phimag_mode(_p(phiR, _f32p), _p(phiI, _f32p), _p(out, _f32p), phiR.size, mode)
    return out


def mriq_pack(kx, ky, kz, phiMag) -> np.ndarray:
    return np.ascontiguousarray(np.stack([_c32(kx), _c32(ky), _c32(kz), _c32(phiMag)], axis=1))


def mriq_f32(kvals, x, y, z, Qr, Qi, start=0, end=None):
    kvals, x, y, z = _c32(kvals), _c32(x), _c32(y), _c32(z)
    if end is None:
        end = x.size // 256
    lib().tko_mriq_f32(_p(kvals, _f32p), kvals.shape[0], _p(x, _f32p), _p(y, _f32p), _p(z, _f32p),
                       _p(Qr, _f32p), _p(Qi, _f32p), x.size // 256, start, end)
    return Qr, Qi


def mriq_f64(kvals, x, y, z, start=0, end=None):
    kvals, x, y, z = _c32(kvals), _c32(x), _c32(y), _c32(z)
    if end is None:
        end = x.size // 256
    Qr = np.zeros(x.size, dtype=np.float64)
    Qi = np.zeros(x.size, dtype=np.float64)
    lib().tko_mriq_f64(_p(kvals, _f32p), kvals.shape[0], _p(x, _f32p), _p(y, _f32p), _p(z, _f32p),
                       _p(Qr, _f64p), _p(Qi, _f64p), x.size // 256, start, end)
    return Qr, Qi


def mrif_pack(kx, ky, kz, phiR, phiI, dR, dI) -> np.ndarray:
    """The packed MRI-FHd table: numK x {Kx, Ky, Kz, RhoPhiR}, then numK x RhoPhiI (5 * numK floats)."""
    n = kx.size
    out = np.empty(5 * n, dtype=np.float32)
    lib().tko_mrif_pack(*[_p(_c32(v), _f32p) for v in (kx, ky, kz, phiR, phiI, dR, dI)], _p(out, _f32p), n)
    return out


def mrif_f32(kvals, x, y, z, outR, outI, start=0, end=None, mode: int = 0):
    gx = x.size // 256
    if end is None:
        end = gx
    kvals = _c32(kvals)
    lib().tko_mrif_f32(_p(kvals, _f32p), kvals.size // 5, _p(x, _f32p), _p(y, _f32p), _p(z, _f32p),
                       _p(outR, _f32p), _p(outI, _f32p), gx, start, end, mode)
    return outR, outI


def mrif_f64(kvals, x, y, z, start=0, end=None):
    gx = x.size // 256
    if end is None:
        end = gx
    kvals = _c32(kvals)
    o_r = np.zeros(x.size, dtype=np.float64)
    o_i = np.zeros(x.size, dtype=np.float64)
    lib().tko_mrif_f64(_p(kvals, _f32p), kvals.size // 5, _p(x, _f32p), _p(y, _f32p), _p(z, _f32p),
                       _p(o_r, _f64p), _p(o_i, _f64p), gx, start, end)
    return o_r, o_i


# ---------------------------------------------------------------- im2col ----
def conv_mnk(args14):
    a = (C.c_int * 14)(*[int(v) for v in args14])
    out = (C.c_int * 3)()
    lib().tko_conv_mnk(a, out)
    return tuple(out)


def im2col_f32(im, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h=1, dil_w=1) -> np.ndarray:
    im = _c32(im)
    c, h, w = im.shape
    hcol = (h + 2 * pad_h - (dil_h * (kh - 1) + 1)) // stride_h + 1
    wcol = (w + 2 * pad_w - (dil_w * (kw - 1) + 1)) // stride_w + 1
    col = np.empty((c * kh * kw, hcol * wcol), dtype=np.float32)
    lib().tko_im2col_f32(_p(im, _f32p), c, h, w, kh, kw, pad_h, pad_w, stride_h, stride_w, dil_h, dil_w,
                         _p(col, _f32p))
    return col


# ------------------------------------------------------------------ sgemm ----
def sgemm_grid(M: int, N: int):
    return M // 128, N // 16


def sgemm_f32(A_km, B_kn, C_nm, start=0, end=None) -> np.ndarray:
    """C = 2 C + 2 A B in place; A_km [K][M], B_kn [K][N], C_nm [N][M] (the reference's layouts)."""
    K, M = A_km.shape
    N = B_kn.shape[1]
    gx, gy = sgemm_grid(M, N)
    if end is None:
        end = gx * gy
    lib().tko_sgemm_f32(_p(_c32(A_km), _f32p), _p(_c32(B_kn), _f32p), _p(C_nm, _f32p), M, N, K, start, end)
    return C_nm


# -------------------------------------------------------------------- lbm ----
LBM_ENTRIES = 20


def lbm_margin(nx: int, ny: int) -> int:
    """floats in front of (and behind) the grid: two z-planes (src/header/lbm_header.h:246, REAL_MARGIN)"""
    return 2 * nx * ny


def lbm_f32(src_full, dst_full, nx, ny, nz, start=0, end=None, contract=1) -> np.ndarray:
    """One time step.  src_full / dst_full: flat arrays of margin + 20 nx ny nz + margin floats."""
    if end is None:
        end = ny * nz
    m = lbm_margin(nx, ny)
    assert src_full.size == dst_full.size == 2 * m + LBM_ENTRIES * nx * ny * nz and dst_full.dtype == np.float32
    src_full = _c32(src_full)
    lib().tko_lbm_f32(_p(src_full[m:], _f32p), _p(dst_full[m:], _f32p), nx, ny, nz, start, end, contract)
    return dst_full


# -------------------------------------------------------------------- fft ----
def fft256_f32(data, start=0, end=None, contract=1) -> np.ndarray:
    """data: [nfft][256][2] float32, transformed in place."""
    nfft = data.shape[0]
    if end is None:
        end = nfft
    assert data.dtype == np.float32 and data.flags.c_contiguous and data.shape[1:] == (256, 2)
    lib().tko_fft256_f32(_p(data, _f32p), nfft, start, end, contract)
    return data


def fft256_f64(data) -> np.ndarray:
    data = _c32(data)
    out = np.empty(data.shape, dtype=np.float64)
    lib().tko_fft256_f64(_p(data, _f32p), _p(out, _f64p), data.shape[0])
    return out


# ------------------------------------------------------------------ cutcp ----
def cutcp_neighbours(h: float, cutoff: float) -> np.ndarray:
    nbr = np.zeros((11 * 11 * 11, 3), dtype=np.int32)
    n = lib().tko_cutcp_neighbours(C.c_float(h), C.c_float(cutoff), _p(nbr, _i32p))
    return np.ascontiguousarray(nbr[:n])


def cutcp_bin_dims(nx, ny, nz, h, cutoff):
    out = (C.c_int * 4)()
    lib().tko_cutcp_bin_dims(nx, ny, nz, C.c_float(h), C.c_float(cutoff), out)
    return tuple(out)


def cutcp_bin_atoms(atoms_xyzq, dims):
    """bins [bz][by][bx][8][4] (margin bins included) and the number of atoms that found no room"""
    atoms_xyzq = _c32(atoms_xyzq)
    bins = np.zeros((dims[2], dims[1], dims[0], 8, 4), dtype=np.float32)
    extra = lib().tko_cutcp_bin_atoms(_p(atoms_xyzq, _f32p), atoms_xyzq.shape[0], (C.c_int * 4)(*dims), _p(bins, _f32p))
    return bins, int(extra)


def cutcp_f32(bins, dims, nbr, h, cutoff, regions, gx, gy, gz, start=0, end=None, contract=1) -> np.ndarray:
    """regions: [gz][gy][gx][512] float32, overwritten for the blocks of [start, end)"""
    if end is None:
        end = gx * gy * gz
    nbr = np.ascontiguousarray(nbr, dtype=np.int32)
    cutoff2 = np.float32(cutoff) * np.float32(cutoff)
    lib().tko_cutcp_f32(_p(_c32(bins), _f32p), (C.c_int * 4)(*dims), _p(nbr, _i32p), nbr.shape[0], C.c_float(h),
                        C.c_float(cutoff2), C.c_float(np.float32(1.0) / cutoff2), _p(regions, _f32p), gx, gy, gz, start, end,
                        contract)
    return regions


# ------------------------------------------------------------ comparisons ----
def bit_mismatches(a, b) -> int:
    a, b = _c32(a).ravel(), _c32(b).ravel()
    assert a.size == b.size
    return int(lib().tko_count_bit_mismatch_f32(_p(a, _f32p), _p(b, _f32p), C.c_int64(a.size)))


def max_scaled_err(got, want, scale=None, floor=1e-30) -> float:
    got = _c32(got).ravel()
    want = np.ascontiguousarray(want, dtype=np.float64).ravel()
    sp = None
    if scale is not None:
        scale = np.ascontiguousarray(scale, dtype=np.float64).ravel()
        sp = _p(scale, _f64p)
    return float(lib().tko_max_scaled_err(_p(got, _f32p), _p(want, _f64p), sp, C.c_double(floor),
                                          C.c_int64(got.size)))
