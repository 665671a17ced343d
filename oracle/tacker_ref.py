"""ctypes front end of oracle/_ref/libtacker_ref.so: the reference's own CUDA kernels built for sm_100.

TEST INFRASTRUCTURE ONLY (see ref_shim.cu).  Needs a GPU; device buffers are raw addresses.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libtacker_ref.so")
_lib = None


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
    return _lib


def _vp(x):
    return C.c_void_p(int(x))


def _f32p(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def alpha() -> float:
    return lib().ref_alpha_times_1000() / 1000.0


def tzgemm(A, B, Cm, M, N, K, start, end, grid, stream=0) -> int:
    return lib().ref_tzgemm(_vp(A), _vp(B), _vp(Cm), M, N, K, start, end, grid, _vp(stream))


def stencil(c0, c1, A0, Anext, nx, ny, nz, start, end, grid, stream=0) -> int:
    return lib().ref_stencil(C.c_float(c0), C.c_float(c1), _vp(A0), _vp(Anext), nx, ny, nz, start, end, grid,
                             _vp(stream))


def cp(packed_host: np.ndarray, spacing, lattice, gx, gy, start, end, grid, stream=0) -> int:
    packed_host = np.ascontiguousarray(packed_host, dtype=np.float32)
    return lib().ref_cp(_f32p(packed_host), packed_host.shape[0], C.c_float(spacing), _vp(lattice), gx, gy, start,
                        end, grid, _vp(stream))


def mriq(kvals_host: np.ndarray, x, y, z, Qr, Qi, gx, start, end, grid, stream=0) -> int:
    kvals_host = np.ascontiguousarray(kvals_host, dtype=np.float32)
    return lib().ref_mriq(_f32p(kvals_host), kvals_host.shape[0], _vp(x), _vp(y), _vp(z), _vp(Qr), _vp(Qi), gx, start,
                          end, grid, _vp(stream))


def mix_stencil(c0, c1, A0, Anext, nx, ny, nz, cd_start, cd_end, A, B, Cm, M, N, K, tz_start, tz_end, grid,
                stream=0) -> int:
    return lib().ref_mix_stencil(C.c_float(c0), C.c_float(c1), _vp(A0), _vp(Anext), nx, ny, nz, cd_start, cd_end,
                                 _vp(A), _vp(B), _vp(Cm), M, N, K, tz_start, tz_end, grid, _vp(stream))


def cp_load_atoms(packed_host: np.ndarray) -> int:
    packed_host = np.ascontiguousarray(packed_host, dtype=np.float32)
    return lib().ref_cp_load_atoms(_f32p(packed_host), packed_host.shape[0])


def cp_launch(numatoms, spacing, lattice, gx, gy, start, end, grid, stream=0) -> int:
    return lib().ref_cp_launch(numatoms, C.c_float(spacing), _vp(lattice), gx, gy, start, end, grid, _vp(stream))


def mix_cp(numatoms, spacing, lattice, gx, gy, cd_start, cd_end, A, B, Cm, M, N, K, tz_start, tz_end, grid,
           stream=0) -> int:
    return lib().ref_mix_cp(numatoms, C.c_float(spacing), _vp(lattice), gx, gy, cd_start, cd_end, _vp(A), _vp(B),
                            _vp(Cm), M, N, K, tz_start, tz_end, grid, _vp(stream))


def mrif(kvals_aos_host: np.ndarray, x, y, z, outR, outI, gx, start, end, grid, stream=0) -> int:
    """kvals_aos_host: [numK][5] float32 = {Kx, Ky, Kz, RhoPhiR, RhoPhiI} (the reference's struct order)."""
    kvals_aos_host = np.ascontiguousarray(kvals_aos_host, dtype=np.float32)
    return lib().ref_mrif(_f32p(kvals_aos_host), kvals_aos_host.shape[0], _vp(x), _vp(y), _vp(z), _vp(outR), _vp(outI),
                          gx, start, end, grid, _vp(stream))


def mriq_load_kvals(kvals_host: np.ndarray) -> int:
    kvals_host = np.ascontiguousarray(kvals_host, dtype=np.float32)
    return lib().ref_mriq_load_kvals(_f32p(kvals_host), kvals_host.shape[0])


def mriq_launch(numK, x, y, z, Qr, Qi, gx, start, end, grid, stream=0) -> int:
    return lib().ref_mriq_launch(numK, _vp(x), _vp(y), _vp(z), _vp(Qr), _vp(Qi), gx, start, end, grid, _vp(stream))


def mix_mriq(numK, x, y, z, Qr, Qi, gx, cd_start, cd_end, A, B, Cm, M, N, K, tz_start, tz_end, grid, stream=0) -> int:
    return lib().ref_mix_mriq(numK, _vp(x), _vp(y), _vp(z), _vp(Qr), _vp(Qi), gx, cd_start, cd_end, _vp(A), _vp(B),
                              _vp(Cm), M, N, K, tz_start, tz_end, grid, _vp(stream))


# ---- sgemm, lbm, fft, cutcp (oracle/_ref/libtacker_ref_more.so) ----------------------------------------------
LIB_MORE_PATH = os.path.join(_HERE, "_ref", "libtacker_ref_more.so")
_lib_more = None


def more_available() -> bool:
    return os.path.exists(LIB_MORE_PATH)


def lib_more() -> C.CDLL:
    global _lib_more
    if _lib_more is None:
        _lib_more = C.CDLL(LIB_MORE_PATH)
    return _lib_more


def sgemm(A, B, Cm, M, N, K, start, end, grid, stream=0) -> int:
    return lib_more().ref_sgemm(_vp(A), _vp(B), _vp(Cm), M, N, K, start, end, grid, _vp(stream))


def lbm_dims():
    out = (C.c_int * 4)()
    lib_more().ref_lbm_dims(out)
    return tuple(out)


def lbm(src, dst, start, end, grid, stream=0) -> int:
    return lib_more().ref_lbm(_vp(src), _vp(dst), start, end, grid, _vp(stream))


def fft(data, nfft, start, end, grid, stream=0) -> int:
    return lib_more().ref_fft(_vp(data), nfft, start, end, grid, _vp(stream))


def cutcp_prepare(atoms_xyzq: np.ndarray, nx, ny, nz, h, cutoff, nbins_cap=65536):
    """The reference's own binning: (bins [nbins_cap][8][4] from the base address, neighbour offsets [1331][3], dims)."""
    atoms_xyzq = np.ascontiguousarray(atoms_xyzq, dtype=np.float32)
    bins = np.zeros((nbins_cap, 8, 4), dtype=np.float32)
    nbr = np.zeros((11 * 11 * 11, 3), dtype=np.int32)
    dims = (C.c_int * 5)()
    rc = lib_more().ref_cutcp_prepare(_f32p(atoms_xyzq), atoms_xyzq.shape[0], nx, ny, nz, C.c_float(h), C.c_float(cutoff),
                                      _f32p(bins), nbins_cap, nbr.ctypes.data_as(C.POINTER(C.c_int)), dims)
    assert rc == 0, rc
    return bins, nbr, tuple(dims)


def cutcp(nbr_host: np.ndarray, bx, by, c, bins_dev, h, cutoff2, inv_cutoff2, regions_dev, gx, gy, gz, start, end, grid,
          stream=0) -> int:
    nbr_host = np.ascontiguousarray(nbr_host, dtype=np.int32)
    return lib_more().ref_cutcp(nbr_host.ctypes.data_as(C.POINTER(C.c_int)), nbr_host.shape[0], bx, by, c, _vp(bins_dev),
                                C.c_float(h), C.c_float(cutoff2), C.c_float(inv_cutoff2), _vp(regions_dev), gx, gy, gz,
                                start, end, grid, _vp(stream))


# ---- the unfused ori_* kernels (oracle/_ref/libtacker_ref_ori.so) ----------------------------------------------
LIB_ORI_PATH = os.path.join(_HERE, "_ref", "libtacker_ref_ori.so")
_lib_ori = None


def ori_available() -> bool:
    return os.path.exists(LIB_ORI_PATH)


def lib_ori() -> C.CDLL:
    global _lib_ori
    if _lib_ori is None:
        _lib_ori = C.CDLL(LIB_ORI_PATH)
    return _lib_ori


def ori_stencil(c0, c1, A0, Anext, nx, ny, nz, stream=0) -> int:
    return lib_ori().ref_ori_stencil(C.c_float(c0), C.c_float(c1), _vp(A0), _vp(Anext), nx, ny, nz, _vp(stream))


def ori_cp(packed_host: np.ndarray, spacing, lattice, gx, gy, stream=0) -> int:
    packed_host = np.ascontiguousarray(packed_host, dtype=np.float32)
    return lib_ori().ref_ori_cp(_f32p(packed_host), packed_host.shape[0], C.c_float(spacing), _vp(lattice), gx, gy,
                                _vp(stream))


def ori_mriq(kvals_host: np.ndarray, x, y, z, Qr, Qi, numX, stream=0) -> int:
    kvals_host = np.ascontiguousarray(kvals_host, dtype=np.float32)
    return lib_ori().ref_ori_mriq(_f32p(kvals_host), kvals_host.shape[0], _vp(x), _vp(y), _vp(z), _vp(Qr), _vp(Qi), numX,
                                  _vp(stream))


def ori_mrif(kvals_aos_host: np.ndarray, x, y, z, outR, outI, numX, stream=0) -> int:
    kvals_aos_host = np.ascontiguousarray(kvals_aos_host, dtype=np.float32)
    return lib_ori().ref_ori_mrif(_f32p(kvals_aos_host), kvals_aos_host.shape[0], _vp(x), _vp(y), _vp(z), _vp(outR),
                                  _vp(outI), numX, _vp(stream))


def ori_sgemm(A, B, Cm, M, N, K, stream=0) -> int:
    return lib_ori().ref_ori_sgemm(_vp(A), _vp(B), _vp(Cm), M, N, K, _vp(stream))


def ori_lbm(src, dst, stream=0) -> int:
    return lib_ori().ref_ori_lbm(_vp(src), _vp(dst), _vp(stream))


def ori_fft(data, nfft, stream=0) -> int:
    return lib_ori().ref_ori_fft(_vp(data), nfft, _vp(stream))


def ori_cutcp(nbr_host: np.ndarray, bx, by, c, bins_dev, h, cutoff2, inv_cutoff2, regions_dev, gx, gy, gz, stream=0) -> int:
    nbr_host = np.ascontiguousarray(nbr_host, dtype=np.int32)
    return lib_ori().ref_ori_cutcp(nbr_host.ctypes.data_as(C.POINTER(C.c_int)), nbr_host.shape[0], bx, by, c,
                                   _vp(bins_dev), C.c_float(h), C.c_float(cutoff2), C.c_float(inv_cutoff2),
                                   _vp(regions_dev), gx, gy, gz, _vp(stream))
