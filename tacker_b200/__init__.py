"""tacker_b200: B200-native fused tensor-core / CUDA-core kernels behind a C ABI.

The product is the shared library ``lib/libtacker_b200.so`` (hand-written sm_100a CUDA, see
``include/tacker_b200.h``) and the C++ host in ``host/``.  This Python package only loads
the library and exposes its entry points to tests and to the benchmark; PyTorch is used by
callers for device memory and streams, never for the arithmetic.

There is no fallback path: importing works anywhere, but :func:`lib` raises if the shared
library has not been built, and every launcher returns ``TK_ERR_CUDA`` without a GPU.
"""
from __future__ import annotations

import ctypes as C
import os

from . import _build

__all__ = ["lib", "LIB_PATH", "TackerError", "check", "KEYS"]

LIB_PATH = _build.LIB_PATH
_lib = None

LAUNCH_FN = C.CFUNCTYPE(C.c_int, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_uint), C.POINTER(C.c_uint),
                        C.c_uint, C.c_void_p)

KEYS = ("gptb_tzgemm", "gptb_tzgemm_acc", "gptb_stencil", "gptb_cp", "gptb_mriq", "gptb_mrif", "tzgemm_stencil",
        "tzgemm_cp", "tzgemm_mriq", "tzgemm_mrif", "ori_stencil", "ori_cp", "ori_mriq", "ori_mrif", "gptb_tzconv",
        "tzconv_stencil", "tzconv_cp", "tzconv_mriq", "tzconv_mrif",
        "gptb_sgemm", "tzgemm_sgemm", "ori_sgemm", "gptb_lbm", "tzgemm_lbm", "ori_lbm",
        "gptb_fft", "tzgemm_fft", "ori_fft", "gptb_cutcp", "tzgemm_cutcp", "ori_cutcp",
        "tzconv_sgemm", "tzconv_lbm", "tzconv_fft", "tzconv_cutcp")


class TackerError(RuntimeError):
    def __init__(self, status: int, where: str = ""):
        self.status = status
        text = lib().tk_status_string(status).decode()
        detail = lib().tk_last_error().decode()
        super().__init__(f"{where}: {text} ({status})" + (f": {detail}" if detail else ""))


class KernelInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("threads_tensor", "threads_cd_min", "threads_cd_default",
                                       "regs_per_thread", "static_smem", "dynamic_smem", "tmem_columns",
                                       "max_ctas_per_sm", "nparams")]


def lib() -> C.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built: there is no substitute path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m tacker_b200._build` "
                "(needs nvcc; the kernels are sm_100a only and there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        l.tk_status_string.restype = C.c_char_p
        l.tk_last_error.restype = C.c_char_p
        l.tk_key.restype = C.c_char_p
        l.tk_lookup.restype = C.c_void_p
        l.tk_lookup.argtypes = [C.c_char_p]
        l.tk_query.argtypes = [C.c_char_p, C.POINTER(KernelInfo)]
        l.tk_set_option.argtypes = [C.c_char_p, C.c_int]
        l.tk_get_option.argtypes = [C.c_char_p, C.POINTER(C.c_int)]
        _lib = l
    return _lib


def check(status: int, where: str = "") -> None:
    if status != 0:
        raise TackerError(status, where)
