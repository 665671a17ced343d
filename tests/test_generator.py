"""Fused-kernel generator: candidate enumeration and emission on the CPU, the emitted module on a GPU."""
import ctypes
import os

import pytest


def test_candidates_respect_the_sm_limits():
    from tacker_b200.fusion import data

    for cd in data.KERNELS:
        cands = data.fuse_kernel_info(cd)
        assert cands, cd
        for c in cands:
            assert c.r1 == 1 and c.threads == 192 + 32 * c.r2 <= data.MAX_THREADS_PER_CTA
            assert c.smem <= data.SMEM_PER_CTA and c.gemm.tmem <= data.TMEM_COLUMNS
            assert c.threads * max(data.TENSOR_ROLE_REGS, data.KERNELS[cd].regs) <= data.REGS_PER_SM
            assert c.name == f"tzgemm_{cd}_1_{c.r2}"
    # the stencil's rings compete with the GEMM stages for shared memory: the deepest pipeline leaves no room
    names = {(c.gemm.bn, c.gemm.stages, c.r2) for c in data.fuse_kernel_info("stencil")}
    assert (128, 4, 12) in names and (256, 3, 8) in names and (256, 3, 12) not in names and (256, 4, 24) not in names


def test_emitted_source_compiles_and_exports_its_launcher(tmp_path):
    from tacker_b200.fusion import data, gen_mix, gen_run

    c = [x for x in data.fuse_kernel_info("mriq") if x.r2 == 8][0]
    src = gen_mix.generate_mixed_kernel(c)
    assert "__launch_bounds__(448, 1)" in src and "mriq_role<false, 2>" in src and "gemm_role<256, 3>" in src
    cu = gen_run.emit(c, str(tmp_path))
    so = gen_run.compile_module(cu)
    mod = ctypes.CDLL(so)
    assert hasattr(mod, "tk_launch_tzgemm_mriq_1_8")
    info = (ctypes.c_int * 4)()
    mod.tk_generated_info_tzgemm_mriq_1_8(info)
    assert list(info) == [448, 256, 3, 8]


@pytest.mark.gpu
def test_generated_modules_match_the_solo_kernels(cuda, tmp_path):
    from tacker_b200.fusion import data, gen_run, gen_test

    for cd, w in (("stencil", 12), ("cp", 8), ("mriq", 16), ("mrif", 12), ("sgemm", 8), ("lbm", 12), ("fft", 8), ("cutcp", 16)):
        c = [x for x in data.fuse_kernel_info(cd) if x.r2 == w][0]
        so = gen_run.compile_module(gen_run.emit(c, str(tmp_path)))
        r = gen_test.check_module(so, c.name, cd)
        assert r["ok"], r
