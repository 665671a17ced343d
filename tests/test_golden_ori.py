"""Pins the CPU checker against the reference's UNFUSED kernels (ori_stencil, ori_cp, ori_mriq, ori_mrif, ori_sgemm,
ori_lbm, ori_fft, ori_cutcp), the ones the outputs must match.  No GPU needed.

tests/golden/ref_ori.npz holds their outputs (compiled for sm_100 from the reference tree by `make -C oracle ref`, run
on a B200 by tests/golden/make_golden_ori.py) on the seeded whole-launch cases of the two other generators.  They are
bit-identical to the persistent-block forms pinned in ref_<name>.npz, so every check of test_golden.py and
test_golden_more.py holds for them too; the restatement is also recomputed here against them directly.
"""
import os

import numpy as np
import pytest

from helpers import coulomb_inputs, fft_inputs, sgemm_inputs, stencil_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ori():
    g = np.load(os.path.join(GOLDEN, "ref_ori.npz"))
    return {k: g[k] for k in g.files}


def _pinned(name):
    g = np.load(os.path.join(GOLDEN, f"ref_{name}.npz"))
    return {k: (g[k] if g[k].ndim else g[k].item()) for k in g.files}


@pytest.mark.parametrize("name,key,ori_key", [
    ("stencil", "out", "stencil"), ("stencil_cfg2coef", "out", "stencil_cfg2coef"), ("cp", "out", "cp"),
    ("cp_cfg3spacing", "out", "cp_cfg3spacing"), ("mriq", "qr", "mriq_qr"), ("mriq", "qi", "mriq_qi"),
    ("mrif", "outR", "mrif_r"), ("mrif", "outI", "mrif_i"), ("sgemm", "out", "sgemm"), ("fft", "out", "fft"),
    ("cutcp", "out", "cutcp"), ("lbm", "sample", "lbm_sample"), ("lbm", "digest", "lbm_digest")])
def test_unfused_kernels_equal_the_persistent_block_forms_bitwise(oracle, ori, name, key, ori_key):
    want, got = _pinned(name)[key], ori[ori_key]
    assert want.shape == got.shape
    if got.dtype == np.float32:
        assert oracle.bit_mismatches(got, want) == 0
    else:
        assert np.array_equal(got, want)


@pytest.mark.parametrize("name", ["stencil", "stencil_cfg2coef"])
def test_stencil_restatement_against_ori_stencil(oracle, ori, name):
    g = _pinned(name)
    A0 = stencil_inputs(oracle, g["nx"], g["ny"], g["nz"], seed=g["seed"])
    want = oracle.stencil_sweep_f32(np.float32(g["c0"]), np.float32(g["c1"]), A0, A0.copy(), contract=1)
    assert oracle.bit_mismatches(ori[name], want) == 0


@pytest.mark.parametrize("name", ["cp", "cp_cfg3spacing"])
def test_coulomb_restatement_against_ori_cp(oracle, ori, name):
    g = _pinned(name)
    atoms = coulomb_inputs(oracle, g["natoms"], g["box"], seed=g["seed"], spacing=g["spacing"], zplane=g["zplane"])
    packed = oracle.cp_pack_atoms(atoms, g["zplane"])
    want = oracle.cp_f32(packed, g["spacing"], np.zeros((g["ny"], g["nx"]), np.float32), chunk=64)
    assert oracle.bit_mismatches(ori[name], want) == 0


def test_sgemm_and_fft_restatements_against_ori_kernels(oracle, ori):
    g = _pinned("sgemm")
    a, b, cm = sgemm_inputs(oracle, g["M"], g["N"], g["K"], seed=g["seed"])
    assert oracle.bit_mismatches(ori["sgemm"], oracle.sgemm_f32(a, b, cm.copy(), g["start"], g["end"])) == 0
    g = _pinned("fft")
    d = fft_inputs(oracle, g["nfft"], seed=g["seed"])
    w64 = oracle.fft256_f64(d)
    assert np.abs(ori["fft"] - w64).max() <= 1e-5 * np.abs(w64).max()
