"""Pins the CPU checker against the reference itself (no GPU needed).

tests/golden/ref_*.npz hold outputs of the reference's own CUDA kernels (compiled for sm_100 from
the reference tree by `make -C oracle ref`, run on a B200 by tests/golden/make_golden.py) on seeded
inputs; the inputs are regenerated here from the stored seeds and pushed through the restatement.
"""
import os

import numpy as np
import pytest

from helpers import coulomb_inputs, gemm_inputs, mrif_inputs, mriq_inputs, stencil_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    g = np.load(os.path.join(GOLDEN, f"ref_{name}.npz"))
    return {k: (g[k] if g[k].ndim else g[k].item()) for k in g.files}


@pytest.mark.parametrize("name", ["stencil", "stencil_cfg2coef"])
def test_stencil_restatement_is_bit_exact(oracle, name):
    g = _load(name)
    A0 = stencil_inputs(oracle, g["nx"], g["ny"], g["nz"], seed=g["seed"])
    want = oracle.stencil_sweep_f32(np.float32(g["c0"]), np.float32(g["c1"]), A0, A0.copy(), contract=1)
    assert oracle.bit_mismatches(g["out"], want) == 0
    # the uncontracted form differs from the reference in the last place on some cells: contract=1 is
    # the reference's arithmetic, not an arbitrary choice
    other = oracle.stencil_sweep_f32(np.float32(g["c0"]), np.float32(g["c1"]), A0, A0.copy(), contract=0)
    assert oracle.bit_mismatches(g["out"], other) > 0
    f64 = oracle.stencil_sweep_f64(g["c0"], g["c1"], A0)
    assert np.abs(g["out"] - f64).max() <= 1e-5 * np.abs(f64).max()


@pytest.mark.parametrize("name", ["cp", "cp_cfg3spacing"])
def test_coulomb_restatement_is_bit_exact(oracle, name):
    g = _load(name)
    atoms = coulomb_inputs(oracle, g["natoms"], g["box"], seed=g["seed"], spacing=g["spacing"], zplane=g["zplane"])
    packed = oracle.cp_pack_atoms(atoms, g["zplane"])
    want = oracle.cp_f32(packed, g["spacing"], np.zeros((g["ny"], g["nx"]), np.float32), chunk=64)
    assert oracle.bit_mismatches(g["out"], want) == 0
    f64, mag = oracle.cp_f64(packed, g["spacing"], g["nx"], g["ny"])
    assert oracle.max_scaled_err(g["out"], f64, mag) <= 1e-5


def test_mriq_restatement_matches_to_sincos_rounding(oracle):
    """The reference calls cosf/sinf (<= 2 ulp); the restatement rounds binary64 cos/sin once.  With the
    same binary32 phase and the same fma accumulation the two stay within a few ulp of the sum."""
    g = _load("mriq")
    k, phi, xyz = mriq_inputs(oracle, g["numK"], g["numX"], seed=g["seed"])
    kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
    n = g["numX"]
    qr, qi = oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(n, np.float32), np.zeros(n, np.float32))
    peak = max(np.abs(g["qr"]).max(), np.abs(g["qi"]).max())
    assert np.abs(qr - g["qr"]).max() <= 4e-7 * peak and np.abs(qi - g["qi"]).max() <= 4e-7 * peak
    r64, i64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2])
    assert np.abs(g["qr"] - r64).max() <= 1e-5 * peak and np.abs(g["qi"] - i64).max() <= 1e-5 * peak


def test_mrif_restatement_matches_to_sincos_rounding(oracle):
    """MRI-FHd: the reference's g_general_ptb_mrif (300 samples: one full 256-entry constant tile and a ragged one)
    against the restatement with the contractions nvcc applies (mode 0); the other choice (mode 1) is further off."""
    g = _load("mrif")
    k, phi, d, xyz = mrif_inputs(oracle, g["numK"], g["numX"], seed=g["seed"])
    kv = oracle.mrif_pack(k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])
    n = g["numX"]
    err = {}
    for mode in (0, 1):
        o_r, o_i = oracle.mrif_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(n, np.float32), np.zeros(n, np.float32), mode=mode)
        err[mode] = max(np.abs(o_r - g["outR"]).max(), np.abs(o_i - g["outI"]).max())
    peak = max(np.abs(g["outR"]).max(), np.abs(g["outI"]).max())
    assert err[0] <= 4e-7 * peak and err[0] <= err[1]
    r64, i64 = oracle.mrif_f64(kv, xyz[0], xyz[1], xyz[2])
    assert np.abs(g["outR"] - r64).max() <= 1e-5 * peak and np.abs(g["outI"] - i64).max() <= 1e-5 * peak


def test_tzgemm_restatement_matches_reference_wmma(oracle):
    g = _load("tzgemm")
    _, a, _, b = gemm_inputs(oracle, g["M"], g["N"], g["K"], seed=g["seed"])
    assert abs(g["alpha"] - 1.1) < 1e-6                       # src/header/tzgemm_header.h:64
    want = oracle.tzgemm_f64(a, b, alpha=g["alpha"])
    mag = g["alpha"] * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T)
    assert (np.abs(g["out"] - want) / mag).max() <= 1e-3
    ref32 = oracle.tzgemm_f32(a, b, alpha=g["alpha"])
    assert np.abs(g["out"] - ref32).max() <= 1e-3 * mag.max()
