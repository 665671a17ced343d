"""Pins the CPU restatements of sgemm, lbm, fft and cutcp against the reference itself (no GPU needed).

tests/golden/ref_{sgemm,lbm,fft,cutcp}*.npz hold outputs of the reference's own persistent-block kernels (compiled for
sm_100 from the reference tree by `make -C oracle ref`, run on a B200 by tests/golden/make_golden_more.py) on seeded
inputs; the inputs are regenerated here from the stored seeds.  sgemm is bit-exact; the other three differ from the
GPU in the rounding of cosf / sinf / rsqrt and in which multiply-adds the compiler fused, so they are held to a few
units in the last place of the largest value.
"""
import os
import sys

import numpy as np
import pytest

from helpers import cutcp_inputs, fft_inputs, lbm_inputs, sgemm_inputs

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GOLDEN)


def _load(name):
    g = np.load(os.path.join(GOLDEN, f"ref_{name}.npz"))
    return {k: (g[k] if g[k].ndim else g[k].item()) for k in g.files}


@pytest.mark.parametrize("name", ["sgemm", "sgemm_part"])
def test_sgemm_restatement_is_bit_exact(oracle, name):
    g = _load(name)
    a, b, c = sgemm_inputs(oracle, g["M"], g["N"], g["K"], seed=g["seed"])
    want = oracle.sgemm_f32(a, b, c.copy(), g["start"], g["end"])
    assert oracle.bit_mismatches(g["out"], want) == 0
    gx = g["M"] // 128
    touched = np.zeros((g["N"], g["M"]), bool)
    for p in range(g["start"], g["end"]):
        bx, by = p % gx, p // gx
        touched[by * 16:(by + 1) * 16, bx * 128:(bx + 1) * 128] = True
    assert np.array_equal(g["out"] != c, touched)          # blocks outside the range keep their C


@pytest.mark.parametrize("name", ["lbm", "lbm_part"])
def test_lbm_restatement(oracle, name):
    from make_golden_more import lbm_sample_index

    g = _load(name)
    nx, ny, nz = (int(v) for v in g["dims"])
    src, dst = lbm_inputs(oracle, nx, ny, nz, seed=g["seed"])
    want = oracle.lbm_f32(src, dst.copy(), nx, ny, nz, g["start"], g["end"])
    idx = lbm_sample_index(want.size, g["seed"])
    assert np.abs(want[idx] - g["sample"]).max() <= 2e-6     # values are O(1): a few ulp
    # the same cells are written: where the reference left the random fill, so does the restatement
    assert np.array_equal(want[idx] == dst[idx], g["sample"] == dst[idx])


@pytest.mark.parametrize("name", ["fft", "fft_part"])
def test_fft_restatement(oracle, name):
    g = _load(name)
    d = fft_inputs(oracle, g["nfft"], seed=g["seed"])
    want = oracle.fft256_f32(d.copy(), g["start"], g["end"])
    w64 = oracle.fft256_f64(d)
    scale = float(np.abs(w64).max())
    assert np.abs(want - g["out"]).max() <= 5e-7 * scale
    s, e = g["start"], g["end"]
    assert np.abs(g["out"][s:e] - w64[s:e]).max() <= 5e-7 * scale
    assert np.array_equal(g["out"][:s], d[:s]) and np.array_equal(g["out"][e:], d[e:])


@pytest.mark.parametrize("name", ["cutcp", "cutcp_256"])
def test_cutcp_restatement(oracle, name):
    g = _load(name)
    n, h, cutoff = g["n"], g["h"], g["cutoff"]
    atoms = cutcp_inputs(oracle, n, n, n, h, seed=g["seed"])
    dims = oracle.cutcp_bin_dims(n, n, n, h, cutoff)
    nbr = oracle.cutcp_neighbours(h, cutoff)
    assert nbr.shape[0] == 335                      # cutoff 12 A, bins of 4 A: the 7^3 cube without its 8 corners
    if g["nbrlen"]:
        nbr = nbr[:g["nbrlen"]]
    bins, _ = oracle.cutcp_bin_atoms(atoms, dims)
    r = (n + 7) // 8
    want = oracle.cutcp_f32(bins, dims, nbr, h, cutoff, np.zeros((r, r, r, 512), np.float32), r, r, r, g["start"], g["end"])
    scale = float(np.abs(g["out"]).max())
    assert scale > 0 and np.abs(want - g["out"]).max() <= 5e-7 * scale
    assert np.array_equal(want != 0, g["out"] != 0)
