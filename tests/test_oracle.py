"""The CPU checker against independent numpy restatements and its own invariants (no GPU)."""
import numpy as np
import pytest

from helpers import coulomb_inputs, gemm_inputs, mriq_inputs, stencil_inputs


def test_f16_round_trip_matches_numpy(oracle):
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * 3,
        rng.standard_normal(2000).astype(np.float32) * 1e-5,      # half subnormals
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.9e-8, 3.1e-8, np.inf, -np.inf],
                 dtype=np.float32),
    ])
    bits = oracle.f32_to_f16_bits(x)
    want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(bits, want)
    back = oracle.f16_bits_to_f32(bits)
    assert np.array_equal(back.view(np.uint32), want.view(np.float16).astype(np.float32).view(np.uint32))


def test_rng_is_counter_based_and_in_range(oracle):
    a = oracle.uniform_f32(1000, 7, -1.0, 1.0)
    b = oracle.uniform_f32(500, 7, -1.0, 1.0)
    assert np.array_equal(a[:500], b)                     # element i does not depend on n
    assert a.min() >= -1.0 and a.max() < 1.0
    assert abs(float(a.mean())) < 0.1
    assert not np.array_equal(a, oracle.uniform_f32(1000, 8, -1.0, 1.0))
    bits, vals = oracle.uniform_f16(1000, 7, -1.0, 1.0)
    assert np.array_equal(bits.view(np.float16).astype(np.float32), vals)
    n = oracle.normal_f32(20000, 3)
    assert abs(float(n.mean())) < 0.05 and abs(float(n.std()) - 1.0) < 0.05


def test_tzgemm_dims_round_down_to_128(oracle):
    # src/tzgemm_kernel.h:30-48
    assert oracle.tzgemm_dims(1024, 1024, 1024) == (1024, 1024, 1024, 256)
    assert oracle.tzgemm_dims(50176, 64, 27) == (50176, 128, 128, 784 * 2)
    assert oracle.tzgemm_dims(1, 1000, 4096) == (128, 896, 4096, 2 * 14)
    assert oracle.tzgemm_dims(4096, 4096, 1024)[3] == 4096
    assert oracle.tzgemm_dims(2048, 2048, 2048)[3] == 1024


def test_tzgemm_matches_numpy_and_honours_tile_range(oracle):
    M, N, K = 128, 192, 128
    _, a, _, b = gemm_inputs(oracle, M, N, K)
    want = 1.1 * (a.astype(np.float64) @ b.astype(np.float64).T)
    got64 = oracle.tzgemm_f64(a, b, alpha=1.1)
    assert np.allclose(got64, want, rtol=1e-12, atol=1e-12)
    got32 = oracle.tzgemm_f32(a, b, alpha=1.1)
    assert np.abs(got32 - want).max() < 1e-4
    # tiles [2, 5) of a 2 x 3 tile grid: (0,2), (1,0), (1,1)
    part = oracle.tzgemm_f32(a, b, alpha=1.0, start=2, end=5, out=np.full((M, N), -7.0, dtype=np.float32))
    full = oracle.tzgemm_f32(a, b, alpha=1.0)
    mask = np.zeros((M, N), dtype=bool)
    mask[0:64, 128:192] = True
    mask[64:128, 0:128] = True
    assert np.array_equal(part[mask], full[mask])
    assert np.all(part[~mask] == -7.0)


def test_tzgemm_sampled_agrees_with_full(oracle):
    M, N, K = 128, 128, 256
    _, a, _, b = gemm_inputs(oracle, M, N, K, seed=3)
    rows = np.array([0, 5, 127, 64], dtype=np.int32)
    cols = np.array([0, 77, 127, 1], dtype=np.int32)
    val, mag = oracle.tzgemm_sampled(a, b, rows, cols, alpha=1.0)
    full = oracle.tzgemm_f64(a, b)
    assert np.allclose(val, full[rows, cols], rtol=1e-13)
    assert np.all(mag >= np.abs(val))


def _numpy_stencil(A0, c0, c1, out):
    s = (A0[2:, 1:-1, 1:-1] + A0[:-2, 1:-1, 1:-1])
    s = s + A0[1:-1, 2:, 1:-1]
    s = s + A0[1:-1, :-2, 1:-1]
    s = s + A0[1:-1, 1:-1, 2:]
    s = s + A0[1:-1, 1:-1, :-2]
    out[1:-1, 1:-1, 1:-1] = s * np.float32(c1) - A0[1:-1, 1:-1, 1:-1] * np.float32(c0)
    return out


@pytest.mark.parametrize("shape", [(8, 8, 70), (5, 9, 130), (3, 4, 64), (16, 12, 200)])
def test_stencil_sweep_matches_numpy_bitwise(oracle, shape):
    nz, ny, nx = shape
    A0 = stencil_inputs(oracle, nx, ny, nz)
    c0, c1 = np.float32(1 / 6), np.float32(1 / 36)
    want = _numpy_stencil(A0, c0, c1, A0.copy())
    got = oracle.stencil_sweep_f32(c0, c1, A0, A0.copy(), contract=0)
    assert oracle.bit_mismatches(got, want) == 0
    # the two FMA contractions stay within an ulp or two of the uncontracted form
    for mode in (1, 2):
        alt = oracle.stencil_sweep_f32(c0, c1, A0, A0.copy(), contract=mode)
        assert np.abs(alt - want).max() <= 2.4e-7
    # boundary cells are never written
    sentinel = np.full_like(A0, -9.0)
    got = oracle.stencil_sweep_f32(c0, c1, A0, sentinel)
    inner = np.zeros(A0.shape, dtype=bool)
    inner[1:-1, 1:-1, 1:-1] = True
    assert np.all(got[~inner] == -9.0) and np.all(got[inner] != -9.0)
    f64 = oracle.stencil_sweep_f64(c0, c1, A0)
    assert np.abs(f64[inner] - want[inner]).max() < 1e-6


def test_stencil_block_range_and_jacobi(oracle):
    nz, ny, nx = 6, 12, 192          # 3 x 3 virtual blocks
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=2)
    full = oracle.stencil_sweep_f32(0.5, 0.25, A0, A0.copy())
    parts = A0.copy()
    for s, e in ((0, 2), (2, 7), (7, 9)):
        oracle.stencil_sweep_f32(0.5, 0.25, A0, parts, start=s, end=e)
    assert oracle.bit_mismatches(parts, full) == 0
    one = oracle.stencil_sweep_f32(0.5, 0.25, A0, np.full_like(A0, 3.0), start=4, end=5)   # block (1,1)
    touched = one != 3.0
    assert touched[1:-1, 4:8, 64:128].all() and touched.sum() == (nz - 2) * 4 * 64
    # ping-pong: three sweeps == three manual sweeps with swapped roles
    a, b = A0.copy(), A0.copy()
    res = oracle.stencil_jacobi_f32(0.5, 0.25, a, b, 3)
    x, y = A0.copy(), A0.copy()
    for _ in range(3):
        _numpy_stencil(x, np.float32(0.5), np.float32(0.25), y)
        x, y = y, x
    assert oracle.bit_mismatches(res, x) == 0


def test_coulomb_matches_numpy(oracle):
    nx, ny, h, z = 128, 16, 0.125, 4.0
    atoms = coulomb_inputs(oracle, 150, 8.0, spacing=h, zplane=z)
    packed = oracle.cp_pack_atoms(atoms, z)
    assert np.array_equal(packed[:, 2], (np.float32(z) - atoms[:, 2]) ** 2)
    lat64, mag = oracle.cp_f64(packed, h, nx, ny)
    X = (np.float32(h) * np.arange(nx, dtype=np.float32)).astype(np.float64)
    Y = (np.float32(h) * np.arange(ny, dtype=np.float32)).astype(np.float64)
    want = np.zeros((ny, nx))
    for a in packed.astype(np.float64):
        want += a[3] / np.sqrt((X[None, :] - a[0]) ** 2 + (Y[:, None] - a[1]) ** 2 + a[2])
    assert np.allclose(lat64, want, rtol=1e-12, atol=1e-12)
    lat32 = oracle.cp_f32(packed, h, np.zeros((ny, nx), dtype=np.float32))
    assert oracle.max_scaled_err(lat32, lat64, mag) < 2e-6
    # accumulation (+=) and block ranges: two half-ranges on a pre-filled lattice == one full pass
    base = np.full((ny, nx), 2.0, dtype=np.float32)
    once = oracle.cp_f32(packed, h, base.copy())
    twice = base.copy()
    oracle.cp_f32(packed, h, twice, start=0, end=1)
    oracle.cp_f32(packed, h, twice, start=1, end=2)
    assert oracle.bit_mismatches(once, twice) == 0
    assert np.abs(once - 2.0 - lat32).max() < 1e-4


def test_mriq_matches_numpy(oracle):
    numK, numX = 96, 512
    k, phi, xyz = mriq_inputs(oracle, numK, numX)
    mag = oracle.mriq_phimag(phi[0], phi[1])
    assert np.allclose(mag, phi[0] ** 2 + phi[1] ** 2, rtol=3e-7)
    kv = oracle.mriq_pack(k[0], k[1], k[2], mag)
    qr64, qi64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2])
    arg = 2 * np.pi * (k.astype(np.float64).T @ xyz.astype(np.float64))      # [numK, numX]
    wr = (mag[:, None] * np.cos(arg)).sum(0)
    wi = (mag[:, None] * np.sin(arg)).sum(0)
    scale = float(mag.sum())
    # the oracle forms the phase in binary32 like the reference; that alone costs ~1e-5 rad per term
    assert np.abs(qr64 - wr).max() / scale < 2e-5 and np.abs(qi64 - wi).max() / scale < 2e-5
    qr, qi = oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(numX, np.float32), np.zeros(numX, np.float32))
    assert np.abs(qr - qr64).max() / scale < 1e-6 and np.abs(qi - qi64).max() / scale < 1e-6
    # accumulates onto the previous content, block ranges compose
    qr2 = np.ones(numX, np.float32)
    qi2 = np.ones(numX, np.float32)
    oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], qr2, qi2, start=0, end=1)
    oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], qr2, qi2, start=1, end=2)
    assert np.abs(qr2 - 1 - qr).max() < 1e-4


def test_im2col_and_conv_shape(oracle):
    rng = np.random.default_rng(5)
    im = rng.standard_normal((3, 9, 7)).astype(np.float32)
    col = oracle.im2col_f32(im, 3, 3, 1, 1, 2, 1)
    hcol, wcol = (9 + 2 - 3) // 2 + 1, (7 + 2 - 3) // 1 + 1
    pad = np.pad(im, ((0, 0), (1, 1), (1, 1)))
    want = np.empty((27, hcol * wcol), dtype=np.float32)
    for c in range(3):
        for i in range(3):
            for j in range(3):
                want[c * 9 + i * 3 + j] = pad[c, i:i + 2 * hcol:2, j:j + wcol].reshape(-1)
    assert np.array_equal(col, want)
    # VGG16 conv1_2 at batch 1: 224x224x64 -> M = 50176, N = 64, K = 576 (src/TaskManager.cu:92-123)
    assert oracle.conv_mnk([1, 64, 224, 224, 64, 64, 3, 3, 1, 1, 1, 1, 1, 1]) == (50176, 64, 576)
