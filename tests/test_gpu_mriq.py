"""MRI-Q Fourier sum through the C ABI against the CPU checker (B200 only).

Tolerance 1e-5 relative, taken normwise (largest |Q| of the output) and against sum_k phiMag_k per
voxel; a voxel whose sum cancels has no meaningful element-wise relative error.
"""
import numpy as np
import pytest

from helpers import mriq_inputs, to_dev

pytestmark = pytest.mark.gpu


def _run(torch, ops, k, phi, xyz, qr0=None, qi0=None, start=0, end=None, grid=None, block=256):
    numK, numX = k.shape[1], xyz.shape[1]
    dk = [to_dev(torch, k[i]) for i in range(3)]
    dphi = [to_dev(torch, phi[i]) for i in range(2)]
    dx = [to_dev(torch, xyz[i]) for i in range(3)]
    kv = torch.empty((numK, 4), dtype=torch.float32, device="cuda")
    qr = to_dev(torch, np.zeros(numX, np.float32) if qr0 is None else qr0)
    qi = to_dev(torch, np.zeros(numX, np.float32) if qi0 is None else qi0)
    st = torch.cuda.current_stream().cuda_stream
    ops.mriq_pack_kvalues(dk[0].data_ptr(), dk[1].data_ptr(), dk[2].data_ptr(), dphi[0].data_ptr(),
                          dphi[1].data_ptr(), numK, kv.data_ptr(), st)
    ops.gptb_mriq(numK, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(),
                  kv.data_ptr(), numX, start=start, end=end, grid=grid, block=block).execute(st)
    torch.cuda.synchronize()
    return qr.cpu().numpy(), qi.cpu().numpy(), kv.cpu().numpy()


def _tol_check(oracle, got_r, got_i, kv, xyz, numX, start=0, end=None):
    r32 = np.zeros(numX, np.float32)
    i32 = np.zeros(numX, np.float32)
    oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], r32, i32, start=start, end=end)
    r64, i64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2], start=start, end=end)
    scale = float(kv[:, 3].sum())
    norm = max(np.abs(r64).max(), np.abs(i64).max())
    for got, w32, w64 in ((got_r, r32, r64), (got_i, i32, i64)):
        assert np.abs(got - w32).max() <= 1e-5 * norm
        assert np.abs(got - w64).max() <= 1e-5 * norm
        assert np.abs(got - w64).max() <= 1e-5 * scale


@pytest.mark.parametrize("accurate", [0, 1])
@pytest.mark.parametrize("numK", [1, 2, 63, 256, 1025])
def test_small_cases(cuda, oracle, accurate, numK):
    from tacker_b200 import ops

    numX = 1024
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=numK)
    ops.set_option("mriq_accurate", accurate)
    try:
        qr, qi, kv = _run(cuda, ops, k, phi, xyz, grid=3, block=96)
    finally:
        ops.set_option("mriq_accurate", 0)
    want_kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
    assert oracle.bit_mismatches(kv, want_kv) == 0
    _tol_check(oracle, qr, qi, kv, xyz, numX)


@pytest.mark.parametrize("split", [64, 100, 0, -1])
@pytest.mark.parametrize("numK", [1, 65, 256, 1025])
def test_sample_split_items(cuda, oracle, split, numK):
    """Work items that cover a range of the samples and add their partial sums to Q with reductions."""
    from tacker_b200 import ops

    numX = 1024
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=50 + numK)
    qr0 = oracle.uniform_f32(numX, 903, -2.0, 2.0)
    qi0 = oracle.uniform_f32(numX, 904, -2.0, 2.0)
    ops.set_option("mriq_split", split)
    try:
        qr, qi, kv = _run(cuda, ops, k, phi, xyz, qr0=qr0, qi0=qi0, start=1, end=3, grid=3, block=96)
    finally:
        ops.set_option("mriq_split", -1)
    outside = np.ones(numX, dtype=bool)
    outside[256:768] = False
    assert np.array_equal(qr[outside], qr0[outside]) and np.array_equal(qi[outside], qi0[outside])
    wr, wi = qr0.copy(), qi0.copy()
    oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], wr, wi, start=1, end=3)
    scale = float(kv[:, 3].sum()) + 2.0
    assert np.abs(qr - wr).max() <= 1e-5 * scale and np.abs(qi - wi).max() <= 1e-5 * scale


@pytest.mark.parametrize("rng", [(0, 1), (2, 3), (1, 4), (0, 4), (3, 3), (2, 9)])
def test_virtual_block_range_and_accumulate(cuda, oracle, rng):
    from tacker_b200 import ops

    numK, numX = 128, 1024
    start, end = rng
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=3)
    qr0 = oracle.uniform_f32(numX, 901, -2.0, 2.0)
    qi0 = oracle.uniform_f32(numX, 902, -2.0, 2.0)
    qr, qi, kv = _run(cuda, ops, k, phi, xyz, qr0=qr0, qi0=qi0, start=start, end=end, grid=2, block=64)
    lo, hi = start * 256, min(end, 4) * 256
    outside = np.ones(numX, dtype=bool)
    outside[lo:hi] = False
    assert np.array_equal(qr[outside], qr0[outside]) and np.array_equal(qi[outside], qi0[outside])
    wr, wi = qr0.copy(), qi0.copy()
    oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], wr, wi, start=start, end=min(end, 4))
    scale = float(kv[:, 3].sum())
    assert np.abs(qr - wr).max() <= 1e-5 * scale and np.abs(qi - wi).max() <= 1e-5 * scale


def test_config4_full_size(cuda, oracle):
    """2048 k-space samples, 262,144 voxels in [-32, 32)^3."""
    from tacker_b200 import ops

    numK, numX = 2048, 262144
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=0)
    qr, qi, kv = _run(cuda, ops, k, phi, xyz)
    # binary64 reference on 32 of the 1024 virtual blocks
    blocks = list(range(0, 1024, 33))
    scale = float(kv[:, 3].sum())
    worst, norm = 0.0, 0.0
    for p in blocks:
        r64, i64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2], start=p, end=p + 1)
        sl = slice(p * 256, p * 256 + 256)
        worst = max(worst, np.abs(qr[sl] - r64[sl]).max(), np.abs(qi[sl] - i64[sl]).max())
        norm = max(norm, np.abs(r64[sl]).max(), np.abs(i64[sl]).max())
    assert worst <= 1e-5 * norm and worst <= 1e-5 * scale
    # linearity in the sample set: first half + second half of the samples == all samples
    qa, ia, _ = _run(cuda, ops, k[:, :1024], phi[:, :1024], xyz)
    qb, ib, _ = _run(cuda, ops, k[:, 1024:], phi[:, 1024:], xyz)
    assert np.abs(qa + qb - qr).max() <= 1e-5 * norm and np.abs(ia + ib - qi).max() <= 1e-5 * norm
    assert np.isfinite(qr).all() and np.isfinite(qi).all()
