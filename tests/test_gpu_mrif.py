"""MRI-FHd through the C ABI against the CPU checker (B200 only).

Tolerance 1e-5 relative, taken against the largest |out| and against sum_k (|RhoPhiR_k| + |RhoPhiI_k|) per voxel
(a voxel whose sum cancels has no meaningful element-wise relative error).  The accurate mode repeats the
reference's arithmetic (binary64 product for the phase, cosf / sinf) and is held to the rounding of those two
functions; the default mode reduces the phase exactly and uses the hardware sin / cos.
"""
import numpy as np
import pytest

from helpers import mrif_inputs, to_dev

pytestmark = pytest.mark.gpu


def _run(torch, ops, k, phi, d, xyz, r0=None, i0=None, start=0, end=None, grid=None, block=256):
    numK, numX = k.shape[1], xyz.shape[1]
    dev = [to_dev(torch, v) for v in (k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])]
    dx = [to_dev(torch, xyz[i]) for i in range(3)]
    kv = torch.empty(5 * numK, dtype=torch.float32, device="cuda")
    o_r = to_dev(torch, np.zeros(numX, np.float32) if r0 is None else r0)
    o_i = to_dev(torch, np.zeros(numX, np.float32) if i0 is None else i0)
    st = torch.cuda.current_stream().cuda_stream
    ops.mrif_pack_kvalues(*[t.data_ptr() for t in dev], numK, kv.data_ptr(), st)
    ops.gptb_mrif(numK, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), o_r.data_ptr(), o_i.data_ptr(),
                  kv.data_ptr(), numX, start=start, end=end, grid=grid, block=block).execute(st)
    torch.cuda.synchronize()
    return o_r.cpu().numpy(), o_i.cpu().numpy(), kv.cpu().numpy()


def _scale(kv):
    n = kv.size // 5
    return float(np.abs(kv[3:4 * n:4]).sum() + np.abs(kv[4 * n:]).sum())


@pytest.mark.parametrize("accurate", [0, 1])
@pytest.mark.parametrize("vpt", [2, 4])
@pytest.mark.parametrize("numK", [1, 3, 64, 257, 1025])
def test_small_cases(cuda, oracle, accurate, vpt, numK):
    from tacker_b200 import ops

    numX = 1024
    k, phi, d, xyz = mrif_inputs(oracle, numK, numX, seed=numK)
    ops.set_option("mrif_accurate", accurate)
    ops.set_option("mriq_vpt", vpt)
    try:
        o_r, o_i, kv = _run(cuda, ops, k, phi, d, xyz, grid=3, block=96)
    finally:
        ops.set_option("mrif_accurate", 0)
        ops.set_option("mriq_vpt", 2)
    assert oracle.bit_mismatches(kv, oracle.mrif_pack(k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])) == 0
    w_r, w_i = oracle.mrif_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(numX, np.float32), np.zeros(numX, np.float32))
    r64, i64 = oracle.mrif_f64(kv, xyz[0], xyz[1], xyz[2])
    norm = max(np.abs(r64).max(), np.abs(i64).max())
    for got, w32, w64 in ((o_r, w_r, r64), (o_i, w_i, i64)):
        assert np.abs(got - w32).max() <= 1e-5 * norm
        assert np.abs(got - w64).max() <= 1e-5 * norm
        assert np.abs(got - w64).max() <= 1e-5 * _scale(kv)
    if accurate:   # the reference's own arithmetic: only cosf / sinf rounding (<= 2 ulp each) separates it from the checker
        assert np.abs(o_r - w_r).max() <= 4e-7 * _scale(kv) and np.abs(o_i - w_i).max() <= 4e-7 * _scale(kv)


@pytest.mark.parametrize("split", [64, 100, 0, -1])
@pytest.mark.parametrize("rng", [(0, 1), (1, 3), (0, 4), (3, 3), (2, 9)])
def test_virtual_block_range_split_and_accumulate(cuda, oracle, split, rng):
    from tacker_b200 import ops

    numK, numX = 200, 1024
    start, end = rng
    k, phi, d, xyz = mrif_inputs(oracle, numK, numX, seed=3)
    r0 = oracle.uniform_f32(numX, 905, -2.0, 2.0)
    i0 = oracle.uniform_f32(numX, 906, -2.0, 2.0)
    ops.set_option("mriq_split", split)
    try:
        o_r, o_i, kv = _run(cuda, ops, k, phi, d, xyz, r0=r0, i0=i0, start=start, end=end, grid=2, block=64)
    finally:
        ops.set_option("mriq_split", -1)
    lo, hi = start * 256, min(end, 4) * 256
    outside = np.ones(numX, dtype=bool)
    outside[lo:hi] = False
    assert np.array_equal(o_r[outside], r0[outside]) and np.array_equal(o_i[outside], i0[outside])
    w_r, w_i = r0.copy(), i0.copy()
    oracle.mrif_f32(kv, xyz[0], xyz[1], xyz[2], w_r, w_i, start=start, end=min(end, 4))
    scale = _scale(kv) + 2.0
    assert np.abs(o_r - w_r).max() <= 1e-5 * scale and np.abs(o_i - w_i).max() <= 1e-5 * scale


def test_full_size(cuda, oracle):
    """2048 samples x 262,144 voxels (the shape of the MRI-Q configuration), sampled binary64 reference + linearity."""
    from tacker_b200 import ops

    numK, numX = 2048, 262144
    k, phi, d, xyz = mrif_inputs(oracle, numK, numX, seed=0)
    o_r, o_i, kv = _run(cuda, ops, k, phi, d, xyz, block=512)
    worst, norm = 0.0, 0.0
    for p in range(0, 1024, 41):
        r64, i64 = oracle.mrif_f64(kv, xyz[0], xyz[1], xyz[2], start=p, end=p + 1)
        sl = slice(p * 256, p * 256 + 256)
        worst = max(worst, np.abs(o_r[sl] - r64[sl]).max(), np.abs(o_i[sl] - i64[sl]).max())
        norm = max(norm, np.abs(r64[sl]).max(), np.abs(i64[sl]).max())
    assert worst <= 1e-5 * norm and worst <= 1e-5 * _scale(kv)
    ra, ia, _ = _run(cuda, ops, k[:, :1024], phi[:, :1024], d[:, :1024], xyz, block=512)
    rb, ib, _ = _run(cuda, ops, k[:, 1024:], phi[:, 1024:], d[:, 1024:], xyz, block=512)
    assert np.abs(ra + rb - o_r).max() <= 1e-5 * norm and np.abs(ia + ib - o_i).max() <= 1e-5 * norm
    assert np.isfinite(o_r).all() and np.isfinite(o_i).all()


@pytest.mark.parametrize("pair", [-1, 1])
@pytest.mark.parametrize("cd_threads", [64, 320])
def test_fused_with_tzgemm(cuda, oracle, cd_threads, pair):
    """tzgemm_mrif: with unsplit work items the fused launch leaves bit for bit what the two solo launches leave."""
    from helpers import gemm_inputs, half_dev
    from tacker_b200 import ops

    M, N, K = 512, 512, 128
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=44)
    A, B = half_dev(cuda, a_bits), half_dev(cuda, b_bits)
    numK, numX = 150, 2048
    k, phi, d, xyz = mrif_inputs(oracle, numK, numX, seed=9)
    dev = [to_dev(cuda, v) for v in (k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])]
    dx = [to_dev(cuda, xyz[i]) for i in range(3)]
    kv = cuda.empty(5 * numK, dtype=cuda.float32, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    ops.mrif_pack_kvalues(*[t.data_ptr() for t in dev], numK, kv.data_ptr(), st)
    out = {}
    ops.set_option("mriq_split", 0)
    ops.set_option("mix_pair", pair)
    try:
        for mode in ("solo", "fused"):
            Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
            o_r = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
            o_i = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
            tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, start=5, end=60, grid=4,
                                 round_dims=False)
            cd = ops.gptb_mrif(numK, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), o_r.data_ptr(), o_i.data_ptr(),
                               kv.data_ptr(), numX, start=1, end=7, grid=4, block=cd_threads)
            if mode == "solo":
                tz.execute(st)
                cd.execute(st)
            else:
                ops.mix(cd, tz, cd_threads=cd_threads, grid=4).execute(st)
            cuda.cuda.synchronize()
            assert ops.device_status() == 0
            out[mode] = (Cd.cpu().numpy(), o_r.cpu().numpy(), o_i.cpu().numpy())
    finally:
        ops.set_option("mriq_split", -1)
        ops.set_option("mix_pair", 0)
    for i in range(3):
        assert np.array_equal(out["solo"][i], out["fused"][i])
    kvh = kv.cpu().numpy()
    r64, i64 = oracle.mrif_f64(kvh, xyz[0], xyz[1], xyz[2], start=1, end=7)
    assert np.abs(out["fused"][1] - r64).max() <= 1e-5 * _scale(kvh)
    assert np.abs(out["fused"][2] - i64).max() <= 1e-5 * _scale(kvh)
    assert np.abs(out["fused"][1]).max() > 0
