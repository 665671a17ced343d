"""Fused tensor-core + CUDA-core kernels through the C ABI (B200 only).

A fused launch must leave exactly what the two solo launches leave: the CUDA-core role runs the
same device function, so with a fixed summation order (stencil always; Coulomb and MRI-Q with unsplit
work items) its output is bit-identical to the solo kernel's, and the tensor role's tiles are bit-identical
to the solo tzgemm's.  With split work items (the default of the fast modes: partial sums are added with
reductions in no fixed order) the CUDA-core output is held to the operator's tolerance instead.
"""
import numpy as np
import pytest

from helpers import coulomb_inputs, gemm_inputs, half_dev, mriq_inputs, stencil_inputs, to_dev

pytestmark = pytest.mark.gpu


def _gemm_setup(torch, oracle, M, N, K, seed):
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=seed)
    return half_dev(torch, a_bits), half_dev(torch, b_bits), a, b


@pytest.mark.parametrize("cd_threads", [64, 128, 256, 512])
@pytest.mark.parametrize("ranges", [((0, 9), (0, 24)), ((2, 7), (5, 19)), ((0, 9), (0, 0)), ((0, 0), (0, 24))])
def test_tzgemm_stencil(cuda, oracle, cd_threads, ranges):
    from tacker_b200 import ops

    (cs, ce), (ts, te) = ranges
    M, N, K = 256, 384, 256
    nz, ny, nx = 10, 12, 192
    A, B, a, b = _gemm_setup(cuda, oracle, M, N, K, 4)
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=6)
    st = cuda.cuda.current_stream().cuda_stream
    out = {}
    for mode in ("solo", "fused"):
        Cd = cuda.full((M, N), -3.0, dtype=cuda.float32, device="cuda")
        d0, d1 = to_dev(cuda, A0), to_dev(cuda, np.full_like(A0, 9.0))
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.1, start=ts, end=te, grid=2,
                             round_dims=False)
        cd = ops.gptb_stencil(0.5, 0.25, d0.data_ptr(), d1.data_ptr(), nx, ny, nz, start=cs, end=ce, grid=2,
                              block=cd_threads)
        if mode == "solo":
            tz.execute(st)
            cd.execute(st)
        else:
            ops.mix(cd, tz, cd_threads=cd_threads, grid=2).execute(st)
        cuda.cuda.synchronize()
        assert ops.device_status() == 0
        out[mode] = (Cd.cpu().numpy(), d1.cpu().numpy())
    assert np.array_equal(out["solo"][0], out["fused"][0])
    assert np.array_equal(out["solo"][1], out["fused"][1])
    want = oracle.stencil_sweep_f32(0.5, 0.25, A0, np.full_like(A0, 9.0), start=cs, end=ce, contract=1)
    assert oracle.bit_mismatches(out["fused"][1], want) == 0
    if te > ts:
        ref = oracle.tzgemm_f64(a, b, alpha=1.1, start=ts, end=te)
        written = out["fused"][0] != -3.0
        assert written.sum() == (te - ts) * 64 * 64
        assert np.abs(out["fused"][0][written] - ref[written]).max() <= 1e-3 * K


@pytest.mark.parametrize("split", [0, -1, 64])
@pytest.mark.parametrize("cd_threads", [32, 256])
def test_tzgemm_cp(cuda, oracle, cd_threads, split):
    from tacker_b200 import ops

    ops.set_option("cp_split", split)
    try:
        _tzgemm_cp(cuda, oracle, ops, cd_threads, split)
    finally:
        ops.set_option("cp_split", -1)


def _tzgemm_cp(cuda, oracle, ops, cd_threads, split):

    M, N, K = 384, 256, 128
    nx, ny, h, z = 256, 32, 0.125, 2.0
    A, B, a, b = _gemm_setup(cuda, oracle, M, N, K, 8)
    atoms = coulomb_inputs(oracle, 130, 16.0, seed=2, spacing=h, zplane=z)
    raw = to_dev(cuda, atoms)
    packed = cuda.empty_like(raw)
    st = cuda.cuda.current_stream().cuda_stream
    ops.cp_pack_atoms(raw.data_ptr(), atoms.shape[0], z, packed.data_ptr(), st)
    out = {}
    for mode in ("solo", "fused"):
        Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
        lat = cuda.zeros((ny, nx), dtype=cuda.float32, device="cuda")
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, grid=3, round_dims=False)
        cd = ops.gptb_cp(atoms.shape[0], h, lat.data_ptr(), packed.data_ptr(), nx, ny, start=1, end=7, grid=3,
                         block=cd_threads)
        if mode == "solo":
            tz.execute(st)
            cd.execute(st)
        else:
            ops.mix(cd, tz, cd_threads=cd_threads, grid=3).execute(st)
        cuda.cuda.synchronize()
        assert ops.device_status() == 0
        out[mode] = (Cd.cpu().numpy(), lat.cpu().numpy())
    assert np.array_equal(out["solo"][0], out["fused"][0])
    if split == 0:
        assert np.array_equal(out["solo"][1], out["fused"][1])
    pk = oracle.cp_pack_atoms(atoms, z)
    ref32 = oracle.cp_f32(pk, h, np.zeros((ny, nx), np.float32), start=1, end=7, chunk=64)
    _, mag = oracle.cp_f64(pk, h, nx, ny, start=1, end=7)
    touched = mag > 0
    assert np.all(out["fused"][1][~touched] == 0)
    assert (np.abs(out["fused"][1] - ref32)[touched] / mag[touched]).max() <= 1e-5
    assert np.abs(out["fused"][0] - oracle.tzgemm_f64(a, b)).max() <= 1e-3 * K


@pytest.mark.parametrize("split", [0, -1, 64])
@pytest.mark.parametrize("cd_threads", [64, 256])
def test_tzgemm_mriq(cuda, oracle, cd_threads, split):
    from tacker_b200 import ops

    ops.set_option("mriq_split", split)
    try:
        _tzgemm_mriq(cuda, oracle, ops, cd_threads, split)
    finally:
        ops.set_option("mriq_split", -1)


def _tzgemm_mriq(cuda, oracle, ops, cd_threads, split):

    M, N, K = 256, 256, 192
    numK, numX = 200, 2048
    A, B, a, b = _gemm_setup(cuda, oracle, M, N, K, 12)
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=7)
    dk = [to_dev(cuda, k[i]) for i in range(3)]
    dphi = [to_dev(cuda, phi[i]) for i in range(2)]
    dx = [to_dev(cuda, xyz[i]) for i in range(3)]
    kv = cuda.empty((numK, 4), dtype=cuda.float32, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    ops.mriq_pack_kvalues(dk[0].data_ptr(), dk[1].data_ptr(), dk[2].data_ptr(), dphi[0].data_ptr(),
                          dphi[1].data_ptr(), numK, kv.data_ptr(), st)
    out = {}
    for mode in ("solo", "fused"):
        Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
        qr = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
        qi = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, start=3, end=16, grid=2,
                             round_dims=False)
        cd = ops.gptb_mriq(numK, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(),
                           kv.data_ptr(), numX, start=0, end=8, grid=2, block=cd_threads)
        if mode == "solo":
            tz.execute(st)
            cd.execute(st)
        else:
            ops.mix(cd, tz, cd_threads=cd_threads, grid=2).execute(st)
        cuda.cuda.synchronize()
        assert ops.device_status() == 0
        out[mode] = (Cd.cpu().numpy(), qr.cpu().numpy(), qi.cpu().numpy())
    for i in range(3 if split == 0 else 1):
        assert np.array_equal(out["solo"][i], out["fused"][i])
    kvh = kv.cpu().numpy()
    r64, i64 = oracle.mriq_f64(kvh, xyz[0], xyz[1], xyz[2])
    scale = float(kvh[:, 3].sum())
    assert np.abs(out["fused"][1] - r64).max() <= 1e-5 * scale
    assert np.abs(out["fused"][2] - i64).max() <= 1e-5 * scale


@pytest.mark.parametrize("cd", ["stencil", "cp", "mriq"])
@pytest.mark.parametrize("tz_range", [(0, 96), (7, 70), (95, 96)])
def test_fused_kernels_on_cta_pairs(cuda, oracle, cd, tz_range):
    """The fused kernels whose tensor role runs on clusters of two CTAs (option mix_pair = 1) leave what the
    single-CTA fused kernels leave: GEMM tiles and stencil bit for bit, Coulomb / MRI-Q bit for bit with unsplit
    work items."""
    from tacker_b200 import ops

    M, N, K = 512, 768, 128                       # 8 x 12 = 96 tiles
    A, B, a, b = _gemm_setup(cuda, oracle, M, N, K, 31)
    st = cuda.cuda.current_stream().cuda_stream
    nz, ny, nx = 8, 16, 256
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=9)
    atoms = coulomb_inputs(oracle, 100, 16.0, seed=4, spacing=0.125, zplane=2.0)
    raw = to_dev(cuda, atoms)
    packed = cuda.empty_like(raw)
    ops.cp_pack_atoms(raw.data_ptr(), atoms.shape[0], 2.0, packed.data_ptr(), st)
    k, phi, xyz = mriq_inputs(oracle, 96, 1024, seed=8)
    dk = [to_dev(cuda, k[i]) for i in range(3)]
    dphi = [to_dev(cuda, phi[i]) for i in range(2)]
    dx = [to_dev(cuda, xyz[i]) for i in range(3)]
    kv = cuda.empty((96, 4), dtype=cuda.float32, device="cuda")
    ops.mriq_pack_kvalues(dk[0].data_ptr(), dk[1].data_ptr(), dk[2].data_ptr(), dphi[0].data_ptr(),
                          dphi[1].data_ptr(), 96, kv.data_ptr(), st)
    out = {}
    ops.set_option("cp_split", 0)
    ops.set_option("mriq_split", 0)
    try:
        for pair in (-1, 1):
            ops.set_option("mix_pair", pair)
            Cd = cuda.full((M, N), -3.0, dtype=cuda.float32, device="cuda")
            tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.1, start=tz_range[0],
                                 end=tz_range[1], grid=6, round_dims=False)
            if cd == "stencil":
                d0, d1 = to_dev(cuda, A0), to_dev(cuda, np.full_like(A0, 9.0))
                cdk = ops.gptb_stencil(0.5, 0.25, d0.data_ptr(), d1.data_ptr(), nx, ny, nz, grid=6, block=192)
                res = [d1]
            elif cd == "cp":
                lat = cuda.zeros((32, 256), dtype=cuda.float32, device="cuda")
                cdk = ops.gptb_cp(atoms.shape[0], 0.125, lat.data_ptr(), packed.data_ptr(), 256, 32, grid=6, block=192)
                res = [lat]
            else:
                qr = cuda.zeros(1024, dtype=cuda.float32, device="cuda")
                qi = cuda.zeros(1024, dtype=cuda.float32, device="cuda")
                cdk = ops.gptb_mriq(96, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(),
                                    kv.data_ptr(), 1024, grid=6, block=192)
                res = [qr, qi]
            ops.mix(cdk, tz, cd_threads=192, grid=6).execute(st)
            cuda.cuda.synchronize()
            assert ops.device_status() == 0
            out[pair] = [Cd.cpu().numpy()] + [r.cpu().numpy() for r in res]
    finally:
        ops.set_option("mix_pair", 0)
        ops.set_option("cp_split", -1)
        ops.set_option("mriq_split", -1)
    for x, y in zip(out[-1], out[1]):
        assert np.array_equal(x, y)
    written = out[1][0] != -3.0
    assert written.sum() == (tz_range[1] - tz_range[0]) * 64 * 64
    assert np.abs(out[1][0] - oracle.tzgemm_f64(a, b, alpha=1.1))[written].max() <= 1e-3 * K
    assert np.abs(out[1][1]).max() > 0


def test_fused_full_size_config2_properties(cuda, oracle):
    """GEMM 4096 x 4096 x 1024 fused with one 512 x 512 x 64 sweep per launch, GEMM tiles split over 10 launches."""
    from tacker_b200 import ops

    M = N = 4096
    K = 1024
    nx, ny, nz = 512, 512, 64
    A, B, a, b = _gemm_setup(cuda, oracle, M, N, K, 1)
    Cd = cuda.full((M, N), float("nan"), dtype=cuda.float32, device="cuda")
    A0 = stencil_inputs(oracle, nx, ny, nz)
    x, y = to_dev(cuda, A0), to_dev(cuda, A0)
    c0, c1 = np.float32(1 / 6), np.float32(-1 / 6)
    st = cuda.cuda.current_stream().cuda_stream
    bounds = [round(i * 4096 / 10) for i in range(11)]
    for it in range(10):
        src, dst = (x, y) if it % 2 == 0 else (y, x)
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0)
        cd = ops.gptb_stencil(c0, c1, src.data_ptr(), dst.data_ptr(), nx, ny, nz)
        ops.mix(cd, tz, cd_threads=256, tz_range=(bounds[it], bounds[it + 1])).execute(st)
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    got = Cd.cpu().numpy()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(3)
    rows = rng.integers(0, M, 20000).astype(np.int32)
    cols = rng.integers(0, N, 20000).astype(np.int32)
    val, mag = oracle.tzgemm_sampled(a, b, rows, cols)
    assert (np.abs(got[rows, cols] - val) / mag).max() <= 1e-3
    p, q = A0.copy(), A0.copy()
    want = oracle.stencil_jacobi_f32(c0, c1, p, q, 10, contract=1)
    assert oracle.bit_mismatches(x.cpu().numpy(), want) == 0
