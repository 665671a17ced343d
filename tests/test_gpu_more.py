"""sgemm, lbm, fft and cutcp through the C ABI against the CPU checker and the fixtures of the reference's own
kernels (B200 only).

All four have one fixed sequence of operations per output, so the solo kernel, the fused kernel and the reference's
kernel are expected to agree bit for bit; the CPU checker agrees with them bit for bit where its C arithmetic can
(sgemm) and to the rounding of cosf / sinf / rsqrt and of the compiler's contractions elsewhere (tolerances below).
"""
import os

import numpy as np
import pytest

from helpers import cutcp_inputs, fft_inputs, gemm_inputs, half_dev, lbm_conflicts, lbm_inputs, sgemm_inputs, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _st(torch):
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture(autouse=True)
def unsplit_items(cuda):
    """The bit-for-bit comparisons need work items that keep the reference's order of additions (launches as small as
    these would otherwise be cut into items that add partial sums in no fixed order); the split forms have tests of
    their own below."""
    from tacker_b200 import ops

    ops.set_option("sgemm_split", 0)
    ops.set_option("cutcp_split", 0)
    yield
    ops.set_option("sgemm_split", -1)
    ops.set_option("cutcp_split", -1)


def _golden(name):
    path = os.path.join(GOLDEN, f"ref_{name}.npz")
    assert os.path.exists(path), f"{path} is missing (tests/golden/make_golden_more.py writes it)"
    return np.load(path)


# ---------------------------------------------------------------------------------------- sgemm ----
def _sgemm(torch, ops, a, b, c, start=0, end=None, grid=3, block=96):
    K, M = a.shape
    N = b.shape[1]
    dA, dB, dC = to_dev(torch, a), to_dev(torch, b), to_dev(torch, c)
    ops.gptb_sgemm(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K, start=start, end=end, grid=grid,
                   block=block).execute(_st(torch))
    torch.cuda.synchronize()
    return dC.cpu().numpy()


@pytest.mark.parametrize("shape", [(128, 16, 1), (128, 16, 8), (256, 64, 72), (384, 48, 41), (128, 272, 24)])
def test_sgemm_small_cases(cuda, oracle, shape):
    from tacker_b200 import ops

    M, N, K = shape
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=M + N + K)
    got = _sgemm(cuda, ops, a, b, c, grid=2, block=160)
    want = oracle.sgemm_f32(a, b, c.copy())
    assert oracle.bit_mismatches(got, want) == 0
    ref64 = 2.0 * c + 2.0 * (b.T.astype(np.float64) @ a.astype(np.float64))
    assert np.abs(got - ref64).max() <= 1e-6 * K * 4


def test_sgemm_ranges_compose_and_leave_the_rest(cuda, oracle):
    from tacker_b200 import ops

    M, N, K = 384, 80, 32
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=5)
    part = _sgemm(cuda, ops, a, b, c, start=4, end=11)
    want = oracle.sgemm_f32(a, b, c.copy(), 4, 11)
    assert oracle.bit_mismatches(part, want) == 0
    assert (part != c).any() and (part == c).any()
    whole = oracle.sgemm_f32(a, b, c.copy())
    two = _sgemm(cuda, ops, a, b, _sgemm(cuda, ops, a, b, c, start=0, end=7), start=7, end=None)
    assert oracle.bit_mismatches(two, whole) == 0


@pytest.mark.parametrize("name", ["sgemm", "sgemm_part"])
def test_sgemm_reference_fixture(cuda, oracle, name):
    from tacker_b200 import ops

    g = _golden(name)
    M, N, K = int(g["M"]), int(g["N"]), int(g["K"])
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=int(g["seed"]))
    got = _sgemm(cuda, ops, a, b, c, start=int(g["start"]), end=int(g["end"]))
    assert oracle.bit_mismatches(got, g["out"]) == 0


@pytest.mark.parametrize("split", [-1, 8, 24, 64])
def test_sgemm_split_items(cuda, oracle, split):
    """Work items that cover a part of K: C is doubled by a kernel of its own, then every item adds 2 x its partial sums."""
    from tacker_b200 import ops

    M, N, K = 256, 48, 200
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=9)
    ops.set_option("sgemm_split", split)
    got = _sgemm(cuda, ops, a, b, c, start=1, end=5, grid=4, block=128)
    want = oracle.sgemm_f32(a, b, c.copy(), 1, 5)
    assert np.array_equal(got != c, want != c)                 # the same blocks, nothing else
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    if split > 0:
        assert oracle.bit_mismatches(got, want) > 0            # really another order of additions


@pytest.mark.parametrize("coop", [2, 1, 0])
@pytest.mark.parametrize("case", [(384, 320, 41, 0, None, 256), (128, 528, 24, 0, None, 512), (256, 272, 19, 5, 29, 256),
                                  (384, 160, 64, 7, 8, 256), (128, 1024, 35, 0, None, 256)])
def test_sgemm_warps_of_a_cta_as_one_group(cuda, oracle, coop, case):
    """Launches over many column blocks: the warps of a CTA share the A slices (groups of 6 to 16 column blocks, ragged
    last groups, block ranges that cut groups, a range too short for the form; coop = 2 takes the form wherever it
    can, 1 only where every CTA gets a full group); bit for bit the same as the per-warp form and the reference's order
    of additions."""
    from tacker_b200 import ops

    M, N, K, start, end, block = case
    ops.set_option("sgemm_coop", coop)
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=M + N + K + 1)
    got = _sgemm(cuda, ops, a, b, c, start=start, end=end, grid=3, block=block)
    ops.set_option("sgemm_coop", 1)
    total = (M // 128) * (N // 16)
    want = oracle.sgemm_f32(a, b, c.copy(), start, total if end is None else end)
    assert oracle.bit_mismatches(got, want) == 0


@pytest.mark.parametrize("split", [-1, 16, 40])
def test_sgemm_groups_split_in_k(cuda, oracle, split):
    from tacker_b200 import ops

    M, N, K = 256, 400, 136
    a, b, c = sgemm_inputs(oracle, M, N, K, seed=31)
    ops.set_option("sgemm_split", split)
    ops.set_option("sgemm_coop", 2)
    got = _sgemm(cuda, ops, a, b, c, grid=2, block=256)
    ops.set_option("sgemm_coop", 1)
    want = oracle.sgemm_f32(a, b, c.copy())
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    if split > 0:
        assert oracle.bit_mismatches(got, want) > 0            # really another order of additions


# ------------------------------------------------------------------------------------------ lbm ----
def _lbm(torch, ops, oracle, src, dst, nx, ny, nz, start=0, end=None, grid=3, block=96):
    m = oracle.lbm_margin(nx, ny)
    dS, dD = to_dev(torch, src), to_dev(torch, dst)
    ops.gptb_lbm(dS.data_ptr() + 4 * m, dD.data_ptr() + 4 * m, nx, ny, nz, start=start, end=end, grid=grid,
                 block=block).execute(_st(torch))
    torch.cuda.synchronize()
    return dD.cpu().numpy()


@pytest.mark.parametrize("dims", [(32, 2, 3), (32, 3, 2), (128, 4, 5), (96, 7, 3)])
def test_lbm_small_cases(cuda, oracle, dims):
    from tacker_b200 import ops

    nx, ny, nz = dims
    src, dst = lbm_inputs(oracle, nx, ny, nz, seed=nx + ny)
    got = _lbm(cuda, ops, oracle, src, dst, nx, ny, nz)
    want = oracle.lbm_f32(src, dst.copy(), nx, ny, nz)
    once = ~lbm_conflicts(oracle, nx, ny, nz)     # addresses with one writer; the others have no defined winner
    # the checker's contraction choices are a model of the compiler's: a few ulp at most where they differ
    assert np.abs(got - want)[once].max() <= 4e-6
    assert np.array_equal((got != dst)[once], (want != dst)[once]) and (got != dst).mean() > 0.4


def test_lbm_range_leaves_other_rows(cuda, oracle):
    from tacker_b200 import ops

    nx, ny, nz = 64, 6, 6
    src, dst = lbm_inputs(oracle, nx, ny, nz, seed=3)
    got = _lbm(cuda, ops, oracle, src, dst, nx, ny, nz, start=7, end=19)
    want = oracle.lbm_f32(src, dst.copy(), nx, ny, nz, 7, 19)
    once = ~lbm_conflicts(oracle, nx, ny, nz, 7, 19)
    assert np.abs(got - want)[once].max() <= 4e-6
    assert np.array_equal(got != dst, want != dst)      # exactly the cells the reference's blocks write


@pytest.mark.parametrize("name", ["lbm", "lbm_part"])
def test_lbm_reference_fixture(cuda, oracle, name):
    from tacker_b200 import ops

    sys_path_golden()
    from make_golden_more import lbm_digest, lbm_sample_index

    g = _golden(name)
    nx, ny, nz = (int(v) for v in g["dims"])
    src, dst = lbm_inputs(oracle, nx, ny, nz, seed=int(g["seed"]))
    got = _lbm(cuda, ops, oracle, src, dst, nx, ny, nz, start=int(g["start"]), end=int(g["end"]), grid=296, block=512)
    idx = lbm_sample_index(got.size, int(g["seed"]))
    assert oracle.bit_mismatches(got[idx], g["sample"]) == 0
    assert np.array_equal(lbm_digest(got), g["digest"])


def sys_path_golden():
    import sys

    if GOLDEN not in sys.path:
        sys.path.insert(0, GOLDEN)


# ------------------------------------------------------------------------------------------ fft ----
def _fft(torch, ops, d, start=0, end=None, grid=3, block=96):
    dd = to_dev(torch, d)
    ops.gptb_fft(dd.data_ptr(), d.shape[0], start=start, end=end, grid=grid, block=block).execute(_st(torch))
    torch.cuda.synchronize()
    return dd.cpu().numpy()


@pytest.mark.parametrize("nfft", [1, 5, 64, 301])
def test_fft_small_cases(cuda, oracle, nfft):
    from tacker_b200 import ops

    d = fft_inputs(oracle, nfft, seed=nfft)
    got = _fft(cuda, ops, d, grid=2, block=128)
    w32 = oracle.fft256_f32(d.copy())
    w64 = oracle.fft256_f64(d)
    scale = float(np.abs(w64).max())
    assert np.abs(got - w32).max() <= 2e-6 * scale      # cosf / sinf of the device and of the host differ by an ulp or two
    assert np.abs(got - w64).max() <= 1e-5 * scale
    numpy_fft = np.fft.fft(d[..., 0].astype(np.float64) + 1j * d[..., 1].astype(np.float64), axis=1)
    assert np.abs(got[..., 0] + 1j * got[..., 1] - numpy_fft).max() <= 1e-5 * scale


def test_fft_range_and_roundtrip(cuda, oracle):
    from tacker_b200 import ops

    d = fft_inputs(oracle, 12, seed=2)
    got = _fft(cuda, ops, d, start=4, end=9)
    assert np.array_equal(got[:4], d[:4]) and np.array_equal(got[9:], d[9:]) and (got[4:9] != d[4:9]).any()
    # inverse through conjugation: conj(F(conj(F(x)))) = 256 x
    full = _fft(cuda, ops, d)
    conj = full.copy()
    conj[..., 1] = -conj[..., 1]
    back = _fft(cuda, ops, conj)
    back[..., 1] = -back[..., 1]
    assert np.abs(back / 256.0 - d).max() <= 1e-5


@pytest.mark.parametrize("name", ["fft", "fft_part"])
def test_fft_reference_fixture(cuda, oracle, name):
    from tacker_b200 import ops

    g = _golden(name)
    d = fft_inputs(oracle, int(g["nfft"]), seed=int(g["seed"]))
    got = _fft(cuda, ops, d, start=int(g["start"]), end=int(g["end"]))
    assert oracle.bit_mismatches(got, g["out"]) == 0


# ---------------------------------------------------------------------------------------- cutcp ----
def _cutcp_setup(torch, ops, oracle, n, h, cutoff, seed, nbrlen=0):
    atoms = cutcp_inputs(oracle, n, n, n, h, seed=seed)
    dims = oracle.cutcp_bin_dims(n, n, n, h, cutoff)
    nbr = oracle.cutcp_neighbours(h, cutoff)
    if nbrlen:
        nbr = nbr[:nbrlen]
    bins, _ = oracle.cutcp_bin_atoms(atoms, dims)
    dB = to_dev(torch, bins)
    dN3 = to_dev(torch, nbr)
    dN = torch.zeros((nbr.shape[0], 4), dtype=torch.int32, device="cuda")
    ops.cutcp_pack_neighbours(dN3.data_ptr(), nbr.shape[0], dN.data_ptr(), _st(torch))
    c = dims[3]
    zero = dB.data_ptr() + 16 * 8 * ((c * dims[1] + c) * dims[0] + c)
    return dict(bins=bins, dims=dims, nbr=nbr, dB=dB, dN=dN, zero=zero, g=(n + 7) // 8, h=h, cutoff=cutoff)


def _cutcp(torch, ops, s, start=0, end=None, grid=3, block=96, regions=None):
    g = s["g"]
    dR = torch.zeros((g, g, g, 512), dtype=torch.float32, device="cuda") if regions is None else regions
    c2 = np.float32(s["cutoff"]) * np.float32(s["cutoff"])
    k = ops.gptb_cutcp(s["dims"][0], s["dims"][1], s["zero"], s["h"], float(c2), float(np.float32(1.0) / c2), dR.data_ptr(),
                       s["dN"].data_ptr(), s["nbr"].shape[0], g, g, g, start=start, end=end, grid=grid, block=block)
    k.execute(_st(torch))
    torch.cuda.synchronize()
    return dR.cpu().numpy()


@pytest.mark.parametrize("n,cutoff", [(8, 12.0), (16, 12.0), (16, 7.5), (24, 4.0)])
def test_cutcp_small_cases(cuda, oracle, n, cutoff):
    from tacker_b200 import ops

    s = _cutcp_setup(cuda, ops, oracle, n, 0.5, cutoff, seed=n)
    got = _cutcp(cuda, ops, s)
    g = s["g"]
    want = oracle.cutcp_f32(s["bins"], s["dims"], s["nbr"], 0.5, cutoff, np.zeros((g, g, g, 512), np.float32), g, g, g)
    # rsqrt.approx against 1 / sqrtf: 2 ulp per term, a few hundred terms of both signs per point
    scale = float(np.abs(want).max())
    assert scale > 0 and np.abs(got - want).max() <= 2e-5 * scale


def test_cutcp_range(cuda, oracle):
    from tacker_b200 import ops

    s = _cutcp_setup(cuda, ops, oracle, 24, 0.5, 12.0, seed=4)
    got = _cutcp(cuda, ops, s, start=5, end=17)
    whole = _cutcp(cuda, ops, s)
    g = s["g"]
    for p in range(g * g * g):
        rx, ry, rz = p // (g * g), (p // g) % g, p % g
        if 5 <= p < 17:
            assert np.array_equal(got[rz, ry, rx], whole[rz, ry, rx])
        else:
            assert not got[rz, ry, rx].any()


@pytest.mark.parametrize("split", [-1, 8, 50])
def test_cutcp_split_items(cuda, oracle, split):
    """Work items that cover a part of the neighbour list: the regions are zeroed by a kernel of its own, then every item
    adds its partial sums.  Regions outside the block range keep what they held."""
    from tacker_b200 import ops

    s = _cutcp_setup(cuda, ops, oracle, 16, 0.5, 12.0, seed=12)
    g = s["g"]
    ops.set_option("cutcp_split", 0)
    exact = _cutcp(cuda, ops, s, start=2, end=7)
    ops.set_option("cutcp_split", split)
    pre = cuda.full((g, g, g, 512), 3.5, dtype=cuda.float32, device="cuda")
    got = _cutcp(cuda, ops, s, start=2, end=7, grid=4, block=256, regions=pre)
    for p in range(g * g * g):
        rx, ry, rz = p // (g * g), (p // g) % g, p % g
        if 2 <= p < 7:
            assert np.abs(got[rz, ry, rx] - exact[rz, ry, rx]).max() <= 1e-5 * np.abs(exact).max()
        else:
            assert (got[rz, ry, rx] == 3.5).all()


@pytest.mark.parametrize("name", ["cutcp", "cutcp_256"])
def test_cutcp_reference_fixture(cuda, oracle, name):
    from tacker_b200 import ops

    g = _golden(name)
    s = _cutcp_setup(cuda, ops, oracle, int(g["n"]), float(g["h"]), float(g["cutoff"]), seed=int(g["seed"]),
                     nbrlen=int(g["nbrlen"]))
    got = _cutcp(cuda, ops, s, start=int(g["start"]), end=int(g["end"]))
    assert oracle.bit_mismatches(got, g["out"]) == 0


# ---------------------------------------------------------------------------------------- fused ----
@pytest.fixture(params=[-1, 1], ids=["one_cta", "cta_pairs"])
def tensor_role(request, cuda):
    """Both forms of the tensor role inside the fused kernels: on one CTA, and on CTA pairs."""
    from tacker_b200 import ops

    ops.set_option("mix_pair", request.param)
    yield request.param
    ops.set_option("mix_pair", 0)


@pytest.mark.parametrize("cd_threads", [64, 256, 512])
@pytest.mark.parametrize("kind", ["sgemm", "lbm", "fft", "cutcp"])
def test_fused_with_tzgemm_is_bit_identical_to_solo(cuda, oracle, kind, cd_threads, tensor_role):
    from tacker_b200 import ops

    M, N, K = 512, 512, 128
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=61)
    A, B = half_dev(cuda, a_bits), half_dev(cuda, b_bits)
    st = _st(cuda)
    if kind == "sgemm":
        sa, sb, sc = sgemm_inputs(oracle, 256, 96, 40, seed=6)
        dA, dB = to_dev(cuda, sa), to_dev(cuda, sb)
        make = lambda: to_dev(cuda, sc)
        cdk = lambda out: ops.gptb_sgemm(dA.data_ptr(), dB.data_ptr(), out.data_ptr(), 256, 96, 40, start=1, end=11, grid=4,
                                         block=cd_threads)
    elif kind == "lbm":
        nx, ny, nz = 64, 5, 4
        src, dst = lbm_inputs(oracle, nx, ny, nz, seed=6)
        m = oracle.lbm_margin(nx, ny)
        dS = to_dev(cuda, src)
        make = lambda: to_dev(cuda, dst)
        cdk = lambda out: ops.gptb_lbm(dS.data_ptr() + 4 * m, out.data_ptr() + 4 * m, nx, ny, nz, start=2, end=19, grid=4,
                                       block=cd_threads)
    elif kind == "fft":
        d = fft_inputs(oracle, 40, seed=6)
        make = lambda: to_dev(cuda, d)
        cdk = lambda out: ops.gptb_fft(out.data_ptr(), 40, start=3, end=37, grid=4, block=cd_threads)
    else:
        s = _cutcp_setup(cuda, ops, oracle, 16, 0.5, 12.0, seed=6)
        g = s["g"]
        c2 = np.float32(144.0)
        make = lambda: cuda.zeros((g, g, g, 512), dtype=cuda.float32, device="cuda")
        cdk = lambda out: ops.gptb_cutcp(s["dims"][0], s["dims"][1], s["zero"], 0.5, float(c2), float(np.float32(1.0) / c2),
                                         out.data_ptr(), s["dN"].data_ptr(), s["nbr"].shape[0], g, g, g, start=1, end=8,
                                         grid=4, block=cd_threads)
    res = {}
    for mode in ("solo", "fused", "fused_empty_gemm", "fused_empty_cd"):
        Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
        out = make()
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, start=5, end=60, grid=4,
                             round_dims=False)
        cd = cdk(out)
        if mode == "solo":
            tz.execute(st)
            cd.execute(st)
        elif mode == "fused":
            ops.mix(cd, tz, cd_threads=cd_threads, grid=4).execute(st)
        elif mode == "fused_empty_gemm":
            ops.mix(cd, tz, cd_threads=cd_threads, grid=4, tz_range=(0, 0)).execute(st)
        else:
            ops.mix(cd, tz, cd_threads=cd_threads, grid=4, cd_range=(0, 0)).execute(st)
        cuda.cuda.synchronize()
        assert ops.device_status() == 0
        res[mode] = (Cd.cpu().numpy(), out.cpu().numpy())
    # lbm: addresses that two cells write have no defined winner (in the reference either); everything else is compared
    once = ~lbm_conflicts(oracle, 64, 5, 4, 2, 19) if kind == "lbm" else np.ones(res["solo"][1].shape, bool)
    assert np.array_equal(res["solo"][0], res["fused"][0]) and np.array_equal(res["solo"][1][once], res["fused"][1][once])
    assert np.abs(res["fused"][0]).max() > 0
    assert not res["fused_empty_gemm"][0].any() and np.array_equal(res["fused_empty_gemm"][1][once], res["solo"][1][once])
    assert np.array_equal(res["fused_empty_cd"][0], res["solo"][0])
    assert np.array_equal(res["fused_empty_cd"][1], make().cpu().numpy())
    if kind in ("sgemm", "cutcp"):      # the default, split work items inside the fused kernel: same values to 1e-5
        ops.set_option("sgemm_split", -1)
        ops.set_option("cutcp_split", -1)
        Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
        out = make()
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, start=5, end=60, grid=4,
                             round_dims=False)
        ops.mix(cdk(out), tz, cd_threads=cd_threads, grid=4).execute(st)
        cuda.cuda.synchronize()
        assert ops.device_status() == 0
        assert np.array_equal(Cd.cpu().numpy(), res["solo"][0])
        assert np.abs(out.cpu().numpy() - res["solo"][1]).max() <= 1e-5 * np.abs(res["solo"][1]).max()
    ref = oracle.tzgemm_f64(a, b)
    tiles = np.zeros((M // 64, N // 64), bool).ravel()
    tiles[5:60] = True
    mask = np.kron(tiles.reshape(M // 64, N // 64), np.ones((64, 64), bool))
    assert np.abs(res["fused"][0] - ref * mask).max() <= 1e-3 * K


def test_ori_launch_shape(cuda, oracle):
    """ori_<k>: the original grid from the solo argument list alone."""
    from tacker_b200 import ops

    a, b, c = sgemm_inputs(oracle, 128, 32, 16, seed=8)
    dA, dB, dC = to_dev(cuda, a), to_dev(cuda, b), to_dev(cuda, c)
    ops.OriSGEMMKernel(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), 128, 32, 16).execute(_st(cuda))
    d = fft_inputs(oracle, 7, seed=8)
    dd = to_dev(cuda, d)
    ops.OriFFTKernel(dd.data_ptr(), 7).execute(_st(cuda))
    cuda.cuda.synchronize()
    assert oracle.bit_mismatches(dC.cpu().numpy(), oracle.sgemm_f32(a, b, c.copy())) == 0
    assert np.abs(dd.cpu().numpy() - oracle.fft256_f32(d.copy())).max() <= 1e-4


# ------------------------------------------------------------------------- the reference's sizes ----
def test_sgemm_reference_size_sampled(cuda, oracle):
    """4096 x 4128 x 4064 (src/ori_kernel/sgemm_kernel.cu:85-87): sampled outputs against binary64 dot products, and the
    default (split) items against the unsplit ones."""
    from tacker_b200 import ops

    M, N, K = 4096, 4128, 4064
    gen = cuda.Generator(device="cuda").manual_seed(5)
    A = cuda.rand(K, M, device="cuda", generator=gen)
    B = cuda.rand(K, N, device="cuda", generator=gen)
    C0 = cuda.rand(N, M, device="cuda", generator=gen)
    outs = {}
    for split in (0, -1):
        ops.set_option("sgemm_split", split)
        C = C0.clone()
        ops.gptb_sgemm(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, grid=ops.sm_count(), block=512).execute(_st(cuda))
        cuda.cuda.synchronize()
        outs[split] = C
    rng = np.random.default_rng(1)
    ms, ns = rng.integers(0, M, 300), rng.integers(0, N, 300)
    a = A[:, ms].double().cpu().numpy()
    b = B[:, ns].double().cpu().numpy()
    want = 2.0 * C0[ns, ms].double().cpu().numpy() + 2.0 * (a * b).sum(axis=0)
    for split, C in outs.items():
        got = C[ns, ms].cpu().numpy()
        # 4064 binary32 additions in sequence (the reference's order): a few units of 1e-6 relative
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max(), split
    assert float((outs[0] - outs[-1]).abs().max()) <= 1e-5 * float(outs[0].abs().max())


def test_fft_reference_size(cuda, oracle):
    """10240 transforms (FFT_B, src/header/fft_header.h:13) against numpy's, and Parseval's sum on every one."""
    from tacker_b200 import ops

    d = fft_inputs(oracle, 10240, seed=77)
    got = _fft(cuda, ops, d, grid=296, block=512)
    want = np.fft.fft(d[..., 0].astype(np.float64) + 1j * d[..., 1].astype(np.float64), axis=1)
    scale = float(np.abs(want).max())
    assert np.abs(got[..., 0] + 1j * got[..., 1] - want).max() <= 1e-5 * scale
    energy_in = (d.astype(np.float64) ** 2).sum(axis=(1, 2))
    energy_out = (got.astype(np.float64) ** 2).sum(axis=(1, 2)) / 256.0
    assert np.abs(energy_out - energy_in).max() <= 1e-5 * energy_in.max()


def test_cutcp_reference_size_sampled(cuda, oracle):
    """The reference's launch (26 x 26 x 2 regions of a 208-point lattice, 335 neighbour bins): a sample of regions against
    the CPU checker, unsplit items bit for bit against split ones to 1e-5, and superposition (the potential of all atoms =
    the potential of the even bins' atoms + that of the odd bins')."""
    from tacker_b200 import ops

    atoms = cutcp_inputs(oracle, 208, 208, 16, 0.5, seed=31)
    dims = oracle.cutcp_bin_dims(208, 208, 16, 0.5, 12.0)
    nbr = oracle.cutcp_neighbours(0.5, 12.0)
    bins, _ = oracle.cutcp_bin_atoms(atoms, dims)
    dN = cuda.zeros((nbr.shape[0], 4), dtype=cuda.int32, device="cuda")
    ops.cutcp_pack_neighbours(to_dev(cuda, nbr).data_ptr(), nbr.shape[0], dN.data_ptr(), _st(cuda))
    c = dims[3]

    def run(b, split):
        dB = to_dev(cuda, b)
        zero = dB.data_ptr() + 128 * ((c * dims[1] + c) * dims[0] + c)
        dR = cuda.zeros((2, 26, 26, 512), dtype=cuda.float32, device="cuda")
        ops.set_option("cutcp_split", split)
        ops.gptb_cutcp(dims[0], dims[1], zero, 0.5, 144.0, float(np.float32(1.0) / np.float32(144.0)), dR.data_ptr(),
                       dN.data_ptr(), nbr.shape[0], 26, 26, 2, grid=296, block=512).execute(_st(cuda))
        cuda.cuda.synchronize()
        return dR.cpu().numpy()

    exact, split = run(bins, 0), run(bins, -1)
    scale = float(np.abs(exact).max())
    assert np.abs(exact - split).max() <= 1e-5 * scale
    want = np.zeros_like(exact)
    picks = [0, 1, 27, 700, 1351]
    for p in picks:
        oracle.cutcp_f32(bins, dims, nbr, 0.5, 12.0, want, 26, 26, 2, p, p + 1)
    for p in picks:
        rx, ry, rz = p // 52, (p // 2) % 26, p % 2
        assert np.abs(exact[rz, ry, rx] - want[rz, ry, rx]).max() <= 2e-5 * scale
    even = bins.copy()
    odd = bins.copy()
    parity = (np.indices(bins.shape[:3]).sum(axis=0) % 2).astype(bool)
    even[parity] = 0.0
    odd[~parity] = 0.0
    assert np.abs(run(even, 0) + run(odd, 0) - exact).max() <= 1e-5 * scale
