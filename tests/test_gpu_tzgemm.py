"""tcgen05 tzgemm through the C ABI against the CPU checker (B200 only).

Tolerance: |got - want| <= 1e-3 * sum_k |a_ik||b_jk| with `want` accumulated in binary64 -- the
stated 1e-3 relative bound, measured against the magnitude of the dot product so that outputs
that cancel to ~0 do not blow the ratio up; the plain element-wise relative error is also
checked wherever |want| is not tiny.
"""
import numpy as np
import pytest

from helpers import gemm_inputs, half_dev

pytestmark = pytest.mark.gpu

REL_TOL = 1e-3


def _run(torch, ops, a_bits, b_bits, M, N, K, alpha, start=0, end=None, grid=None, sentinel=None):
    A = half_dev(torch, a_bits)
    B = half_dev(torch, b_bits)
    Cd = torch.full((M, N), float("nan") if sentinel is None else sentinel, dtype=torch.float32, device="cuda")
    k = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=alpha, start=start, end=end,
                        grid=grid, round_dims=False)
    k.execute(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return Cd.cpu().numpy()


def _check(oracle, got, a, b, alpha):
    want = oracle.tzgemm_f64(a, b, alpha=alpha)
    mag = abs(alpha) * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T)
    assert np.isfinite(got).all()
    err = np.abs(got - want) / mag
    assert err.max() <= REL_TOL, f"scaled error {err.max():.3e}"
    big = np.abs(want) > 0.05 * mag
    assert (np.abs(got - want)[big] / np.abs(want)[big]).max() <= REL_TOL
    # and close to the binary32 triple loop the configuration names as its check
    ref32 = oracle.tzgemm_f32(a, b, alpha=alpha)
    assert np.abs(got - ref32).max() <= REL_TOL * mag.max()


@pytest.mark.parametrize("bn", [0, 128, 256])
@pytest.mark.parametrize("alpha", [1.0, 1.1])
def test_config1_1024_cubed(cuda, oracle, bn, alpha):
    from tacker_b200 import ops

    ops.set_option("tzgemm_bn", bn)
    try:
        M = N = K = 1024
        a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=0)
        got = _run(cuda, ops, a_bits, b_bits, M, N, K, alpha)
        _check(oracle, got, a, b, alpha)
    finally:
        ops.set_option("tzgemm_bn", 0)


@pytest.mark.parametrize("shape", [(128, 128, 128), (128, 64, 64), (256, 192, 128), (384, 320, 448),
                                   (128, 896, 4096), (1024, 128, 64)])
@pytest.mark.parametrize("bn", [128, 256])
def test_small_and_ragged_shapes(cuda, oracle, shape, bn):
    from tacker_b200 import ops

    M, N, K = shape
    ops.set_option("tzgemm_bn", bn)
    try:
        a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=M + N + K)
        got = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.0, grid=3)
        _check(oracle, got, a, b, 1.0)
    finally:
        ops.set_option("tzgemm_bn", 0)


@pytest.mark.parametrize("shape", [(256, 256, 128), (384, 320, 192), (1024, 1024, 1024), (640, 1280, 256)])
def test_m256_super_tile_kernel(cuda, oracle, shape):
    """The 256 x 256 super-tile form of the solo kernel: same results as the 128-row form, bit for bit."""
    from tacker_b200 import ops

    M, N, K = shape
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=M + K)
    out = {}
    for mode in (-1, 1):
        ops.set_option("tzgemm_m256", mode)
        try:
            out[mode] = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.1, grid=5)
        finally:
            ops.set_option("tzgemm_m256", 0)
    _check(oracle, out[1], a, b, 1.1)
    assert np.array_equal(out[1], out[-1])


@pytest.mark.parametrize("grid", [2, 5, 148])
@pytest.mark.parametrize("shape", [(256, 256, 128), (384, 320, 192), (1024, 1024, 1024), (640, 1280, 256), (128, 512, 64)])
def test_cta_pair_kernel(cuda, oracle, shape, grid):
    """tzgemm on clusters of two CTAs (tcgen05.mma.cta_group::2, 256 x 256 pair tiles): same results as the 128-row
    form, bit for bit -- including M = 128 (2k + 1), where the second CTA of the last pair has no rows, N not a
    multiple of 256, and a shape the pair form does not take (M = 128: the launcher falls back)."""
    from tacker_b200 import ops

    M, N, K = shape
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=M + K + 1)
    out = {}
    for mode in (-1, 1):
        ops.set_option("tzgemm_pair", mode)
        ops.set_option("tzgemm_m256", -1)
        try:
            out[mode] = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.1, grid=grid)
        finally:
            ops.set_option("tzgemm_pair", 0)
            ops.set_option("tzgemm_m256", 0)
    _check(oracle, out[1], a, b, 1.1)
    assert np.array_equal(out[1], out[-1])


@pytest.mark.parametrize("bn", [128, 256, 512, 1024])
@pytest.mark.parametrize("rng", [(0, 1), (5, 6), (3, 17), (7, 8), (0, 24), (23, 24), (9, 9), (11, 40)])
def test_virtual_block_range_is_exact(cuda, oracle, bn, rng):
    """Tiles outside [start, end) keep the sentinel; tiles inside match (src/gptb_kernel/tzgemm_kernel.cu:243-249)."""
    from tacker_b200 import ops

    M, N, K = 256, 384, 128          # 4 x 6 = 24 tiles of 64 x 64
    start, end = rng
    if bn == 512:                    # stands for the 256 x 256 super-tile kernel
        ops.set_option("tzgemm_m256", 1)
    elif bn == 1024:                 # stands for the kernel on CTA pairs
        ops.set_option("tzgemm_pair", 1)
    else:
        ops.set_option("tzgemm_bn", bn)
        ops.set_option("tzgemm_m256", -1)
    try:
        a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=9)
        got = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.1, start=start, end=end, grid=2, sentinel=-123.0)
    finally:
        ops.set_option("tzgemm_bn", 0)
        ops.set_option("tzgemm_m256", 0)
        ops.set_option("tzgemm_pair", 0)
    want = oracle.tzgemm_f64(a, b, alpha=1.1)
    inside = np.zeros((M, N), dtype=bool)
    for p in range(start, min(end, 24)):
        r, c = (p // 6) * 64, (p % 6) * 64
        inside[r:r + 64, c:c + 64] = True
    assert np.all(got[~inside] == -123.0)
    if inside.any():
        assert np.abs(got[inside] - want[inside]).max() <= REL_TOL * K


def test_ranges_compose_to_full_result(cuda, oracle):
    from tacker_b200 import ops

    M, N, K = 512, 512, 256
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=21)
    full = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.0)
    A = half_dev(cuda, a_bits)
    B = half_dev(cuda, b_bits)
    Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
    for s, e in ((0, 13), (13, 14), (14, 50), (50, 64)):
        ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, start=s, end=e,
                        grid=5).execute(cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert np.array_equal(Cd.cpu().numpy(), full)       # same tiles, same arithmetic: bit-identical


@pytest.mark.parametrize("shape", [(4096, 4096, 1024), (2048, 2048, 2048), (4096, 4096, 2048)])
def test_full_size_configs_sampled(cuda, oracle, shape):
    """Headline GEMM shapes: 65,536 sampled outputs plus the four corner tiles, binary64 reference."""
    from tacker_b200 import ops

    M, N, K = shape
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=1)
    got = _run(cuda, ops, a_bits, b_bits, M, N, K, 1.0)
    rng = np.random.default_rng(0)
    rows = rng.integers(0, M, 65536).astype(np.int32)
    cols = rng.integers(0, N, 65536).astype(np.int32)
    corner = [(r, c) for r0 in (0, M - 64) for c0 in (0, N - 64) for r in range(r0, r0 + 64, 9)
              for c in range(c0, c0 + 64, 7)]
    rows = np.concatenate([rows, np.array([r for r, _ in corner], dtype=np.int32)])
    cols = np.concatenate([cols, np.array([c for _, c in corner], dtype=np.int32)])
    val, mag = oracle.tzgemm_sampled(a, b, rows, cols, alpha=1.0)
    assert np.isfinite(got).all()
    assert (np.abs(got[rows, cols] - val) / mag).max() <= REL_TOL
    # size-independent property: row sums of C equal A . (column sums of B^T), checked in binary64
    want_rowsum = a.astype(np.float64) @ b.astype(np.float64).sum(0)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).sum(0)
    assert (np.abs(got.astype(np.float64).sum(1) - want_rowsum) / scale).max() <= REL_TOL


def test_bad_arguments_return_status(cuda):
    import ctypes as C

    from tacker_b200 import ops

    A = cuda.zeros(128 * 128, dtype=cuda.float16, device="cuda")
    Cd = cuda.zeros(128 * 128, dtype=cuda.float32, device="cuda")

    def status(m, n, k, a_ptr=None, nparams=17):
        p = [C.c_void_p(a_ptr or A.data_ptr()), C.c_void_p(A.data_ptr()), C.c_void_p(Cd.data_ptr()), C.c_int(m),
             C.c_int(n), C.c_int(k), C.c_float(1.0)] + [C.c_int(1)] * 6 + [C.c_int(0), C.c_int(1), C.c_int(4),
                                                                          C.c_int(0)]
        return ops.raw_launch("gptb_tzgemm", p[:nparams], (4, 1, 1), (192, 1, 1))

    assert status(128, 128, 128) == 0
    assert status(100, 128, 128) == -3          # M not a multiple of 128
    assert status(128, 128, 96) == -3           # K not a multiple of 64
    assert status(128, 128, 128, a_ptr=A.data_ptr() + 2) == -2
    assert status(128, 128, 128, nparams=16) == -1
    cuda.cuda.synchronize()


@pytest.mark.parametrize("shape", [(128, 512, 4096), (128, 4096, 2048), (256, 64, 8192), (1024, 1024, 1024)])
def test_k_split_form_for_skinny_problems(cuda, oracle, shape):
    """gptb_tzgemm_acc: K ranges on different CTAs, partial products reduced into a zeroed C."""
    import ctypes as C

    from tacker_b200 import ops

    M, N, K = shape
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=K)
    A, B = half_dev(cuda, a_bits), half_dev(cuda, b_bits)
    Cd = cuda.zeros((M, N), dtype=cuda.float32, device="cuda")
    ori = ops.OriTZGEMMKernel(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, 1.1, round_dims=False)
    k = ops.GPTBKernel("tzgemm", "gptb_tzgemm_acc", ori, (ops.sm_count(), 1, 1), (192, 1, 1), 0, ori.ori_blks)
    k.execute(cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    _check(oracle, Cd.cpu().numpy(), a, b, 1.1)


def test_bounded_wait_runs_out_and_reports(cuda, oracle):
    """A wait that nothing satisfies ends by itself: with the test hook the producer issues no operand loads, the MMA
    issuer's wait for them expires after the (shortened) budget, the kernel returns with its tensor memory freed, the
    status word names the wait, and the next ordinary launch is correct."""
    import tacker_b200
    from tacker_b200 import ops

    M, N, K = 128, 128, 128
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=77)
    A, B = half_dev(cuda, a_bits), half_dev(cuda, b_bits)
    Cd = cuda.full((M, N), -5.0, dtype=cuda.float32, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    ops.set_option("tzgemm_pair", -1)
    ops.set_option("wait_budget_us", 200)
    ops.set_option("test_skip_loads", 1)
    try:
        k = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), M, N, K, alpha=1.0, grid=1, round_dims=False)
        k.execute(st)
        cuda.cuda.synchronize()                      # the launch ends by itself
        assert ops.get_option("test_skip_loads") == 0
        assert tacker_b200.lib().tk_device_check() == -7     # TK_ERR_DEVICE_WAIT, and the word is cleared
        assert ops.device_status() == 0
        assert bool((Cd == -5.0).all())              # nothing was written
    finally:
        ops.set_option("wait_budget_us", 1000000)
        ops.set_option("test_skip_loads", 0)
        ops.set_option("tzgemm_pair", 0)
    k.execute(st)                                    # the same kernel object, ordinary launch
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    _check(oracle, Cd.cpu().numpy(), a, b, 1.0)
