"""Work-distribution invariants of the persistent kernels, checked exhaustively on the CPU: every virtual
block of [start, end) is executed exactly once, nothing outside it is touched, for any grid size."""
import ctypes as C

import numpy as np
import pytest


@pytest.fixture(scope="module")
def lib():
    import tacker_b200
    from tacker_b200 import _build

    _build.build_library()
    return tacker_b200.lib()


def _p(a):
    return a.ctypes.data_as(C.POINTER(C.c_int))


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("shape", [(128, 64), (128, 128), (256, 384), (384, 320), (1024, 1024), (128, 896)])
def test_tzgemm_plan_covers_each_tile_of_the_range_exactly_once(lib, bn, shape):
    M, N = shape
    tiles = (M // 64) * (N // 64)
    rng = np.random.default_rng(M + N + bn)
    ranges = [(0, tiles), (0, 1), (tiles - 1, tiles), (3, 3), (0, tiles + 50)]
    ranges += [tuple(sorted(rng.integers(0, tiles + 1, 2))) for _ in range(12)]
    for start, end in ranges:
        for ctas in (1, 2, 3, 5, 148):
            cover = np.zeros(tiles, dtype=np.int32)
            work = np.zeros(ctas, dtype=np.int32)
            assert lib.tk_plan_tzgemm(M, N, bn, int(start), int(end), ctas, _p(cover), _p(work)) == 0
            want = np.zeros(tiles, dtype=np.int32)
            want[int(start):min(int(end), tiles)] = 1
            assert np.array_equal(cover, want), (shape, bn, start, end, ctas)
            if ctas == 1:
                assert work[0] >= (want.sum() + (bn // 64) * 2 - 1) // ((bn // 64) * 2)   # at least tiles / tiles-per-super-tile


def test_tzgemm_plan_rejects_bad_shapes(lib):
    cover = np.zeros(16, dtype=np.int32)
    assert lib.tk_plan_tzgemm(100, 128, 128, 0, 1, 1, _p(cover), None) == -1
    assert lib.tk_plan_tzgemm(128, 128, 64, 0, 1, 1, _p(cover), None) == -1


@pytest.mark.parametrize("nz", [3, 4, 10, 64, 65])
@pytest.mark.parametrize("launch", [(1, 1), (2, 3), (148, 8), (148, 16), (296, 8), (7, 5)])
def test_stencil_plan_computes_each_interior_plane_once(lib, nz, launch):
    ctas, warps = launch
    gx, gy = 3, 5
    blocks = gx * gy
    for start, end in ((0, blocks), (2, 9), (14, 15), (4, 4), (5, 40)):
        planes = np.zeros(blocks * nz, dtype=np.int32)
        loads = np.zeros(blocks * nz, dtype=np.int32)
        split = (C.c_int * 2)()
        assert lib.tk_plan_stencil(nz, start, end, gx, gy, ctas, warps, _p(planes), _p(loads), split) == 0
        planes, loads = planes.reshape(blocks, nz), loads.reshape(blocks, nz)
        want = np.zeros((blocks, nz), dtype=np.int32)
        want[start:min(end, blocks), 1:nz - 1] = 1
        assert np.array_equal(planes, want), (nz, launch, start, end)
        if end > start:
            slabs, per = split[0], split[1]
            assert slabs * per >= nz - 2 and (slabs - 1) * per < nz - 2
            # every item streams its planes plus one halo plane on each side, nothing else
            assert loads[start:min(end, blocks)].sum() == (min(end, blocks) - start) * ((nz - 2) + 2 * slabs)
            assert loads[:start].sum() == 0 and loads[min(end, blocks):].sum() == 0


def test_stencil_split_fills_the_launched_warps(lib):
    # 1024 bundles of 62 planes on 148 x 16 warps: two slabs per bundle = one round of 2048 items
    split = (C.c_int * 2)()
    planes = np.zeros(1024 * 64, dtype=np.int32)
    assert lib.tk_plan_stencil(64, 0, 1024, 8, 128, 148, 16, _p(planes), None, split) == 0
    assert (split[0], split[1]) == (2, 31)
    assert lib.tk_plan_stencil(64, 0, 1024, 8, 128, 1, 1, _p(planes), None, split) == 0
    assert (split[0], split[1]) == (1, 62)          # one warp: no reason to pay for extra halo planes


@pytest.mark.parametrize("shape", [(128, 64), (256, 256), (384, 320), (1024, 1024), (128, 896), (640, 1280)])
def test_tzgemm_m256_plan_covers_each_tile_of_the_range_exactly_once(lib, shape):
    M, N = shape
    tiles = (M // 64) * (N // 64)
    rng = np.random.default_rng(7 * M + N)
    ranges = [(0, tiles), (0, 1), (tiles - 1, tiles), (2, 2), (0, tiles + 9)]
    ranges += [tuple(sorted(rng.integers(0, tiles + 1, 2))) for _ in range(12)]
    for start, end in ranges:
        for ctas in (1, 3, 148):
            cover = np.zeros(tiles, dtype=np.int32)
            assert lib.tk_plan_tzgemm_m256(M, N, int(start), int(end), ctas, _p(cover)) == 0
            want = np.zeros(tiles, dtype=np.int32)
            want[int(start):min(int(end), tiles)] = 1
            assert np.array_equal(cover, want), (shape, start, end, ctas)
