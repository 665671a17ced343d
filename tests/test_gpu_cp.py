"""Coulomb direct summation through the C ABI against the CPU checker (B200 only).

exact mode (IEEE 1/sqrt, the reference's arithmetic) is bit-exact against the binary32
restatement; the default mode (hardware rsqrt) is held to 1e-5 of sum_a |q_a|/r_a per lattice
point and to 1e-5 of the largest potential, both against the binary32 restatement (the
reference's semantics) and, point-wise scaled, against binary64.
"""
import numpy as np
import pytest

from helpers import coulomb_inputs, to_dev

pytestmark = pytest.mark.gpu


def _run(torch, ops, atoms, zplane, h, nx, ny, base=None, start=0, end=None, grid=None, block=256):
    n = atoms.shape[0]
    raw = to_dev(torch, atoms)
    packed = torch.empty_like(raw)
    lat = to_dev(torch, np.zeros((ny, nx), np.float32) if base is None else base)
    st = torch.cuda.current_stream().cuda_stream
    ops.cp_pack_atoms(raw.data_ptr(), n, zplane, packed.data_ptr(), st)
    ops.gptb_cp(n, h, lat.data_ptr(), packed.data_ptr(), nx, ny, start=start, end=end, grid=grid,
                block=block).execute(st)
    torch.cuda.synchronize()
    return lat.cpu().numpy(), packed.cpu().numpy()


@pytest.mark.parametrize("ppt", [8, 4, 2])
@pytest.mark.parametrize("natoms", [1, 64, 65, 200])
def test_exact_mode_bit_exact(cuda, oracle, ppt, natoms):
    from tacker_b200 import ops

    nx, ny, h, z = 256, 16, 0.1, 0.0              # reference spacing and plane (src/ori_kernel/cp_kernel.cu:276,302)
    atoms = coulomb_inputs(oracle, natoms, 12.0, seed=natoms, spacing=h, zplane=z)
    ops.set_option("cp_exact", 1)
    ops.set_option("cp_ppt", ppt)
    try:
        base = oracle.uniform_f32(nx * ny, 77, -1.0, 1.0).reshape(ny, nx)
        got, packed = _run(cuda, ops, atoms, z, h, nx, ny, base=base, grid=3, block=96)
    finally:
        ops.set_option("cp_exact", 0)
        ops.set_option("cp_ppt", 8)
    assert oracle.bit_mismatches(packed, oracle.cp_pack_atoms(atoms, z)) == 0
    want = oracle.cp_f32(oracle.cp_pack_atoms(atoms, z), h, base.copy(), chunk=64)
    assert oracle.bit_mismatches(got, want) == 0


@pytest.mark.parametrize("ppt", [8, 4, 2])
def test_fast_mode_within_tolerance(cuda, oracle, ppt):
    from tacker_b200 import ops

    nx, ny, h, z = 512, 64, 0.125, 32.0
    atoms = coulomb_inputs(oracle, 1000, 64.0, seed=5, spacing=h, zplane=z)
    ops.set_option("cp_ppt", ppt)
    try:
        got, _ = _run(cuda, ops, atoms, z, h, nx, ny)
    finally:
        ops.set_option("cp_ppt", 8)
    packed = oracle.cp_pack_atoms(atoms, z)
    ref32 = oracle.cp_f32(packed, h, np.zeros((ny, nx), np.float32), chunk=64)
    ref64, mag = oracle.cp_f64(packed, h, nx, ny)
    assert (np.abs(got - ref32) / mag).max() <= 1e-5
    assert np.abs(got - ref32).max() <= 1e-5 * np.abs(ref32).max()
    assert oracle.max_scaled_err(got, ref64, mag) <= 1e-5


@pytest.mark.parametrize("split", [64, 128, 0, -1])
@pytest.mark.parametrize("natoms", [1, 64, 65, 200, 1000])
def test_atom_split_items(cuda, oracle, split, natoms):
    """Work items that cover a range of the atom list and add their partial sums with reductions: same result
    within the tolerance for every split (including ragged last ranges), accumulating onto a non-zero lattice,
    inside a virtual-block range only."""
    from tacker_b200 import ops

    nx, ny, h, z = 256, 32, 0.125, 3.0            # 2 x 4 patches
    atoms = coulomb_inputs(oracle, natoms, 24.0, seed=100 + natoms, spacing=h, zplane=z)
    base = oracle.uniform_f32(nx * ny, 78, -1.0, 1.0).reshape(ny, nx)
    ops.set_option("cp_split", split)
    try:
        got, _ = _run(cuda, ops, atoms, z, h, nx, ny, base=base, start=1, end=7, grid=5, block=160)
    finally:
        ops.set_option("cp_split", -1)
    packed = oracle.cp_pack_atoms(atoms, z)
    ref32 = oracle.cp_f32(packed, h, base.copy(), start=1, end=7, chunk=64)
    _, mag = oracle.cp_f64(packed, h, nx, ny, start=1, end=7)
    touched = mag > 0
    assert np.array_equal(got[~touched], base[~touched])
    assert (np.abs(got - ref32)[touched] / (mag[touched] + np.abs(base[touched]))).max() <= 1e-5


@pytest.mark.parametrize("rng", [(0, 1), (3, 4), (1, 6), (0, 8), (7, 8), (2, 2), (5, 20)])
def test_virtual_block_range_is_exact(cuda, oracle, rng):
    from tacker_b200 import ops

    nx, ny, h, z = 256, 32, 0.125, 1.0            # 2 x 4 patches of 128 x 8
    start, end = rng
    atoms = coulomb_inputs(oracle, 70, 16.0, seed=1, spacing=h, zplane=z)
    ops.set_option("cp_exact", 1)
    try:
        got, _ = _run(cuda, ops, atoms, z, h, nx, ny, start=start, end=end, grid=2, block=64)
    finally:
        ops.set_option("cp_exact", 0)
    want = oracle.cp_f32(oracle.cp_pack_atoms(atoms, z), h, np.zeros((ny, nx), np.float32), start=start,
                         end=min(end, 8), chunk=64)
    assert oracle.bit_mismatches(got, want) == 0


def test_config3_full_size(cuda, oracle):
    """8192 atoms in a 64 A cube, 512 x 512 lattice, spacing 0.125 A, slice z = 32 A."""
    from tacker_b200 import ops

    nx = ny = 512
    h, z = 0.125, 32.0
    atoms = coulomb_inputs(oracle, 8192, 64.0, seed=0, spacing=h, zplane=z)
    got, _ = _run(cuda, ops, atoms, z, h, nx, ny)
    packed = oracle.cp_pack_atoms(atoms, z)
    # full binary64 reference on 16 of the 256 patches (2 x 8 rows of the lattice), all atoms
    blocks = [0, 3, 17, 50, 64, 99, 128, 131, 160, 190, 200, 222, 233, 240, 252, 255]
    worst = 0.0
    for p in blocks:
        ref64, mag = oracle.cp_f64(packed, h, nx, ny, start=p, end=p + 1)
        by, bx = p // 4, p % 4
        sl = (slice(by * 8, by * 8 + 8), slice(bx * 128, bx * 128 + 128))
        worst = max(worst, float((np.abs(got[sl] - ref64[sl]) / mag[sl]).max()))
    assert worst <= 1e-5
    # linearity: the potential of all atoms equals the sum over two disjoint halves (separate launches)
    lo, _ = _run(cuda, ops, atoms[:4096], z, h, nx, ny)
    hi, _ = _run(cuda, ops, atoms[4096:], z, h, nx, ny)
    assert np.abs(lo + hi - got).max() <= 1e-5 * np.abs(got).max()
    assert np.isfinite(got).all()


def test_zero_atoms_and_errors(cuda):
    import ctypes as C

    from tacker_b200 import ops

    lat = cuda.full((8, 128), 2.5, dtype=cuda.float32, device="cuda")
    ops.gptb_cp(0, 0.1, lat.data_ptr(), 0, 128, 8).execute()
    cuda.cuda.synchronize()
    assert bool((lat == 2.5).all())
    p = [C.c_int(4), C.c_float(0.1), C.c_void_p(lat.data_ptr()), C.c_void_p(lat.data_ptr() + 4)] + \
        [C.c_int(v) for v in (1, 1, 1, 16, 8, 1, 0, 1, 1, 0)]
    assert ops.raw_launch("gptb_cp", p, (1, 1, 1), (128, 1, 1)) == -2          # atoms not 16-byte aligned
    p[3] = C.c_void_p(0)
    assert ops.raw_launch("gptb_cp", p, (1, 1, 1), (128, 1, 1)) == -1          # atoms missing
