"""Shared input builders for the parity tests (seeded through the oracle's counter RNG)."""
import numpy as np


def to_dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def half_dev(torch, bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.float16)).cuda()


def gemm_inputs(oracle, M, N, K, seed=0):
    a_bits, a = oracle.uniform_f16(M * K, 2 * seed + 11, -1.0, 1.0)
    b_bits, b = oracle.uniform_f16(N * K, 2 * seed + 12, -1.0, 1.0)
    return a_bits.reshape(M, K), a.reshape(M, K), b_bits.reshape(N, K), b.reshape(N, K)


def stencil_inputs(oracle, nx, ny, nz, seed=0):
    return oracle.uniform_f32(nx * ny * nz, 100 + seed, 0.0, 1.0).reshape(nz, ny, nx)


def coulomb_inputs(oracle, natoms, box, seed=0, spacing=0.125, zplane=32.0, min_dist=0.05):
    """atoms {x,y,z,q}: positions uniform in [0,box)^3, charges uniform in [-1,1].  Atoms closer than
    `min_dist` to a lattice point of the slice are pushed off the plane so that 1/r stays well scaled."""
    pos = oracle.uniform_f32(natoms * 3, 200 + seed, 0.0, box).reshape(natoms, 3)
    q = oracle.uniform_f32(natoms, 300 + seed, -1.0, 1.0)
    atoms = np.concatenate([pos, q[:, None]], axis=1).astype(np.float32)
    gxy = np.round(atoms[:, :2] / spacing) * spacing
    d = np.sqrt(((atoms[:, :2] - gxy) ** 2).sum(1) + (atoms[:, 2] - zplane) ** 2)
    near = d < min_dist
    atoms[near, 2] = zplane + 4 * min_dist
    return np.ascontiguousarray(atoms)


def mriq_inputs(oracle, numK, numX, seed=0):
    k = oracle.uniform_f32(3 * numK, 400 + seed, -0.5, 0.5).reshape(3, numK)
    phi = oracle.uniform_f32(2 * numK, 500 + seed, 0.0, 1.0).reshape(2, numK)
    xyz = oracle.uniform_f32(3 * numX, 600 + seed, -32.0, 32.0).reshape(3, numX)
    return k, phi, xyz


def mrif_inputs(oracle, numK, numX, seed=0):
    """k-space samples, phi and d (real / imaginary, uniform in [-1, 1)), voxel coordinates in [-32, 32)^3."""
    k = oracle.uniform_f32(3 * numK, 700 + seed, -0.5, 0.5).reshape(3, numK)
    phi = oracle.uniform_f32(2 * numK, 800 + seed, -1.0, 1.0).reshape(2, numK)
    d = oracle.uniform_f32(2 * numK, 900 + seed, -1.0, 1.0).reshape(2, numK)
    xyz = oracle.uniform_f32(3 * numX, 1000 + seed, -32.0, 32.0).reshape(3, numX)
    return k, phi, d, xyz


def sgemm_inputs(oracle, M, N, K, seed=0):
    """A [K][M], B [K][N], C [N][M] (the reference's layouts), uniform in [0, 1) like its curand fill"""
    a = oracle.uniform_f32(K * M, 1100 + seed, 0.0, 1.0).reshape(K, M)
    b = oracle.uniform_f32(K * N, 1200 + seed, 0.0, 1.0).reshape(K, N)
    c = oracle.uniform_f32(N * M, 1300 + seed, 0.0, 1.0).reshape(N, M)
    return a, b, c


def lbm_inputs(oracle, nx, ny, nz, seed=0):
    """Source and destination grids with their margins, uniform in [0, 1) like the reference's curand fill; the flag
    element is a random bit pattern too (about half of the cells obstacles), as it is there."""
    n = 2 * oracle.lbm_margin(nx, ny) + oracle.LBM_ENTRIES * nx * ny * nz
    src = oracle.uniform_f32(n, 1400 + seed, 0.0, 1.0)
    dst = oracle.uniform_f32(n, 1500 + seed, 0.0, 1.0)
    return src, dst


def fft_inputs(oracle, nfft, seed=0):
    return oracle.uniform_f32(nfft * 512, 1600 + seed, -1.0, 1.0).reshape(nfft, 256, 2)


def cutcp_inputs(oracle, nx, ny, nz, h, seed=0, density=0.1, pad=4.0):
    """atoms {x, y, z, q} at about one per 10 cubic Angstrom in the box of the lattice plus `pad` on every side,
    charges uniform in [-1, 1) and never zero"""
    ext = np.array([nx, ny, nz], dtype=np.float64) * h
    natoms = int(np.prod(ext + 2 * pad) * density)
    pos = oracle.uniform_f32(natoms * 3, 1700 + seed, 0.0, 1.0).reshape(natoms, 3)
    pos = (pos * (ext + 2 * pad) - pad).astype(np.float32)
    q = oracle.uniform_f32(natoms, 1800 + seed, -1.0, 1.0)
    q[q == 0] = 0.5
    return np.ascontiguousarray(np.concatenate([pos, q[:, None]], axis=1).astype(np.float32))


def lbm_conflicts(oracle, nx, ny, nz, start=0, end=None):
    """Boolean mask over the full lattice-Boltzmann array (margins included): addresses that two cells of the block
    range write.  The layout keeps the 20 elements back to back without gaps, so a value sent across the top face
    of element e lands in element e + 1 where a value sent across the bottom face also lands; the reference has the
    same two writers and no order between them."""
    cells = nx * ny * nz
    m = oracle.lbm_margin(nx, ny)
    if end is None:
        end = ny * nz
    dx = [0, 0, 0, 1, -1, 0, 0, 1, -1, 1, -1, 0, 0, 0, 0, 1, 1, -1, -1]
    dy = [0, 1, -1, 0, 0, 0, 0, 1, 1, -1, -1, 1, 1, -1, -1, 0, 0, 0, 0]
    dz = [0, 0, 0, 0, 0, 1, -1, 0, 0, 0, 0, 1, -1, 1, -1, 1, -1, 1, -1]
    rows = np.arange(start, end)
    cell = ((rows % ny) * nx + (rows // ny % nz) * nx * ny)[:, None] + np.arange(nx)[None, :]
    count = np.zeros(2 * m + 20 * cells, dtype=np.int32)
    for e in range(19):
        np.add.at(count, m + e * cells + cell.ravel() + dx[e] + dy[e] * nx + dz[e] * nx * ny, 1)
    return count > 1
