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
