"""Generates tests/golden/ref_*.npz: outputs of the REFERENCE's own kernels (oracle/_ref, built from
the reference tree by `make -C oracle ref`) on the seeded inputs named below.

Run on a machine with a B200 (or any GPU the sm_100 build runs on):
    python tests/golden/make_golden.py [output_dir]
The fixtures pin the CPU restatement (oracle/tacker_oracle.c): tests/test_golden.py recomputes every
case on the CPU and compares.  Inputs are not stored; they are regenerated from the seeds.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")]

import tacker_oracle as oracle  # noqa: E402
import tacker_ref as ref  # noqa: E402
from helpers import coulomb_inputs, gemm_inputs, mrif_inputs, mriq_inputs, stencil_inputs  # noqa: E402

CASES = {
    "stencil": dict(nx=192, ny=12, nz=7, c0=1.0 / 6.0, c1=1.0 / 36.0, seed=11),
    "stencil_cfg2coef": dict(nx=128, ny=8, nz=6, c0=1.0 / 6.0, c1=-1.0 / 6.0, seed=12),
    "cp": dict(nx=128, ny=16, natoms=130, spacing=0.1, zplane=0.0, box=12.0, seed=13),
    "cp_cfg3spacing": dict(nx=128, ny=8, natoms=64, spacing=0.125, zplane=4.0, box=8.0, seed=14),
    "mriq": dict(numK=96, numX=512, seed=15),
    "mrif": dict(numK=300, numX=512, seed=16),
    "tzgemm": dict(M=128, N=128, K=256, seed=16),
}


def main(out_dir):
    import torch

    os.makedirs(out_dir, exist_ok=True)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    report = []

    for name in ("stencil", "stencil_cfg2coef"):
        c = CASES[name]
        A0 = stencil_inputs(oracle, c["nx"], c["ny"], c["nz"], seed=c["seed"])
        gx, gy = oracle.stencil_grid(c["nx"], c["ny"])
        d0, d1 = dev(A0), dev(A0)
        assert ref.stencil(c["c0"], c["c1"], d0.data_ptr(), d1.data_ptr(), c["nx"], c["ny"], c["nz"], 0, gx * gy, 3) == 0
        torch.cuda.synchronize()
        out = d1.cpu().numpy()
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), out=out, **{k: np.asarray(v) for k, v in c.items()})
        for mode in (0, 1, 2):
            w = oracle.stencil_sweep_f32(np.float32(c["c0"]), np.float32(c["c1"]), A0, A0.copy(), contract=mode)
            report.append(f"{name}: oracle contract={mode} bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}")

    for name in ("cp", "cp_cfg3spacing"):
        c = CASES[name]
        atoms = coulomb_inputs(oracle, c["natoms"], c["box"], seed=c["seed"], spacing=c["spacing"], zplane=c["zplane"])
        packed = oracle.cp_pack_atoms(atoms, c["zplane"])
        gx, gy = oracle.cp_grid(c["nx"], c["ny"])
        lat = torch.zeros((c["ny"], c["nx"]), dtype=torch.float32, device="cuda")
        assert ref.cp(packed, c["spacing"], lat.data_ptr(), gx, gy, 0, gx * gy, 2) == 0
        torch.cuda.synchronize()
        out = lat.cpu().numpy()
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), out=out, **{k: np.asarray(v) for k, v in c.items()})
        w = oracle.cp_f32(packed, c["spacing"], np.zeros_like(out), chunk=64)
        report.append(f"{name}: oracle f32 bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}, "
                      f"max abs diff {np.abs(out - w).max():.3e}")

    c = CASES["mriq"]
    k, phi, xyz = mriq_inputs(oracle, c["numK"], c["numX"], seed=c["seed"])
    kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
    dx = [dev(xyz[i]) for i in range(3)]
    qr = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    qi = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    gx = c["numX"] // 256
    assert ref.mriq(kv, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(), gx, 0, gx, 2) == 0
    torch.cuda.synchronize()
    out_r, out_i = qr.cpu().numpy(), qi.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ref_mriq.npz"), qr=out_r, qi=out_i, **{k_: np.asarray(v) for k_, v in c.items()})
    wr, wi = oracle.mriq_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(c["numX"], np.float32), np.zeros(c["numX"], np.float32))
    scale = float(kv[:, 3].sum())
    report.append(f"mriq: oracle f32 vs reference max abs diff Qr {np.abs(out_r - wr).max():.3e} Qi "
                  f"{np.abs(out_i - wi).max():.3e} (sum phiMag {scale:.3f}, max |Q| {np.abs(wr).max():.3f})")

    c = CASES["mrif"]
    k, phi, d, xyz = mrif_inputs(oracle, c["numK"], c["numX"], seed=c["seed"])
    kv = oracle.mrif_pack(k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])
    nk = c["numK"]
    aos = np.concatenate([kv[:4 * nk].reshape(nk, 4), kv[4 * nk:].reshape(nk, 1)], axis=1)   # the reference's struct order
    dx = [dev(xyz[i]) for i in range(3)]
    o_r = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    o_i = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    gx = c["numX"] // 256
    assert ref.mrif(aos, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), o_r.data_ptr(), o_i.data_ptr(), gx, 0, gx, 2) == 0
    torch.cuda.synchronize()
    out_r, out_i = o_r.cpu().numpy(), o_i.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ref_mrif.npz"), outR=out_r, outI=out_i,
                        **{k_: np.asarray(v) for k_, v in c.items()})
    for mode in (0, 1):
        wr, wi = oracle.mrif_f32(kv, xyz[0], xyz[1], xyz[2], np.zeros(c["numX"], np.float32),
                                 np.zeros(c["numX"], np.float32), mode=mode)
        report.append(f"mrif: oracle f32 (contraction mode {mode}) vs reference: bit mismatches outR "
                      f"{oracle.bit_mismatches(out_r, wr)} outI {oracle.bit_mismatches(out_i, wi)} of {out_r.size}, max abs "
                      f"diff {max(np.abs(out_r - wr).max(), np.abs(out_i - wi).max()):.3e} (max |out| {np.abs(wr).max():.3f})")

    c = CASES["tzgemm"]
    a_bits, a, b_bits, b = gemm_inputs(oracle, c["M"], c["N"], c["K"], seed=c["seed"])
    A = torch.from_numpy(a_bits.view(np.float16)).cuda()
    B = torch.from_numpy(b_bits.view(np.float16)).cuda()
    Cd = torch.zeros((c["M"], c["N"]), dtype=torch.float32, device="cuda")
    tiles = (c["M"] // 64) * (c["N"] // 64)
    assert ref.tzgemm(A.data_ptr(), B.data_ptr(), Cd.data_ptr(), c["M"], c["N"], c["K"], 0, tiles, 2) == 0
    torch.cuda.synchronize()
    out = Cd.cpu().numpy()
    np.savez_compressed(os.path.join(out_dir, "ref_tzgemm.npz"), out=out, alpha=np.asarray(ref.alpha()),
                        **{k_: np.asarray(v) for k_, v in c.items()})
    w = oracle.tzgemm_f64(a, b, alpha=ref.alpha())
    report.append(f"tzgemm: reference alpha {ref.alpha()}, max abs diff vs oracle f64 {np.abs(out - w).max():.3e}")

    print("\n".join(report))
    with open(os.path.join(out_dir, "report.txt"), "w") as f:
        f.write("\n".join(report) + "\n")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
