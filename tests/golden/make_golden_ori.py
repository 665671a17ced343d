"""Generates tests/golden/ref_ori.npz: outputs of the REFERENCE's unfused, non-persistent kernels ori_stencil, ori_cp,
ori_mriq, ori_mrif, ori_sgemm, ori_lbm, ori_fft and ori_cutcp (oracle/_ref/libtacker_ref_ori.so, built from the
reference tree by `make -C oracle ref`) on the seeded inputs of make_golden.py / make_golden_more.py (whole launches),
plus report_ori.txt: how they compare with the persistent-block forms pinned in ref_<name>.npz.

Run on a machine with a B200, after the two other generators:   python tests/golden/make_golden_ori.py [output_dir]
tests/test_golden_ori.py recomputes every case on the CPU from the seeds and compares.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests"), HERE]

import tacker_oracle as oracle  # noqa: E402
import tacker_ref as ref  # noqa: E402
from helpers import (coulomb_inputs, cutcp_inputs, fft_inputs, lbm_inputs, mrif_inputs, mriq_inputs, sgemm_inputs,  # noqa: E402
                     stencil_inputs)
from make_golden import CASES as CASES_A  # noqa: E402
from make_golden_more import CASES as CASES_B, lbm_digest, lbm_sample_index  # noqa: E402


def main(out_dir):
    import torch

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out, report = {}, []

    def pinned(name):
        g = np.load(os.path.join(HERE, f"ref_{name}.npz"))
        return {k: g[k] for k in g.files}

    def compare(name, key, got, want):
        report.append(f"{name}: ori_{key} vs the persistent-block form: bit mismatches {oracle.bit_mismatches(got, want)} of "
                      f"{got.size}, max abs diff {np.abs(got - want).max():.3e}")

    for name in ("stencil", "stencil_cfg2coef"):
        c = CASES_A[name]
        A0 = stencil_inputs(oracle, c["nx"], c["ny"], c["nz"], seed=c["seed"])
        d0, d1 = dev(A0), dev(A0)
        assert ref.ori_stencil(c["c0"], c["c1"], d0.data_ptr(), d1.data_ptr(), c["nx"], c["ny"], c["nz"]) == 0
        torch.cuda.synchronize()
        out[name] = d1.cpu().numpy()
        compare(name, "stencil", out[name], pinned(name)["out"])

    for name in ("cp", "cp_cfg3spacing"):
        c = CASES_A[name]
        atoms = coulomb_inputs(oracle, c["natoms"], c["box"], seed=c["seed"], spacing=c["spacing"], zplane=c["zplane"])
        packed = oracle.cp_pack_atoms(atoms, c["zplane"])
        gx, gy = oracle.cp_grid(c["nx"], c["ny"])
        lat = torch.zeros((c["ny"], c["nx"]), dtype=torch.float32, device="cuda")
        assert ref.ori_cp(packed, c["spacing"], lat.data_ptr(), gx, gy) == 0
        torch.cuda.synchronize()
        out[name] = lat.cpu().numpy()
        compare(name, "cp", out[name], pinned(name)["out"])

    c = CASES_A["mriq"]
    k, phi, xyz = mriq_inputs(oracle, c["numK"], c["numX"], seed=c["seed"])
    kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
    dx = [dev(xyz[i]) for i in range(3)]
    qr = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    qi = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    assert ref.ori_mriq(kv, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(), c["numX"]) == 0
    torch.cuda.synchronize()
    out["mriq_qr"], out["mriq_qi"] = qr.cpu().numpy(), qi.cpu().numpy()
    compare("mriq", "mriq Qr", out["mriq_qr"], pinned("mriq")["qr"])
    compare("mriq", "mriq Qi", out["mriq_qi"], pinned("mriq")["qi"])

    c = CASES_A["mrif"]
    k, phi, d, xyz = mrif_inputs(oracle, c["numK"], c["numX"], seed=c["seed"])
    kv = oracle.mrif_pack(k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])
    nk = c["numK"]
    aos = np.concatenate([kv[:4 * nk].reshape(nk, 4), kv[4 * nk:].reshape(nk, 1)], axis=1)   # the reference's struct order
    dx = [dev(xyz[i]) for i in range(3)]
    o_r = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    o_i = torch.zeros(c["numX"], dtype=torch.float32, device="cuda")
    assert ref.ori_mrif(aos, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), o_r.data_ptr(), o_i.data_ptr(), c["numX"]) == 0
    torch.cuda.synchronize()
    out["mrif_r"], out["mrif_i"] = o_r.cpu().numpy(), o_i.cpu().numpy()
    compare("mrif", "mrif outR", out["mrif_r"], pinned("mrif")["outR"])
    compare("mrif", "mrif outI", out["mrif_i"], pinned("mrif")["outI"])

    c = CASES_B["sgemm"]
    a, b, cm = sgemm_inputs(oracle, c["M"], c["N"], c["K"], seed=c["seed"])
    dA, dB, dC = dev(a), dev(b), dev(cm)
    assert ref.ori_sgemm(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), c["M"], c["N"], c["K"]) == 0
    torch.cuda.synchronize()
    out["sgemm"] = dC.cpu().numpy()
    compare("sgemm", "sgemm", out["sgemm"], pinned("sgemm")["out"])

    nx, ny, nz, _ = ref.lbm_dims()
    c = CASES_B["lbm"]
    src, dst = lbm_inputs(oracle, nx, ny, nz, seed=c["seed"])
    m = oracle.lbm_margin(nx, ny)
    dS, dD = dev(src), dev(dst)
    assert ref.ori_lbm(dS.data_ptr() + 4 * m, dD.data_ptr() + 4 * m) == 0
    torch.cuda.synchronize()
    full = dD.cpu().numpy()
    out["lbm_sample"], out["lbm_digest"] = full[lbm_sample_index(full.size, c["seed"])], lbm_digest(full)
    p = pinned("lbm")
    report.append(f"lbm: ori_lbm vs the persistent-block form: digest equal {bool((out['lbm_digest'] == p['digest']).all())}, "
                  f"sample bit mismatches {oracle.bit_mismatches(out['lbm_sample'], p['sample'])} of {out['lbm_sample'].size}")

    c = CASES_B["fft"]
    d = fft_inputs(oracle, c["nfft"], seed=c["seed"])
    dd = dev(d)
    assert ref.ori_fft(dd.data_ptr(), c["nfft"]) == 0
    torch.cuda.synchronize()
    out["fft"] = dd.cpu().numpy()
    compare("fft", "fft", out["fft"], pinned("fft")["out"])

    c = CASES_B["cutcp"]
    n, h, cutoff = c["n"], c["h"], c["cutoff"]
    atoms = cutcp_inputs(oracle, n, n, n, h, seed=c["seed"])
    rbins, _, _ = ref.cutcp_prepare(atoms, n, n, n, h, cutoff)
    dims = oracle.cutcp_bin_dims(n, n, n, h, cutoff)
    nbr = oracle.cutcp_neighbours(h, cutoff)
    nb = dims[0] * dims[1] * dims[2]
    g = (n + 7) // 8
    dB = dev(rbins[:nb])
    dR = torch.zeros((g, g, g, 512), dtype=torch.float32, device="cuda")
    cutoff2 = np.float32(cutoff) * np.float32(cutoff)
    assert ref.ori_cutcp(nbr, dims[0], dims[1], dims[3], dB.data_ptr(), h, cutoff2, np.float32(1.0) / cutoff2, dR.data_ptr(),
                         g, g, g) == 0
    torch.cuda.synchronize()
    out["cutcp"] = dR.cpu().numpy()
    compare("cutcp", "cutcp", out["cutcp"], pinned("cutcp")["out"])

    np.savez_compressed(os.path.join(out_dir, "ref_ori.npz"), **out)
    print("\n".join(report))
    with open(os.path.join(out_dir, "report_ori.txt"), "w") as f:
        f.write("\n".join(report) + "\n")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
