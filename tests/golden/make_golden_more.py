"""Generates tests/golden/ref_{sgemm,lbm,fft,cutcp}.npz: outputs of the REFERENCE's own persistent-block kernels
(oracle/_ref/libtacker_ref_more.so, built from the reference tree by `make -C oracle ref`) on the seeded inputs
named below, plus report_more.txt: how the CPU restatement compares with them.

Run on a machine with a B200:   python tests/golden/make_golden_more.py [output_dir]
Inputs are not stored; tests/test_golden_more.py regenerates them from the seeds.  The lattice-Boltzmann case has
the reference's compiled-in grid (128^3, 168 MB per array), so its fixture holds a seeded sample of the output and a
checksum of all of it instead of the array.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle"), os.path.join(ROOT, "tests")]

import tacker_oracle as oracle  # noqa: E402
import tacker_ref as ref  # noqa: E402
from helpers import cutcp_inputs, fft_inputs, lbm_inputs, sgemm_inputs  # noqa: E402

CASES = {
    "sgemm": dict(M=256, N=64, K=72, seed=21, start=0, end=8),
    "sgemm_part": dict(M=384, N=48, K=40, seed=22, start=2, end=7),
    "lbm": dict(seed=23, start=0, end=128 * 128),
    "lbm_part": dict(seed=24, start=777, end=5000),
    "fft": dict(nfft=24, seed=25, start=0, end=24),
    "fft_part": dict(nfft=10, seed=26, start=3, end=9),
    "cutcp": dict(n=16, h=0.5, cutoff=12.0, seed=27, nbrlen=0, start=0, end=8),        # nbrlen 0 = the whole list
    "cutcp_256": dict(n=24, h=0.5, cutoff=12.0, seed=28, nbrlen=256, start=1, end=26),  # the length the reference hard-codes
}
LBM_SAMPLES = 20000


def lbm_digest(a: np.ndarray):
    """(xor, sum mod 2^64) of the bit patterns"""
    u = a.view(np.uint32).astype(np.uint64)
    return np.array([np.bitwise_xor.reduce(u), u.sum(dtype=np.uint64)], dtype=np.uint64)


def lbm_sample_index(n: int, seed: int) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, n, size=LBM_SAMPLES)


def main(out_dir):
    import torch

    os.makedirs(out_dir, exist_ok=True)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    report = []
    save = lambda name, **kw: np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"),
                                                  **kw, **{k: np.asarray(v) for k, v in CASES[name].items()})

    for name in ("sgemm", "sgemm_part"):
        c = CASES[name]
        a, b, cm = sgemm_inputs(oracle, c["M"], c["N"], c["K"], seed=c["seed"])
        dA, dB, dC = dev(a), dev(b), dev(cm)
        assert ref.sgemm(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), c["M"], c["N"], c["K"], c["start"], c["end"], 3) == 0
        torch.cuda.synchronize()
        out = dC.cpu().numpy()
        save(name, out=out)
        w = oracle.sgemm_f32(a, b, cm.copy(), c["start"], c["end"])
        report.append(f"{name}: oracle bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}")

    nx, ny, nz, entries = ref.lbm_dims()
    assert entries == oracle.LBM_ENTRIES
    for name in ("lbm", "lbm_part"):
        c = CASES[name]
        src, dst = lbm_inputs(oracle, nx, ny, nz, seed=c["seed"])
        m = oracle.lbm_margin(nx, ny)
        dS, dD = dev(src), dev(dst)
        assert ref.lbm(dS.data_ptr() + 4 * m, dD.data_ptr() + 4 * m, c["start"], c["end"], 148) == 0
        torch.cuda.synchronize()
        out = dD.cpu().numpy()
        idx = lbm_sample_index(out.size, c["seed"])
        save(name, sample=out[idx], digest=lbm_digest(out), dims=np.array([nx, ny, nz]))
        for mode in (1, 0):
            w = oracle.lbm_f32(src, dst.copy(), nx, ny, nz, c["start"], c["end"], contract=mode)
            report.append(f"{name}: oracle contract={mode} bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}, "
                          f"max abs diff {np.abs(out - w).max():.3e}, changed {int((out != dst).sum())}")

    for name in ("fft", "fft_part"):
        c = CASES[name]
        d = fft_inputs(oracle, c["nfft"], seed=c["seed"])
        dd = dev(d)
        assert ref.fft(dd.data_ptr(), c["nfft"], c["start"], c["end"], 3) == 0
        torch.cuda.synchronize()
        out = dd.cpu().numpy()
        save(name, out=out)
        w64 = oracle.fft256_f64(d)
        for mode in (1, 0):
            w = oracle.fft256_f32(d.copy(), c["start"], c["end"], contract=mode)
            report.append(f"{name}: oracle contract={mode} bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}, "
                          f"max abs diff {np.abs(out - w).max():.3e}; reference vs binary64 DFT "
                          f"{np.abs(out[c['start']:c['end']] - w64[c['start']:c['end']]).max():.3e} (max |X| {np.abs(w64).max():.1f})")

    for name in ("cutcp", "cutcp_256"):
        c = CASES[name]
        n, h, cutoff = c["n"], c["h"], c["cutoff"]
        atoms = cutcp_inputs(oracle, n, n, n, h, seed=c["seed"])
        rbins, rnbr, rdims = ref.cutcp_prepare(atoms, n, n, n, h, cutoff)
        dims = oracle.cutcp_bin_dims(n, n, n, h, cutoff)
        nbr = oracle.cutcp_neighbours(h, cutoff)
        bins, extra = oracle.cutcp_bin_atoms(atoms, dims)
        nb = dims[0] * dims[1] * dims[2]
        report.append(f"{name}: bin dims {dims} vs reference {rdims[:4]}; neighbour list {nbr.shape[0]} entries, equal to the "
                      f"reference's {bool((rnbr[:nbr.shape[0]] == nbr).all() and not rnbr[nbr.shape[0]:].any())}; bins equal "
                      f"{bool((rbins[:nb].reshape(bins.shape) == bins).all())}; {extra} of {atoms.shape[0]} atoms found no room")
        use = nbr if c["nbrlen"] == 0 else nbr[:c["nbrlen"]]
        g = (n + 7) // 8
        dB = dev(rbins[:nb])
        dR = torch.zeros((g, g, g, 512), dtype=torch.float32, device="cuda")
        cutoff2 = np.float32(cutoff) * np.float32(cutoff)
        assert ref.cutcp(use, dims[0], dims[1], dims[3], dB.data_ptr(), h, cutoff2, np.float32(1.0) / cutoff2, dR.data_ptr(),
                         g, g, g, c["start"], c["end"], 3) == 0
        torch.cuda.synchronize()
        out = dR.cpu().numpy()
        save(name, out=out)
        for mode in (1, 0):
            w = oracle.cutcp_f32(bins, dims, use, h, cutoff, np.zeros_like(out), g, g, g, c["start"], c["end"], contract=mode)
            report.append(f"{name}: oracle contract={mode} bit mismatches {oracle.bit_mismatches(out, w)} of {out.size}, max abs "
                          f"diff {np.abs(out - w).max():.3e} (max |V| {np.abs(out).max():.3f})")

    print("\n".join(report))
    with open(os.path.join(out_dir, "report_more.txt"), "w") as f:
        f.write("\n".join(report) + "\n")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
