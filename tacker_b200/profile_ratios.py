"""Re-profiles the per-K block ratios of the fused pairs on the GPU at hand and writes them into the model
configuration files (the B200 form of the reference's fusion/gptb_profile/profile.py and
fusion/expr_load_ratio/*.py, whose results are the `"<K>": ratio` tables of src/config/kinfo-*.json).

    python -m tacker_b200.profile_ratios [--write] [--out DIR] [--fill 0.8]

ratio[K] = CUDA-core virtual blocks to co-run per 64x64 tzgemm tile of depth K such that the CUDA-core part
takes `fill` x the time of the GEMM part (both measured solo, per unit): the scheduler's Aker mode takes
tiles x ratio[K] blocks (src/TaskManager.cu:593-598).  The fused launch of that quantum is then timed
against the two solo launches; pairs/K where fusing does not pay get ratio 0 (never fused).
"""
from __future__ import annotations

import argparse
import glob
import json
import os

KS = (128, 512, 1152, 2304, 4096, 4608)  # the K values the reference tabulates
HOST_CONFIG = os.path.join(os.path.dirname(os.path.abspath(__file__)), "host", "config")


def cutcp_problem(nx: int, ny: int, nz: int, h: float = 0.5, cutoff: float = 12.0, density: float = 0.1, seed: int = 0):
    """Synthetic input of the cutoff-Coulomb kernel: atoms at `density` per cubic Angstrom hashed into bins of 4 A
    (8 atoms each, further atoms of a full bin dropped) and the neighbour offsets, as the reference's host code
    prepares them (src/header/cutcp_header.h:106-300).  Returns bins [bz][by][bx][8][4], offsets [n][4], margin c."""
    import numpy as np

    c = int(np.ceil(cutoff / 4.0))
    g = [(v + 7) // 8 for v in (nx, ny, nz)]
    dims = [int(np.ceil(8 * gi * h / 4.0)) + 2 * c for gi in g]                      # x, y, z
    ext = np.array(dims, dtype=np.float64) * 4.0
    rng = np.random.default_rng(seed)
    n = int(density * ext.prod())
    pos = (rng.random((n, 3)) * ext - 4.0 * c).astype(np.float32)
    q = (rng.random(n) * 2 - 1).astype(np.float32)
    q[q == 0] = 0.5
    ijk = np.floor(pos / 4.0).astype(np.int64) + c
    index = (ijk[:, 2] * dims[1] + ijk[:, 1]) * dims[0] + ijk[:, 0]
    order = np.argsort(index, kind="stable")
    index, pos, q = index[order], pos[order], q[order]
    first = np.searchsorted(index, index, side="left")
    rank = np.arange(n) - first
    keep = rank < 8
    bins = np.zeros((dims[2] * dims[1] * dims[0], 8, 4), dtype=np.float32)
    bins[index[keep], rank[keep], :3] = pos[keep]
    bins[index[keep], rank[keep], 3] = q[keep]
    s = np.sqrt(3.0) if (4.0 / (8 * h)).is_integer() else 2 * np.sqrt(3.0)
    r2 = (cutoff + s * 4.0) ** 2
    r = np.arange(-c, c + 1)
    kk, jj, ii = np.meshgrid(r, r, r, indexing="ij")
    ok = (ii * ii + jj * jj + kk * kk) * 16.0 < r2
    nbr = np.stack([ii[ok], jj[ok], kk[ok], np.zeros(ok.sum(), dtype=np.int64)], axis=1).astype(np.int32)
    return bins.reshape(dims[2], dims[1], dims[0], 8, 4), np.ascontiguousarray(nbr), c


def profile(fill: float = 0.8, m: int = 4096, n: int = 4096, only=None) -> dict:
    import numpy as np
    import torch

    from . import ops

    sms = ops.sm_count()
    stream = torch.cuda.Stream()
    st = stream.cuda_stream

    def t_us(kernels, reps=10):
        g = torch.cuda.CUDAGraph()

        def fn():
            for _ in range(reps):
                for k in kernels:
                    k.execute(st)
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(g, stream=stream):
                fn()
            g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record(stream)
            for _ in range(3):
                g.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 3 / reps * 1e3

    # CUDA-core kernels at their headline sizes
    grid0 = torch.rand(64, 512, 512, device="cuda")
    grid1 = grid0.clone()
    atoms = torch.rand(8192, 4, device="cuda") * 64
    packed = torch.empty_like(atoms)
    ops.cp_pack_atoms(atoms.data_ptr(), 8192, 32.0, packed.data_ptr(), st)
    lat = torch.zeros(512, 512, device="cuda")
    kv = torch.rand(2048, 4, device="cuda") - 0.5
    xyz = [torch.rand(262144, device="cuda") * 64 - 32 for _ in range(3)]
    qr, qi = torch.zeros(262144, device="cuda"), torch.zeros(262144, device="cuda")
    fkv = torch.rand(5 * 2048, device="cuda") - 0.5
    fr, fi = torch.zeros(262144, device="cuda"), torch.zeros(262144, device="cuda")
    # solo launch shape (CTAs per SM, threads) and the CUDA-core thread counts tried for the fused kernel
    cds = {
        "stencil": (lambda s=0, e=None: ops.gptb_stencil(1 / 6, 1 / 36, grid0.data_ptr(), grid1.data_ptr(), 512, 512,
                                                         64, start=s, end=e, grid=sms * 2, block=256), 1024,
                    (2, 256), (320, 448, 576)),
        "cp": (lambda s=0, e=None: ops.gptb_cp(8192, 0.125, lat.data_ptr(), packed.data_ptr(), 512, 512, start=s,
                                               end=e, grid=sms * 2, block=512), 256, (2, 512), (448, 576, 832)),
        "mriq": (lambda s=0, e=None: ops.gptb_mriq(2048, xyz[0].data_ptr(), xyz[1].data_ptr(), xyz[2].data_ptr(),
                                                   qr.data_ptr(), qi.data_ptr(), kv.data_ptr(), 262144, start=s,
                                                   end=e, grid=sms * 2, block=512), 1024, (2, 512), (576, 704, 832)),
        "mrif": (lambda s=0, e=None: ops.gptb_mrif(2048, xyz[0].data_ptr(), xyz[1].data_ptr(), xyz[2].data_ptr(),
                                                   fr.data_ptr(), fi.data_ptr(), fkv.data_ptr(), 262144, start=s,
                                                   end=e, grid=sms * 2, block=512), 1024, (2, 512), (576, 704, 832)),
    }
    # the other four at the reference's sizes: sgemm 4096 x 4128 x 4064, lbm 128^3, fft 10240 x 256, cutcp 208 x 208 x 16
    sa, sb = torch.rand(4064, 4096, device="cuda"), torch.rand(4064, 4128, device="cuda")
    sc = torch.zeros(4128, 4096, device="cuda")
    lmargin, lcells = 2 * 128 * 128, 128 ** 3
    lsrc, ldst = torch.rand(20 * lcells + 2 * lmargin, device="cuda"), torch.rand(20 * lcells + 2 * lmargin, device="cuda")
    fdata = torch.rand(10240, 256, 2, device="cuda") * 2 - 1
    cbins, cnbr, cmargin = cutcp_problem(208, 208, 16)
    dbins, dnbr = torch.from_numpy(cbins).cuda(), torch.from_numpy(cnbr).cuda()
    bdz, bdy, bdx = cbins.shape[:3]
    czero = dbins.data_ptr() + 128 * ((cmargin * bdy + cmargin) * bdx + cmargin)
    cregions = torch.zeros(2 * 26 * 26 * 512, device="cuda")
    cds.update({
        "sgemm": (lambda s=0, e=None: ops.gptb_sgemm(sa.data_ptr(), sb.data_ptr(), sc.data_ptr(), 4096, 4128, 4064, start=s,
                                                     end=e, grid=sms * 2, block=256), 32 * 258, (2, 256), (256, 384)),
        "lbm": (lambda s=0, e=None: ops.gptb_lbm(lsrc.data_ptr() + 4 * lmargin, ldst.data_ptr() + 4 * lmargin, 128, 128, 128,
                                                 start=s, end=e, grid=sms * 2, block=512), 128 * 128, (2, 512),
                (576, 832)),
        "fft": (lambda s=0, e=None: ops.gptb_fft(fdata.data_ptr(), 10240, start=s, end=e, grid=sms * 2, block=512), 10240,
                (2, 512), (320, 576, 832)),
        "cutcp": (lambda s=0, e=None: ops.gptb_cutcp(bdx, bdy, czero, 0.5, 144.0, float(np.float32(1.0) / np.float32(144.0)),
                                                     cregions.data_ptr(), dnbr.data_ptr(), cnbr.shape[0], 26, 26, 2, start=s,
                                                     end=e, grid=sms * 2, block=512), 26 * 26 * 2, (2, 512), (576, 832)),
    })
    if only:
        cds = {k: v for k, v in cds.items() if k in only}
    out = {}
    for cd, (mk, blocks, solo_shape, w_sweep) in cds.items():
        if cd == "sgemm":   # per block in the form the fused kernels run (every warp on its own), not the group form
            ops.set_option("sgemm_coop", 0)
        t_block = t_us([mk()], 3) / blocks
        ops.set_option("sgemm_coop", 1)
        # the CUDA-core thread count of the fused kernel: best on a quantum worth one 4096 x 4096 x 1152 GEMM
        a = (torch.rand(m, 1152, device="cuda") * 2 - 1).half()
        b = (torch.rand(n, 1152, device="cuda") * 2 - 1).half()
        c = torch.zeros(m, n, device="cuda")
        tz = ops.gptb_tzgemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, 1152, alpha=1.0, grid=sms)
        nb = max(1, min(blocks, int(fill * t_us([tz]) / t_block)))
        by_w = {w: t_us([ops.mix(mk(0, nb), tz, cd_threads=w, grid=sms)], 5) for w in w_sweep}
        cd_threads = min(by_w, key=by_w.get)
        del a, b, c, tz
        table = {}
        for k in KS:
            kk = max(128, (k // 128) * 128)  # the reference rounds K down to a multiple of 128
            a = (torch.rand(m, kk, device="cuda") * 2 - 1).half()
            b = (torch.rand(n, kk, device="cuda") * 2 - 1).half()
            c = torch.zeros(m, n, device="cuda")
            tz = ops.gptb_tzgemm(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, kk, alpha=1.0, grid=sms)
            tiles = tz.ptb_end_block_pos
            t_gemm = t_us([tz])
            ratio = fill * (t_gemm / tiles) / t_block
            nb = max(1, min(blocks, int(tiles * ratio)))
            t_cd = t_us([mk(0, nb)], 5)
            t_fused = t_us([ops.mix(mk(0, nb), tz, cd_threads=cd_threads, grid=sms)], 5)
            gain = 1.0 - t_fused / (t_gemm + t_cd)
            table[str(k)] = {"ratio": round(ratio if gain > 0.0 else 0.0, 5), "blocks": nb, "gemm_us": round(t_gemm, 2),
                             "cd_us": round(t_cd, 2), "fused_us": round(t_fused, 2),
                             "fused_vs_sequential": round(t_fused / (t_gemm + t_cd), 4)}
        out[f"tzgemm_{cd}"] = {"cd_us_per_block": round(t_block, 4), "cd_threads": cd_threads, "solo_shape": solo_shape,
                               "blocks": blocks,
                               "fused_us_by_cd_threads": {str(w): round(v, 2) for w, v in by_w.items()}, "table": table}
    return out


def write_configs(result: dict, config_dir: str = HOST_CONFIG, out_dir: str | None = None) -> list:
    """Stores the tables in every kinfo-<model>.json of `config_dir` (rewritten in place, or into `out_dir`)."""
    touched = []
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
    for path in sorted(glob.glob(os.path.join(config_dir, "kinfo-*.json"))):
        if path.endswith("kinfo-common.json"):
            continue
        with open(path) as f:
            cfg = json.load(f)
        if out_dir:
            path = os.path.join(out_dir, os.path.basename(path))
        for pair, r in result.items():
            solo = cfg.setdefault(pair[len("tzgemm_"):], {})
            solo["gridsize"], solo["blocksize"] = r["solo_shape"]
            solo["ori_blks"] = r["blocks"]
            entry = cfg.setdefault(pair, {})
            entry["gridsize"] = 1
            entry["blocksize"] = 192 + r["cd_threads"]
            for k, row in r["table"].items():
                entry[k] = row["ratio"]
            entry["block_ratio"] = r["table"]["4096"]["ratio"]
            entry["best_block_ratio"] = max(row["ratio"] for row in r["table"].values())
        with open(path, "w") as f:
            json.dump(cfg, f, indent=4)
            f.write("\n")
        touched.append(path)
    return touched


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--write", action="store_true", help="store the ratios in tacker_b200/host/config/kinfo-*.json")
    ap.add_argument("--out", default=None, help="with --write: put the updated files there instead of rewriting in place")
    ap.add_argument("--fill", type=float, default=0.8)
    ap.add_argument("--only", default=None, help="comma-separated CUDA-core kernels to profile (default: all eight)")
    args = ap.parse_args(argv)
    result = profile(args.fill, only=args.only.split(",") if args.only else None)
    print(json.dumps(result, indent=1))
    if args.write:
        for p in write_configs(result, out_dir=args.out):
            print("updated", p)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
