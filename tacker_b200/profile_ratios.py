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


def profile(fill: float = 0.8, m: int = 4096, n: int = 4096) -> dict:
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
    out = {}
    for cd, (mk, blocks, solo_shape, w_sweep) in cds.items():
        t_block = t_us([mk()], 3) / blocks
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
    args = ap.parse_args(argv)
    result = profile(args.fill)
    print(json.dumps(result, indent=1))
    if args.write:
        for p in write_configs(result, out_dir=args.out):
            print("updated", p)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
