"""Self-check of a generated module (reference: fusion/code/gen_test.py:58-131 and the *_code.py templates,
which emit a main() that runs ORI, GPTB and the fused kernel on the same seeded inputs and compares).

Here one harness serves every pair: it loads the module, launches the generated kernel and the library's solo
kernels on identical seeded inputs and demands bit-identical outputs of the GEMM and of the stencil, and outputs
within 1e-5 of the Coulomb / MRI-Q kernels (whose split work items sum in no fixed order).
Needs a GPU; PyTorch only provides the device buffers.
"""
from __future__ import annotations

import ctypes as C


def lbm_two_writer_mask(nx: int, ny: int, nz: int):
    """Addresses of the lattice-Boltzmann array (margins included) that two cells write in one step: the 20 elements lie
    back to back, so what leaves element e through its top face lands where element e + 1 receives through its bottom
    face.  The reference's kernel has the same two writers and no order between them."""
    import numpy as np

    cells, m = nx * ny * nz, 2 * nx * ny
    dx = [0, 0, 0, 1, -1, 0, 0, 1, -1, 1, -1, 0, 0, 0, 0, 1, 1, -1, -1]
    dy = [0, 1, -1, 0, 0, 0, 0, 1, 1, -1, -1, 1, 1, -1, -1, 0, 0, 0, 0]
    dz = [0, 0, 0, 0, 0, 1, -1, 0, 0, 0, 0, 1, -1, 1, -1, 1, -1, 1, -1]
    count = np.zeros(2 * m + 20 * cells, dtype=np.int32)
    cell = np.arange(cells)
    for e in range(19):
        np.add.at(count, m + e * cells + cell + dx[e] + dy[e] * nx + dz[e] * nx * ny, 1)
    return count > 1


def check_module(so_path: str, name: str, cd: str) -> dict:
    import numpy as np
    import torch

    from .. import LAUNCH_FN, ops

    mod = C.CDLL(so_path)
    fn = LAUNCH_FN(C.cast(getattr(mod, f"tk_launch_{name}"), C.c_void_p).value)
    info = (C.c_int * 4)()
    getattr(mod, f"tk_generated_info_{name}")(info)
    threads = info[0]
    gen = torch.Generator(device="cuda").manual_seed(7)
    M, N, K = 512, 512, 256
    A = (torch.rand(M, K, device="cuda", generator=gen) * 2 - 1).half()
    B = (torch.rand(N, K, device="cuda", generator=gen) * 2 - 1).half()
    sms = ops.sm_count()

    cut = None
    if cd == "cutcp":
        from ..profile_ratios import cutcp_problem

        cbins, cnbr, cmargin = cutcp_problem(16, 16, 16, seed=3)
        cut = dict(bins=torch.from_numpy(cbins).cuda(), nbr=torch.from_numpy(cnbr).cuda(), n=cnbr.shape[0],
                   bdx=cbins.shape[2], bdy=cbins.shape[1], c=cmargin)
        cut["zero"] = cut["bins"].data_ptr() + 128 * ((cmargin * cut["bdy"] + cmargin) * cut["bdx"] + cmargin)

    def cd_kernel(bufs):
        if cd == "stencil":
            return ops.gptb_stencil(0.5, 0.25, bufs[0].data_ptr(), bufs[1].data_ptr(), 192, 12, 10)
        if cd == "cp":
            return ops.gptb_cp(150, 0.125, bufs[1].data_ptr(), bufs[0].data_ptr(), 256, 32)
        if cd == "mrif":
            return ops.gptb_mrif(64, bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(),
                                 bufs[4].data_ptr(), bufs[5].data_ptr(), 1024)
        if cd == "sgemm":
            return ops.gptb_sgemm(bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), 256, 64, 48)
        if cd == "lbm":
            return ops.gptb_lbm(bufs[0].data_ptr() + 4 * 2 * 64 * 4, bufs[1].data_ptr() + 4 * 2 * 64 * 4, 64, 4, 5)
        if cd == "fft":
            return ops.gptb_fft(bufs[0].data_ptr(), 48)
        if cd == "cutcp":
            inv = float(np.float32(1.0) / np.float32(144.0))
            return ops.gptb_cutcp(cut["bdx"], cut["bdy"], cut["zero"], 0.5, 144.0, inv, bufs[0].data_ptr(),
                                  cut["nbr"].data_ptr(), cut["n"], 2, 2, 2)
        return ops.gptb_mriq(64, bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(),
                             bufs[4].data_ptr(), bufs[5].data_ptr(), 1024)

    def fresh():
        g = torch.Generator(device="cuda").manual_seed(11)
        if cd == "stencil":
            a0 = torch.rand(10, 12, 192, device="cuda", generator=g)
            return [a0, a0.clone()], 1
        if cd == "cp":
            atoms = torch.rand(150, 4, device="cuda", generator=g) * 8
            atoms[:, 2] = (atoms[:, 2] - 4) ** 2 + 0.5
            return [atoms.contiguous(), torch.zeros(32, 256, device="cuda")], 1
        if cd == "sgemm":
            return [torch.rand(48, 256, device="cuda", generator=g), torch.rand(48, 64, device="cuda", generator=g),
                    torch.rand(64, 256, device="cuda", generator=g)], 2
        if cd == "lbm":
            n = 20 * 64 * 4 * 5 + 2 * 2 * 64 * 4
            return [torch.rand(n, device="cuda", generator=g), torch.rand(n, device="cuda", generator=g)], 1
        if cd == "fft":
            return [torch.rand(48, 256, 2, device="cuda", generator=g) * 2 - 1], 0
        if cd == "cutcp":
            return [torch.zeros(2, 2, 2, 512, device="cuda")], 0
        xyz = [torch.rand(1024, device="cuda", generator=g) * 64 - 32 for _ in range(3)]
        if cd == "mrif":
            kv = torch.rand(5 * 64, device="cuda", generator=g) - 0.5
        else:
            kv = torch.rand(64, 4, device="cuda", generator=g) - 0.5
        return xyz + [torch.zeros(1024, device="cuda"), torch.zeros(1024, device="cuda"), kv.contiguous()], 3

    st = torch.cuda.current_stream().cuda_stream
    results = {}
    def launch_generated(cdk, tz, cd_range=None, tz_range=None):
        mk = ops.mix(cdk, tz, cd_threads=threads - 192, grid=sms, cd_range=cd_range, tz_range=tz_range)
        arr = (C.c_void_p * len(mk.kernelParams))(*[C.cast(C.pointer(p), C.c_void_p) for p in mk.kernelParams])
        rc = fn(arr, len(mk.kernelParams), (C.c_uint * 3)(sms, 1, 1), (C.c_uint * 3)(threads, 1, 1), 0, C.c_void_p(st))
        assert rc == 0, f"generated launcher returned {rc}"

    # "halves": the pair as two launches with one side's block range empty (the launcher then runs the other
    # kernel alone), then one with both empty (nothing runs)
    for mode in ("solo", "generated", "halves"):
        bufs, out_idx = fresh()
        Cm = torch.zeros(M, N, device="cuda")
        tz = ops.gptb_tzgemm(A.data_ptr(), B.data_ptr(), Cm.data_ptr(), M, N, K, alpha=1.1, grid=sms)
        cdk = cd_kernel(bufs)
        if mode == "solo":
            tz.execute(st)
            cdk.execute(st)
        elif mode == "generated":
            launch_generated(cdk, tz)
        else:
            launch_generated(cdk, tz, tz_range=(0, 0))
            launch_generated(cdk, tz, cd_range=(0, 0))
            launch_generated(cdk, tz, cd_range=(0, 0), tz_range=(0, 0))
        torch.cuda.synchronize()
        results[mode] = (Cm.cpu().numpy(), bufs[out_idx].cpu().numpy())
    if cd == "lbm":  # compare the addresses with one writer
        once = ~lbm_two_writer_mask(64, 4, 5)
        for mode in results:
            results[mode] = (results[mode][0], results[mode][1][once])
    same_gemm = bool(np.array_equal(results["solo"][0], results["generated"][0]))
    same_cd = bool(np.array_equal(results["solo"][1], results["generated"][1]))
    # Coulomb / MRI-Q items that cover a part of the atom / sample list add their partial sums with reductions in
    # no fixed order: those outputs are held to the operators' 1e-5 tolerance instead of bit identity
    scale = float(np.abs(results["solo"][1]).max())
    cd_err = float(np.abs(results["solo"][1] - results["generated"][1]).max()) / (scale if scale > 0 else 1.0)
    # bit identity where every output has one fixed sequence of operations and one writer; lbm has addresses with two
    # writers (held to the tolerance), the others may run on work items that add partial sums in no fixed order
    cd_ok = same_cd if cd in ("stencil", "fft") else cd_err <= 1e-5
    halves_err = float(np.abs(results["solo"][1] - results["halves"][1]).max()) / (scale if scale > 0 else 1.0)
    halves_ok = bool(np.array_equal(results["solo"][0], results["halves"][0])) and halves_err <= 1e-5
    same_gemm = same_gemm and halves_ok
    return {"name": name, "threads": threads, "gemm_bit_identical": same_gemm, "cd_bit_identical": same_cd,
            "cd_max_rel_err": cd_err, "empty_ranges_ok": halves_ok,
            "ok": same_gemm and cd_ok and bool(np.abs(results["generated"][0]).max() > 0)}
