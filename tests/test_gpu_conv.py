"""Implicit-GEMM convolution (gptb_tzconv and the tzconv_<cd> fused kernels) through the C ABI (B200 only).

Checked against a numpy convolution on the same fp16-rounded operands (fp32 accumulation, tolerance 1e-3 of
sum |x||w| per output like the GEMM) and, bit for bit, against the explicit path it replaces: im2col -> tzgemm ->
bias + activation -> fp16."""
import numpy as np
import pytest

from helpers import to_dev

pytestmark = pytest.mark.gpu


def _case(oracle, H, W, Cin, Cout, seed):
    x = oracle.uniform_f32(H * W * Cin, 1100 + seed, -1.0, 1.0).reshape(H, W, Cin).astype(np.float16)
    w = (oracle.uniform_f32(Cout * 9 * Cin, 1200 + seed, -1.0, 1.0) * np.float32(np.sqrt(6.0 / (9 * Cin)))).astype(np.float16)
    w = w.reshape(Cout, 9 * Cin)                                      # k = (3 i + j) Cin + c
    bias = oracle.uniform_f32(Cout, 1300 + seed, -0.5, 0.5)
    xb = np.zeros((H + 2, W + 2, Cin), np.float16)
    xb[1:-1, 1:-1] = x
    return x, w, bias, xb


def _numpy_conv(xb, w, bias, H, W, act):
    xf = xb.astype(np.float32)
    cols = np.concatenate([xf[i:i + H, j:j + W] for i in range(3) for j in range(3)], axis=2).reshape(H * W, -1)
    wf = w.astype(np.float32)
    y = cols.astype(np.float64) @ wf.astype(np.float64).T + bias
    mag = np.abs(cols).astype(np.float64) @ np.abs(wf).astype(np.float64).T + np.abs(bias)
    if act:
        y = np.maximum(y, 0.0)
    return y.reshape(H, W, -1), mag.reshape(H, W, -1)


def _run_implicit(torch, ops, xb, w, bias, H, W, Cin, Cout, act, start=0, end=None, grid=None, fill=0.0):
    X, Wt, B = to_dev(torch, xb), to_dev(torch, w), to_dev(torch, bias)
    Y = torch.full((H + 2, W + 2, Cout), fill, dtype=torch.float16, device="cuda")
    k = ops.gptb_tzconv(X.data_ptr(), Wt.data_ptr(), Y.data_ptr(), H, W, Cin, Cout, bias=B.data_ptr(), act=act,
                        start=start, end=end, grid=grid)
    k.execute(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return Y.cpu().numpy(), k


@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("shape", [(8, 8, 64, 64), (14, 14, 128, 192), (28, 30, 64, 256), (9, 37, 192, 128)])
def test_matches_numpy_and_the_explicit_path(cuda, oracle, shape, act):
    from tacker_b200 import ops

    H, W, Cin, Cout = shape
    x, w, bias, xb = _case(oracle, H, W, Cin, Cout, H + W)
    got, _ = _run_implicit(cuda, ops, xb, w, bias, H, W, Cin, Cout, act, grid=5)
    # the border is never written
    assert not got[0].any() and not got[-1].any() and not got[:, 0].any() and not got[:, -1].any()
    want, mag = _numpy_conv(xb, w, bias, H, W, act)
    inner = got[1:-1, 1:-1].astype(np.float64)
    assert (np.abs(inner - want) / (mag + 1e-6)).max() <= 1e-3 + 2.0 ** -11     # + the fp16 rounding of the output
    # explicit path: im2col from the fp32 copy of the same image, tzgemm, bias + activation, fp16
    st = cuda.cuda.current_stream().cuda_stream
    M, K = H * W, 9 * Cin
    M_pad = (M + 127) // 128 * 128
    xf = to_dev(cuda, x.astype(np.float32))
    A = cuda.zeros((M_pad, K), dtype=cuda.float16, device="cuda")
    ops.im2col_nhwc_f16(xf.data_ptr(), H, W, Cin, 3, 3, 1, 1, A.data_ptr(), M_pad, K, st)
    Wt = to_dev(cuda, w)
    Cm = cuda.zeros((M_pad, Cout), dtype=cuda.float32, device="cuda")
    ops.gptb_tzgemm(A.data_ptr(), Wt.data_ptr(), Cm.data_ptr(), M_pad, Cout, K, alpha=1.0, round_dims=False).execute(st)
    Bd = to_dev(cuda, bias)
    Yb = cuda.zeros((H + 2, W + 2, Cout), dtype=cuda.float16, device="cuda")
    ops.bias_act_f16_bordered(Cm.data_ptr(), Cout, Bd.data_ptr(), Yb.data_ptr(), H, W, Cout, act, st)
    cuda.cuda.synchronize()
    assert np.array_equal(got.view(np.uint16), Yb.cpu().numpy().view(np.uint16))


@pytest.mark.parametrize("rng", [(0, 1), (3, 9), (0, 400), (17, 18)])
def test_tile_range_is_exact(cuda, oracle, rng):
    from tacker_b200 import ops

    H, W, Cin, Cout = 16, 14, 64, 128                # M = 16 * 16 = 256 rows -> 4 x 2 = 8 tiles
    x, w, bias, xb = _case(oracle, H, W, Cin, Cout, 3)
    full, k = _run_implicit(cuda, ops, xb, w, bias, H, W, Cin, Cout, 1)
    start, end = rng
    got, _ = _run_implicit(cuda, ops, xb, w, bias, H, W, Cin, Cout, 1, start=start, end=end, grid=2, fill=-7.0)
    inside = np.zeros((H + 2, W + 2, Cout), dtype=bool)
    for p in range(start, min(end, 8)):
        r, c = p // 2, p % 2
        for m in range(r * 64, r * 64 + 64):
            oh, ow = divmod(m, W + 2)
            if ow < W and oh < H:
                inside[oh + 1, ow + 1, c * 64:c * 64 + 64] = True
    assert np.all(got[~inside] == np.float16(-7.0))
    assert np.array_equal(got[inside], full[inside])


@pytest.mark.parametrize("cd", ["stencil", "cp", "mriq", "mrif"])
def test_fused_convolution_kernels(cuda, oracle, cd):
    """tzconv_<cd>: the convolution's output is bit for bit the solo kernel's; the CUDA-core side is checked
    against its solo kernel (bit for bit with unsplit work items)."""
    from helpers import coulomb_inputs, mrif_inputs, mriq_inputs, stencil_inputs
    from tacker_b200 import ops

    H, W, Cin, Cout = 20, 20, 128, 128
    x, w, bias, xb = _case(oracle, H, W, Cin, Cout, 5)
    solo, _ = _run_implicit(cuda, ops, xb, w, bias, H, W, Cin, Cout, 1)
    st = cuda.cuda.current_stream().cuda_stream
    X, Wt, B = to_dev(cuda, xb), to_dev(cuda, w), to_dev(cuda, bias)
    ops.set_option("cp_split", 0)
    ops.set_option("mriq_split", 0)
    try:
        outs = {}
        for mode in ("solo", "fused"):
            Y = cuda.zeros((H + 2, W + 2, Cout), dtype=cuda.float16, device="cuda")
            tz = ops.gptb_tzconv(X.data_ptr(), Wt.data_ptr(), Y.data_ptr(), H, W, Cin, Cout, bias=B.data_ptr(), act=1, grid=4)
            if cd == "stencil":
                A0 = stencil_inputs(oracle, 128, 12, 8, seed=2)
                d0, d1 = to_dev(cuda, A0), to_dev(cuda, A0)
                cdk = ops.gptb_stencil(0.5, 0.25, d0.data_ptr(), d1.data_ptr(), 128, 12, 8, grid=4, block=128)
                res = [d1]
            elif cd == "cp":
                atoms = coulomb_inputs(oracle, 90, 16.0, seed=6, spacing=0.125, zplane=2.0)
                raw = to_dev(cuda, atoms)
                packed = cuda.empty_like(raw)
                ops.cp_pack_atoms(raw.data_ptr(), 90, 2.0, packed.data_ptr(), st)
                lat = cuda.zeros((16, 128), dtype=cuda.float32, device="cuda")
                cdk = ops.gptb_cp(90, 0.125, lat.data_ptr(), packed.data_ptr(), 128, 16, grid=4, block=128)
                res = [lat]
            else:
                if cd == "mriq":
                    k, phi, xyz = mriq_inputs(oracle, 70, 512, seed=4)
                    dev = [to_dev(cuda, v) for v in (k[0], k[1], k[2], phi[0], phi[1])]
                    kv = cuda.empty(4 * 70, dtype=cuda.float32, device="cuda")
                    ops.mriq_pack_kvalues(*[t.data_ptr() for t in dev], 70, kv.data_ptr(), st)
                else:
                    k, phi, d, xyz = mrif_inputs(oracle, 70, 512, seed=4)
                    dev = [to_dev(cuda, v) for v in (k[0], k[1], k[2], phi[0], phi[1], d[0], d[1])]
                    kv = cuda.empty(5 * 70, dtype=cuda.float32, device="cuda")
                    ops.mrif_pack_kvalues(*[t.data_ptr() for t in dev], 70, kv.data_ptr(), st)
                dx = [to_dev(cuda, xyz[i]) for i in range(3)]
                qr = cuda.zeros(512, dtype=cuda.float32, device="cuda")
                qi = cuda.zeros(512, dtype=cuda.float32, device="cuda")
                make = ops.gptb_mriq if cd == "mriq" else ops.gptb_mrif
                cdk = make(70, dx[0].data_ptr(), dx[1].data_ptr(), dx[2].data_ptr(), qr.data_ptr(), qi.data_ptr(),
                           kv.data_ptr(), 512, grid=4, block=128)
                res = [qr, qi]
            if mode == "solo":
                tz.execute(st)
                cdk.execute(st)
            else:
                ops.mix(cdk, tz, cd_threads=128, grid=4).execute(st)
            cuda.cuda.synchronize()
            assert ops.device_status() == 0
            outs[mode] = [Y.cpu().numpy()] + [r.cpu().numpy() for r in res]
    finally:
        ops.set_option("cp_split", -1)
        ops.set_option("mriq_split", -1)
    assert np.array_equal(outs["fused"][0].view(np.uint16), solo.view(np.uint16))
    for a, b in zip(outs["solo"], outs["fused"]):
        assert np.array_equal(a, b)
    assert np.abs(outs["fused"][1]).max() > 0


def test_bad_shapes_return_status(cuda):
    import ctypes as C

    from tacker_b200 import ops

    buf = cuda.zeros(1 << 16, dtype=cuda.float16, device="cuda")
    p = buf.data_ptr()

    def status(H, W, Cin, Cout, K=None, M=None):
        M_ = ((H * (W + 2) + 127) // 128) * 128 if M is None else M
        prm = [C.c_void_p(p), C.c_void_p(p), C.c_void_p(p), C.c_int(M_), C.c_int(Cout), C.c_int(9 * Cin if K is None else K),
               C.c_float(1.0), C.c_void_p(0), C.c_int(H), C.c_int(W), C.c_int(Cin), C.c_int(1)] + [C.c_int(1)] * 6 + \
              [C.c_int(0), C.c_int(1), C.c_int(0), C.c_int(0)]
        return ops.raw_launch("gptb_tzconv", prm, (2, 1, 1), (192, 1, 1))

    assert status(8, 8, 64, 64) == 0             # empty range: accepted, nothing launched
    assert status(8, 8, 48, 64) == -3            # channels not a multiple of 64
    assert status(8, 8, 64, 64, K=512) == -3     # K != 9 C
    assert status(8, 8, 64, 64, M=64) == -3      # M too small
