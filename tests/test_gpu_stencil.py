"""7-point stencil kernel through the C ABI against the CPU checker (B200 only).

The device kernel rounds exactly like the checker's contract=1 form (sum*c1 fused with the
subtraction, centre*c0 rounded first), so the comparison is bit-exact; the binary64 form bounds
the stated 1e-5 relative tolerance.
"""
import numpy as np
import pytest

from helpers import stencil_inputs, to_dev

pytestmark = pytest.mark.gpu


def _sweep(torch, ops, A0, Anext, c0, c1, start=0, end=None, grid=None, block=256):
    nz, ny, nx = A0.shape
    d0, d1 = to_dev(torch, A0), to_dev(torch, Anext)
    k = ops.gptb_stencil(c0, c1, d0.data_ptr(), d1.data_ptr(), nx, ny, nz, start=start, end=end, grid=grid,
                         block=block)
    k.execute(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return d1.cpu().numpy()


@pytest.mark.parametrize("shape", [(8, 8, 64), (5, 9, 130), (3, 4, 64), (16, 12, 200), (4, 7, 66), (64, 16, 128),
                                   (2, 8, 64), (9, 5, 37)])
@pytest.mark.parametrize("block", [64, 128, 256, 512])
def test_sweep_bit_exact(cuda, oracle, shape, block):
    from tacker_b200 import ops

    nz, ny, nx = shape
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=nx)
    c0, c1 = np.float32(1 / 6), np.float32(1 / 36)            # src/ori_kernel/stencil_kernel.cu:132-133
    sentinel = np.full_like(A0, -5.0)
    got = _sweep(cuda, ops, A0, sentinel, c0, c1, grid=3, block=block)
    want = oracle.stencil_sweep_f32(c0, c1, A0, sentinel.copy(), contract=1)
    assert oracle.bit_mismatches(got, want) == 0
    f64 = oracle.stencil_sweep_f64(c0, c1, A0, boundary=sentinel)
    inner = np.zeros(A0.shape, dtype=bool)
    inner[1:-1, 1:-1, 1:-1] = True
    if inner.any():
        scale = np.abs(f64[inner]).max()
        assert np.abs(got[inner] - f64[inner]).max() <= 1e-5 * scale


@pytest.mark.parametrize("rng", [(0, 1), (4, 5), (2, 7), (8, 9), (0, 9), (5, 5), (6, 30)])
def test_virtual_block_range_is_exact(cuda, oracle, rng):
    from tacker_b200 import ops

    nz, ny, nx = 6, 12, 192                                   # 3 x 3 virtual blocks
    start, end = rng
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=2)
    sentinel = np.full_like(A0, 3.0)
    got = _sweep(cuda, ops, A0, sentinel, 0.5, 0.25, start=start, end=end, grid=2, block=128)
    want = oracle.stencil_sweep_f32(0.5, 0.25, A0, sentinel.copy(), start=start, end=min(end, 9), contract=1)
    assert oracle.bit_mismatches(got, want) == 0


def test_config2_ten_jacobi_sweeps(cuda, oracle):
    """512 x 512 x 64, c0 = 1/6, c1 = -1/6, zero boundary, 10 ping-pong sweeps (full size)."""
    from tacker_b200 import ops

    nx, ny, nz = 512, 512, 64
    c0, c1 = np.float32(1 / 6), np.float32(-1 / 6)
    A0 = stencil_inputs(oracle, nx, ny, nz)
    A0[0], A0[-1], A0[:, 0], A0[:, -1], A0[:, :, 0], A0[:, :, -1] = 0, 0, 0, 0, 0, 0
    a, b = to_dev(cuda, A0), to_dev(cuda, A0)
    st = cuda.cuda.current_stream().cuda_stream
    for it in range(10):
        src, dst = (a, b) if it % 2 == 0 else (b, a)
        ops.gptb_stencil(c0, c1, src.data_ptr(), dst.data_ptr(), nx, ny, nz).execute(st)
    cuda.cuda.synchronize()
    got = a.cpu().numpy()                                     # 10 sweeps: result back in `a`
    x, y = A0.copy(), A0.copy()
    want = oracle.stencil_jacobi_f32(c0, c1, x, y, 10, contract=1)
    assert oracle.bit_mismatches(got, want) == 0
    assert np.all(got[0] == 0) and np.all(got[:, 0] == 0) and np.all(got[:, :, -1] == 0)


def test_ori_launch_shape_and_errors(cuda, oracle):
    import ctypes as C

    from tacker_b200 import ops

    nz, ny, nx = 5, 8, 128
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=4)
    d0, d1 = to_dev(cuda, A0), to_dev(cuda, A0)
    ops.OriSTENCILKernel(0.5, 0.125, d0.data_ptr(), d1.data_ptr(), nx, ny, nz).execute()
    cuda.cuda.synchronize()
    want = oracle.stencil_sweep_f32(0.5, 0.125, A0, A0.copy(), contract=1)
    assert oracle.bit_mismatches(d1.cpu().numpy(), want) == 0
    p = [C.c_float(1), C.c_float(1), C.c_void_p(d0.data_ptr()), C.c_void_p(d1.data_ptr()), C.c_int(nx), C.c_int(ny),
         C.c_int(nz), C.c_int(2), C.c_int(2), C.c_int(1), C.c_int(16), C.c_int(8), C.c_int(1), C.c_int(0), C.c_int(1),
         C.c_int(4), C.c_int(0)]
    assert ops.raw_launch("gptb_stencil", p, (2, 1, 1), (128, 1, 1)) == -3       # not the 32 x 4 bundle geometry
    assert ops.raw_launch("gptb_stencil", p[:16], (2, 1, 1), (128, 1, 1)) == -1
    assert ops.raw_launch("gptb_stencil", p, (2, 1, 1), (32, 1, 1)) == -3
