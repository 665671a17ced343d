"""Whole-operator entry points and the host-buffer pair through the C ABI (B200 only)."""
import numpy as np
import pytest

from helpers import coulomb_inputs, gemm_inputs, mriq_inputs, stencil_inputs, to_dev

pytestmark = pytest.mark.gpu


def test_mriq_compute_matches_oracle(cuda, oracle):
    from tacker_b200 import ops

    numK, numX = 300, 2048
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=21)
    d = [to_dev(cuda, v) for v in (k[0], k[1], k[2], phi[0], phi[1], xyz[0], xyz[1], xyz[2])]
    qr = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
    qi = cuda.zeros(numX, dtype=cuda.float32, device="cuda")
    scratch = cuda.empty((numK, 4), dtype=cuda.float32, device="cuda")
    ops.mriq_compute(*[t.data_ptr() for t in d[:5]], numK, *[t.data_ptr() for t in d[5:]], qr.data_ptr(),
                     qi.data_ptr(), numX, scratch.data_ptr())
    cuda.cuda.synchronize()
    kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
    r64, i64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2])
    peak = max(np.abs(r64).max(), np.abs(i64).max())
    assert np.abs(qr.cpu().numpy() - r64).max() <= 1e-5 * peak
    assert np.abs(qi.cpu().numpy() - i64).max() <= 1e-5 * peak


def test_coulomb_compute_matches_oracle(cuda, oracle):
    from tacker_b200 import ops

    nx, ny, h, z = 256, 32, 0.125, 3.0
    atoms = coulomb_inputs(oracle, 333, 16.0, seed=8, spacing=h, zplane=z)
    raw = to_dev(cuda, atoms)
    scratch = cuda.empty_like(raw)
    lat = cuda.zeros((ny, nx), dtype=cuda.float32, device="cuda")
    ops.coulomb_compute(raw.data_ptr(), atoms.shape[0], z, h, lat.data_ptr(), nx, ny, scratch.data_ptr())
    cuda.cuda.synchronize()
    pk = oracle.cp_pack_atoms(atoms, z)
    ref32 = oracle.cp_f32(pk, h, np.zeros((ny, nx), np.float32), chunk=64)
    _, mag = oracle.cp_f64(pk, h, nx, ny)
    assert (np.abs(lat.cpu().numpy() - ref32) / mag).max() <= 1e-5


def test_pair_host_buffers(cuda, oracle):
    """Host in, host out: GEMM result and the array after `sweeps` Jacobi sweeps."""
    from tacker_b200 import ops

    M, N, K = 256, 256, 128
    nx, ny, nz, sweeps = 128, 16, 8, 3
    a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=2)
    A0 = stencil_inputs(oracle, nx, ny, nz, seed=3)
    hA = cuda.from_numpy(a_bits.view(np.float16).copy()).pin_memory()
    hB = cuda.from_numpy(b_bits.view(np.float16).copy()).pin_memory()
    hA0 = cuda.from_numpy(A0.copy()).pin_memory()
    hC = cuda.empty((M, N), dtype=cuda.float32).pin_memory()
    hOut = cuda.empty((nz, ny, nx), dtype=cuda.float32).pin_memory()
    nbytes = ops.pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz)
    ws = cuda.empty(nbytes, dtype=cuda.uint8, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    ops.pair_tzgemm_stencil_host(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), M, N, K, 1.0, 0.5, 0.25, hA0.data_ptr(),
                                 hOut.data_ptr(), nx, ny, nz, sweeps, 128, ws.data_ptr(), nbytes, st)
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    x, y = A0.copy(), A0.copy()
    want = oracle.stencil_jacobi_f32(0.5, 0.25, x, y, sweeps, contract=1)
    assert oracle.bit_mismatches(hOut.numpy(), want) == 0
    ref = oracle.tzgemm_f64(a, b)
    assert np.abs(hC.numpy() - ref).max() <= 1e-3 * K
    with pytest.raises(Exception, match="capacity"):
        ops.pair_tzgemm_stencil_host(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), M, N, K, 1.0, 0.5, 0.25,
                                     hA0.data_ptr(), hOut.data_ptr(), nx, ny, nz, sweeps, 128, ws.data_ptr(), 1024, st)


def test_pair_host_rejected_shape_queues_nothing(cuda, oracle):
    """A call refused for its GEMM shape returns before any copy is queued: the workspace keeps its bytes."""
    from tacker_b200 import ops

    M, N, K = 256, 256, 96          # K is not a multiple of 64
    nx, ny, nz = 128, 16, 8
    hA = cuda.ones((M, K), dtype=cuda.float16).pin_memory()
    hB = cuda.ones((N, K), dtype=cuda.float16).pin_memory()
    hA0 = cuda.ones((nz, ny, nx), dtype=cuda.float32).pin_memory()
    hC = cuda.empty((M, N), dtype=cuda.float32).pin_memory()
    hOut = cuda.empty((nz, ny, nx), dtype=cuda.float32).pin_memory()
    nbytes = ops.pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz)
    ws = cuda.full((nbytes,), 0xA5, dtype=cuda.uint8, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    with pytest.raises(Exception, match="shape"):
        ops.pair_tzgemm_stencil_host(hA.data_ptr(), hB.data_ptr(), hC.data_ptr(), M, N, K, 1.0, 0.5, 0.25, hA0.data_ptr(),
                                     hOut.data_ptr(), nx, ny, nz, 2, 128, ws.data_ptr(), nbytes, st)
    cuda.cuda.synchronize()
    assert bool((ws == 0xA5).all())


def test_pair_host_calls_in_flight_keep_their_own_results(cuda, oracle):
    """Four calls queued back to back with different inputs and their own host buffers: the library overlaps their
    uploads, kernels and downloads over two sets of device buffers (the third call reuses the first call's set), and every
    call's results are its own."""
    from tacker_b200 import ops

    M, N, K = 256, 128, 64
    nx, ny, nz, sweeps = 64, 8, 6, 2
    nbytes = ops.pair_tzgemm_stencil_workspace(M, N, K, nx, ny, nz)
    ws = cuda.empty(nbytes, dtype=cuda.uint8, device="cuda")
    st = cuda.cuda.current_stream().cuda_stream
    calls = []
    for i in range(4):
        a_bits, a, b_bits, b = gemm_inputs(oracle, M, N, K, seed=20 + i)
        A0 = stencil_inputs(oracle, nx, ny, nz, seed=30 + i)
        h = dict(a=a, b=b, A0=A0,
                 hA=cuda.from_numpy(a_bits.view(np.float16).copy()).pin_memory(),
                 hB=cuda.from_numpy(b_bits.view(np.float16).copy()).pin_memory(),
                 hA0=cuda.from_numpy(A0.copy()).pin_memory(),
                 hC=cuda.zeros((M, N), dtype=cuda.float32).pin_memory(),
                 hOut=cuda.zeros((nz, ny, nx), dtype=cuda.float32).pin_memory())
        calls.append(h)
    for h in calls:
        ops.pair_tzgemm_stencil_host(h["hA"].data_ptr(), h["hB"].data_ptr(), h["hC"].data_ptr(), M, N, K, 1.0, 0.5, 0.25,
                                     h["hA0"].data_ptr(), h["hOut"].data_ptr(), nx, ny, nz, sweeps, 128, ws.data_ptr(), nbytes,
                                     st)
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    for h in calls:
        x, y = h["A0"].copy(), h["A0"].copy()
        want = oracle.stencil_jacobi_f32(0.5, 0.25, x, y, sweeps, contract=1)
        assert oracle.bit_mismatches(h["hOut"].numpy(), want) == 0
        assert np.abs(h["hC"].numpy() - oracle.tzgemm_f64(h["a"], h["b"])).max() <= 1e-3 * K
