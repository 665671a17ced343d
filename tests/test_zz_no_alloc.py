"""MRI-Q through the entry point that allocates nothing (B200 only).

tk_mriq_compute_static is for callers that may not allocate device memory (a latency-critical loop, a
process whose memory belongs to someone else's pool, a plug-in that only gets its host's buffers): the
packed sample table is a fixed array inside the library.  It must give what tk_mriq_compute gives with
caller scratch -- the same kernels in the same order -- on two calls in a row, the second with fewer samples
so that leftovers of the first call would show.  With unsplit work items (option mriq_split = 0) the summation
order is fixed and the outputs are compared bit for bit; with the default items, whose partial sums are added by
reductions in no fixed order, they are held to the operator's tolerance, 1e-5 of the largest |Q|.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import numpy as np
import pytest

from helpers import mriq_inputs, to_dev

pytestmark = pytest.mark.gpu


def _both(torch, ops, oracle, numK, numX, seed):
    k, phi, xyz = mriq_inputs(oracle, numK, numX, seed=seed)
    d = [to_dev(torch, v) for v in (k[0], k[1], k[2], phi[0], phi[1], xyz[0], xyz[1], xyz[2])]
    ins, pts = [t.data_ptr() for t in d[:5]], [t.data_ptr() for t in d[5:]]
    out = {}
    for name in ("scratch", "static"):
        qr = torch.full((numX,), 0.25, dtype=torch.float32, device="cuda")
        qi = torch.full((numX,), -0.5, dtype=torch.float32, device="cuda")
        if name == "scratch":
            scratch = torch.empty((numK, 4), dtype=torch.float32, device="cuda")
            ops.mriq_compute(*ins, numK, *pts, qr.data_ptr(), qi.data_ptr(), numX, scratch.data_ptr())
        else:
            ops.mriq_compute_static(*ins, numK, *pts, qr.data_ptr(), qi.data_ptr(), numX)
        torch.cuda.synchronize()
        out[name] = (qr.cpu().numpy(), qi.cpu().numpy())
    return out, (k, phi, xyz)


@pytest.mark.parametrize("split", [0, -1])
def test_static_table_matches_caller_scratch_twice(cuda, oracle, split):
    from tacker_b200 import ops

    ops.set_option("mriq_split", split)
    try:
        for numK, numX, seed in ((1500, 2048, 41), (70, 1024, 42)):
            out, (k, phi, xyz) = _both(cuda, ops, oracle, numK, numX, seed)
            kv = oracle.mriq_pack(k[0], k[1], k[2], oracle.mriq_phimag(phi[0], phi[1]))
            r64, i64 = oracle.mriq_f64(kv, xyz[0], xyz[1], xyz[2])
            peak = max(np.abs(r64).max(), np.abs(i64).max())
            if split == 0:
                assert np.array_equal(out["static"][0], out["scratch"][0])
                assert np.array_equal(out["static"][1], out["scratch"][1])
            else:
                assert np.abs(out["static"][0] - out["scratch"][0]).max() <= 1e-5 * peak
                assert np.abs(out["static"][1] - out["scratch"][1]).max() <= 1e-5 * peak
            # and both are right: binary64 checker, 1e-5 of the largest |Q|
            assert np.abs(out["static"][0] - 0.25 - r64).max() <= 1e-5 * peak
            assert np.abs(out["static"][1] + 0.5 - i64).max() <= 1e-5 * peak
    finally:
        ops.set_option("mriq_split", -1)


def test_over_capacity_is_rejected_with_a_message(cuda):
    import tacker_b200
    from tacker_b200 import ops

    t = cuda.zeros(8192, dtype=cuda.float32, device="cuda")
    p = t.data_ptr()
    with pytest.raises(tacker_b200.TackerError, match="exceeds the fixed table of 4096") as e:
        ops.mriq_compute_static(p, p, p, p, p, 4097, p, p, p, p, p, 256)
    assert e.value.status == -8
    ops.mriq_compute_static(p, p, p, p, p, 4096, p, p, p, p, p, 0)        # at the limit, empty job: accepted
    cuda.cuda.synchronize()
