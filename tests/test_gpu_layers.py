"""Layer kernels of the DNN tasks and the batched tzgemm through the C ABI against numpy (B200 only)."""
import numpy as np
import pytest

from helpers import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("geom", [(12, 10, 5, 7, 3, 1, 1), (9, 11, 16, 40, 3, 1, 2), (14, 14, 8, 64, 1, 0, 1)])
def test_conv_as_im2col_plus_tzgemm(cuda, oracle, geom):
    """A convolution computed the way ConvKernel does it: NHWC im2col to fp16, tzgemm, bias + ReLU."""
    from tacker_b200 import ops

    H, W, Cin, Cout, k, pad, stride = geom
    x = oracle.uniform_f32(H * W * Cin, 1, -1.0, 1.0).reshape(H, W, Cin)
    w_bits, w = oracle.uniform_f16(Cout * k * k * Cin, 2, -0.5, 0.5)
    w = w.reshape(Cout, k, k, Cin)
    bias = oracle.uniform_f32(Cout, 3, -0.1, 0.1)
    OH, OW = (H + 2 * pad - k) // stride + 1, (W + 2 * pad - k) // stride + 1
    M, K = OH * OW, k * k * Cin
    M_pad, N_pad, K_pad = -(-M // 128) * 128, 64, -(-K // 64) * 64
    Bw = np.zeros((N_pad, K_pad), dtype=np.uint16)
    Bw[:Cout, :K] = w_bits.reshape(Cout, K)
    dx, dB = to_dev(cuda, x), cuda.from_numpy(Bw.view(np.float16)).cuda()
    dA = cuda.zeros((M_pad, K_pad), dtype=cuda.float16, device="cuda")
    dC = cuda.zeros((M_pad, N_pad), dtype=cuda.float32, device="cuda")
    dy = cuda.zeros((M, Cout), dtype=cuda.float32, device="cuda")
    ops.im2col_nhwc_f16(dx.data_ptr(), H, W, Cin, k, k, pad, stride, dA.data_ptr(), M_pad, K_pad)
    ops.gptb_tzgemm(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M_pad, N_pad, K_pad, alpha=1.0,
                    round_dims=False).execute()
    ops.bias_act_f32(dC.data_ptr(), N_pad, to_dev(cuda, bias).data_ptr(), dy.data_ptr(), M, Cout, Cout, 1)
    cuda.cuda.synchronize()
    # the im2col operand is bit-exact: fp16 rounding of the gathered inputs
    xp = np.pad(x, ((pad, pad), (pad, pad), (0, 0)))
    cols = np.stack([xp[i:i + stride * OH:stride, j:j + stride * OW:stride, :] for i in range(k) for j in range(k)],
                    axis=2).reshape(M, K)
    A = dA.cpu().numpy()
    assert np.array_equal(A[:M, :K].view(np.uint16), oracle.f32_to_f16_bits(cols).reshape(M, K))
    assert not A[M:].any() and not A[:, K:].any()
    want = np.maximum(cols.astype(np.float16).astype(np.float64) @ w.reshape(Cout, K).astype(np.float64).T + bias, 0)
    assert np.abs(dy.cpu().numpy() - want).max() <= 1e-3 * K


def test_elementwise_and_row_kernels(cuda, oracle):
    from tacker_b200 import ops

    rows, cols = 37, 200
    x = oracle.normal_f32(rows * cols, 4).reshape(rows, cols)
    g = oracle.uniform_f32(cols, 5, 0.5, 1.5)
    b = oracle.uniform_f32(cols, 6, -0.5, 0.5)
    dx, dg, db = to_dev(cuda, x), to_dev(cuda, g), to_dev(cuda, b)
    out = cuda.zeros((rows, cols), dtype=cuda.float32, device="cuda")
    ops.softmax_rows_f32(dx.data_ptr(), out.data_ptr(), rows, cols, 0.5)
    e = np.exp(0.5 * x.astype(np.float64) - (0.5 * x).max(1, keepdims=True))
    assert np.abs(out.cpu().numpy() - e / e.sum(1, keepdims=True)).max() < 1e-6
    ops.layernorm_rows_f32(dx.data_ptr(), dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, cols, 1e-5)
    x64 = x.astype(np.float64)
    ln = (x64 - x64.mean(1, keepdims=True)) / np.sqrt(x64.var(1, keepdims=True) + 1e-5) * g + b
    assert np.abs(out.cpu().numpy() - ln).max() < 1e-4
    ops.bias_act_f32(dx.data_ptr(), cols, db.data_ptr(), out.data_ptr(), rows, cols, cols, 2)
    v = x64 + b
    gelu = 0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    assert np.abs(out.cpu().numpy() - gelu).max() < 1e-5
    ops.add_f32(dx.data_ptr(), dx.data_ptr(), out.data_ptr(), rows * cols)
    assert np.array_equal(out.cpu().numpy(), x + x)
    H, W, Cn = 6, 8, 5
    img = oracle.normal_f32(H * W * Cn, 7).reshape(H, W, Cn)
    po = cuda.zeros((H // 2, W // 2, Cn), dtype=cuda.float32, device="cuda")
    ops.maxpool2x2_nhwc_f32(to_dev(cuda, img).data_ptr(), H, W, Cn, po.data_ptr())
    cuda.cuda.synchronize()
    assert np.array_equal(po.cpu().numpy(), img.reshape(H // 2, 2, W // 2, 2, Cn).max(axis=(1, 3)))
    half = cuda.zeros((64, 256), dtype=cuda.float16, device="cuda")
    ops.rows_f32_to_f16(dx.data_ptr(), rows, cols, cols, half.data_ptr(), 64, 256)
    cuda.cuda.synchronize()
    hh = half.cpu().numpy()
    assert np.array_equal(hh[:rows, :cols], x.astype(np.float16)) and not hh[rows:].any() and not hh[:, cols:].any()


def test_row_kernels_on_aligned_shapes(cuda, oracle):
    """The same kernels on the shapes the models use (columns a multiple of 128, 16-byte aligned arrays), where they
    move 16 bytes per thread and the normalisation keeps its row in registers; plus layernorm(a + b) in one pass."""
    from tacker_b200 import ops

    rows, cols = 96, 768
    x = oracle.normal_f32(rows * cols, 14).reshape(rows, cols)
    y = oracle.normal_f32(rows * cols, 15).reshape(rows, cols)
    g = oracle.uniform_f32(cols, 5, 0.5, 1.5)
    b = oracle.uniform_f32(cols, 6, -0.5, 0.5)
    dx, dy, dg, db = to_dev(cuda, x), to_dev(cuda, y), to_dev(cuda, g), to_dev(cuda, b)
    out = cuda.zeros((rows, cols), dtype=cuda.float32, device="cuda")
    x64, y64 = x.astype(np.float64), y.astype(np.float64)
    ln = lambda v: (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5) * g + b
    ops.layernorm_rows_f32(dx.data_ptr(), dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, cols, 1e-5)
    assert np.abs(out.cpu().numpy() - ln(x64)).max() < 1e-4
    ops.add_layernorm_rows_f32(dx.data_ptr(), dy.data_ptr(), dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, cols, 1e-5)
    assert np.abs(out.cpu().numpy() - ln((x + y).astype(np.float64))).max() < 1e-4
    with pytest.raises(Exception):
        ops.add_layernorm_rows_f32(dx.data_ptr(), dy.data_ptr(), dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, 200, 1e-5)
    wide = cuda.zeros((rows, 832), dtype=cuda.float32, device="cuda")                       # leading dimensions beyond cols
    ops.bias_act_f32(dx.data_ptr(), cols, db.data_ptr(), wide.data_ptr(), rows, cols, 832, 2)
    v = x64 + b
    gelu = 0.5 * v * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    w = wide.cpu().numpy()
    assert np.abs(w[:, :cols] - gelu).max() < 1e-5 and not w[:, cols:].any()
    ops.bias_act_f32(dx.data_ptr(), cols, 0, out.data_ptr(), rows, cols, cols, 1)
    assert np.array_equal(out.cpu().numpy(), np.maximum(x, 0))
    ops.add_f32(dx.data_ptr(), dy.data_ptr(), out.data_ptr(), rows * cols)
    assert np.array_equal(out.cpu().numpy(), x + y)
    half = cuda.zeros((128, 832), dtype=cuda.float16, device="cuda")
    ops.rows_f32_to_f16(dx.data_ptr(), rows, cols, cols, half.data_ptr(), 128, 832)
    hh = half.cpu().numpy()
    assert np.array_equal(hh[:rows, :cols], x.astype(np.float16)) and not hh[rows:].any() and not hh[:, cols:].any()
    ops.rows_f32_to_f16(dx.data_ptr(), rows, 764, cols, half.data_ptr(), 128, 832)       # a ragged last group of 8
    hh = half.cpu().numpy()
    assert np.array_equal(hh[:rows, :764], x[:, :764].astype(np.float16)) and not hh[:, 764:].any()
    # heads cut out of a wider row (three projections side by side), both output layouts
    B, S, heads, dh = 2, 64, 3, 64
    q = oracle.normal_f32(B * S * 3 * heads * dh, 16).reshape(B * S, 3 * heads * dh)
    dq = to_dev(cuda, q)
    for part, transpose in ((0, 0), (1, 0), (2, 1)):
        oh = cuda.zeros(B * heads * S * dh, dtype=cuda.float16, device="cuda")
        ops.split_heads_f16(dq.data_ptr(), 3 * heads * dh, part * heads * dh, B, S, heads, dh, transpose, oh.data_ptr())
        cuda.cuda.synchronize()
        want = q[:, part * heads * dh:(part + 1) * heads * dh].reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        if transpose:
            want = want.transpose(0, 1, 3, 2)
        assert np.array_equal(oh.cpu().numpy().reshape(want.shape), want.astype(np.float16))


def test_producers_that_write_the_next_operand(cuda, oracle):
    """Normalisation, bias + GELU, softmax and head merge with an fp16 output (the operand of the product that follows),
    and the heads of three projections cut out in one launch: the same values as the two-step forms, rounded once."""
    from tacker_b200 import ops

    rows, cols = 128, 768
    x = oracle.normal_f32(rows * cols, 21).reshape(rows, cols)
    y = oracle.normal_f32(rows * cols, 22).reshape(rows, cols)
    g = oracle.uniform_f32(cols, 5, 0.5, 1.5)
    b = oracle.uniform_f32(cols, 6, -0.5, 0.5)
    dx, dy, dg, db = to_dev(cuda, x), to_dev(cuda, y), to_dev(cuda, g), to_dev(cuda, b)
    out = cuda.zeros((rows, cols), dtype=cuda.float32, device="cuda")
    oh = cuda.zeros((rows, cols), dtype=cuda.float16, device="cuda")
    for res in (dy.data_ptr(), 0):
        ops.add_layernorm_rows_f32(dx.data_ptr(), res, dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, cols, 1e-5,
                                   out_half=oh.data_ptr())
        cuda.cuda.synchronize()
        assert np.array_equal(oh.cpu().numpy(), out.cpu().numpy().astype(np.float16))
        v = (x + y if res else x).astype(np.float64)
        ln = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5) * g + b
        assert np.abs(out.cpu().numpy() - ln).max() < 1e-4
    # the bias of the product that made `a`, folded in: layernorm((a + bias) + res)
    ops.add_layernorm_rows_f32(dx.data_ptr(), dy.data_ptr(), dg.data_ptr(), db.data_ptr(), out.data_ptr(), rows, cols, 1e-5,
                               bias=dg.data_ptr())
    v = ((x + g) + y).astype(np.float64)
    ln = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5) * g + b
    assert np.abs(out.cpu().numpy() - ln).max() < 1e-4
    ops.bias_act_f32(dx.data_ptr(), cols, db.data_ptr(), out.data_ptr(), rows, cols, cols, 2)
    wide = cuda.zeros((rows, 832), dtype=cuda.float16, device="cuda")
    ops.bias_act_f32_f16(dx.data_ptr(), cols, db.data_ptr(), 0, 0, wide.data_ptr(), 832, rows, cols, 2)
    cuda.cuda.synchronize()
    w = wide.cpu().numpy()
    assert np.array_equal(w[:, :cols], out.cpu().numpy().astype(np.float16)) and not w[:, cols:].any()
    both = cuda.zeros((rows, cols), dtype=cuda.float32, device="cuda")
    ops.bias_act_f32_f16(dx.data_ptr(), cols, db.data_ptr(), both.data_ptr(), cols, oh.data_ptr(), cols, rows, cols, 2)
    assert np.array_equal(both.cpu().numpy(), out.cpu().numpy()) and np.array_equal(oh.cpu().numpy(), w[:, :cols])
    sm = cuda.zeros((rows, cols), dtype=cuda.float32, device="cuda")
    ops.softmax_rows_f32(dx.data_ptr(), sm.data_ptr(), rows, cols, 0.5)
    ops.softmax_rows_f16(dx.data_ptr(), oh.data_ptr(), rows, cols, 0.5)
    cuda.cuda.synchronize()
    assert np.array_equal(oh.cpu().numpy(), sm.cpu().numpy().astype(np.float16))
    B, S, heads, dh = 2, 64, 3, 64
    hidden = heads * dh
    qkv = oracle.normal_f32(B * S * 3 * hidden, 23).reshape(B * S, 3 * hidden)
    dq = to_dev(cuda, qkv)
    q, k, vt = (cuda.zeros(B * heads * S * dh, dtype=cuda.float16, device="cuda") for _ in range(3))
    ops.split_qkv_heads_f16(dq.data_ptr(), 3 * hidden, B, S, heads, dh, q.data_ptr(), k.data_ptr(), vt.data_ptr())
    cuda.cuda.synchronize()
    for part, got in enumerate((q, k, vt)):
        want = qkv[:, part * hidden:(part + 1) * hidden].reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        if part == 2:
            want = want.transpose(0, 1, 3, 2)
        assert np.array_equal(got.cpu().numpy().reshape(want.shape), want.astype(np.float16))
    qb = oracle.uniform_f32(3 * hidden, 25, -0.5, 0.5)
    ops.split_qkv_heads_f16(dq.data_ptr(), 3 * hidden, B, S, heads, dh, q.data_ptr(), k.data_ptr(), vt.data_ptr(),
                            bias=to_dev(cuda, qb).data_ptr())
    cuda.cuda.synchronize()
    for part, got in enumerate((q, k, vt)):
        want = (qkv + qb)[:, part * hidden:(part + 1) * hidden].reshape(B, S, heads, dh).transpose(0, 2, 1, 3)
        if part == 2:
            want = want.transpose(0, 1, 3, 2)
        assert np.array_equal(got.cpu().numpy().reshape(want.shape), want.astype(np.float16))
    ctx = oracle.normal_f32(B * heads * S * dh, 24).reshape(B * heads, S, dh)
    mh = cuda.zeros((B * S, hidden), dtype=cuda.float16, device="cuda")
    ops.merge_heads_f16(to_dev(cuda, ctx).data_ptr(), B, S, heads, dh, mh.data_ptr())
    cuda.cuda.synchronize()
    want = ctx.reshape(B, heads, S, dh).transpose(0, 2, 1, 3).reshape(B * S, hidden)
    assert np.array_equal(mh.cpu().numpy(), want.astype(np.float16))


def test_attention_through_batched_tzgemm(cuda, oracle):
    """softmax(Q K^T / sqrt(d)) V for B*heads independent heads: split, two batched tzgemms, merge."""
    from tacker_b200 import ops

    B, S, heads, dh = 2, 128, 3, 64
    hidden, bh = heads * dh, B * heads
    q, k, v = (oracle.normal_f32(B * S * hidden, s).reshape(B * S, hidden) * 0.5 for s in (11, 12, 13))
    dq, dk, dv = to_dev(cuda, q), to_dev(cuda, k), to_dev(cuda, v)
    qh = cuda.zeros((bh, S, dh), dtype=cuda.float16, device="cuda")
    kh = cuda.zeros((bh, S, dh), dtype=cuda.float16, device="cuda")
    vt = cuda.zeros((bh, dh, S), dtype=cuda.float16, device="cuda")
    ops.split_heads_f16(dq.data_ptr(), hidden, 0, B, S, heads, dh, 0, qh.data_ptr())
    ops.split_heads_f16(dk.data_ptr(), hidden, 0, B, S, heads, dh, 0, kh.data_ptr())
    ops.split_heads_f16(dv.data_ptr(), hidden, 0, B, S, heads, dh, 1, vt.data_ptr())
    scores = cuda.zeros((bh, S, S), dtype=cuda.float32, device="cuda")
    ops.tzgemm_batched(qh.data_ptr(), kh.data_ptr(), scores.data_ptr(), S, S, dh, bh, alpha=1.0 / 8.0)
    ops.softmax_rows_f32(scores.data_ptr(), scores.data_ptr(), bh * S, S, 1.0)
    ph = cuda.zeros((bh, S, S), dtype=cuda.float16, device="cuda")
    ops.rows_f32_to_f16(scores.data_ptr(), bh * S, S, S, ph.data_ptr(), bh * S, S)
    ctx = cuda.zeros((bh, S, dh), dtype=cuda.float32, device="cuda")
    ops.tzgemm_batched(ph.data_ptr(), vt.data_ptr(), ctx.data_ptr(), S, dh, S, bh, alpha=1.0)
    merged = cuda.zeros((B * S, hidden), dtype=cuda.float32, device="cuda")
    ops.merge_heads_f32(ctx.data_ptr(), B, S, heads, dh, merged.data_ptr())
    cuda.cuda.synchronize()
    assert ops.device_status() == 0
    f16 = lambda a: a.astype(np.float16).astype(np.float64)
    want = np.zeros((B * S, hidden))
    for b_ in range(B):
        for h in range(heads):
            sl = slice(b_ * S, (b_ + 1) * S), slice(h * dh, (h + 1) * dh)
            s_ = f16(q[sl]) @ f16(k[sl]).T / 8.0
            p = np.exp(s_ - s_.max(1, keepdims=True))
            p /= p.sum(1, keepdims=True)
            want[sl] = f16(p) @ f16(v[sl])
    assert np.abs(merged.cpu().numpy() - want).max() <= 2e-3


def test_batched_tzgemm_matches_loop(cuda, oracle):
    from tacker_b200 import ops

    M, N, K, batch = 128, 192, 128, 5
    a_bits, a = oracle.uniform_f16(batch * M * K, 21, -1.0, 1.0)
    b_bits, b = oracle.uniform_f16(batch * N * K, 22, -1.0, 1.0)
    dA = cuda.from_numpy(a_bits.view(np.float16)).cuda()
    dB = cuda.from_numpy(b_bits.view(np.float16)).cuda()
    dC = cuda.full((batch, M, N), float("nan"), dtype=cuda.float32, device="cuda")
    ops.tzgemm_batched(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K, batch, alpha=1.1)
    cuda.cuda.synchronize()
    got = dC.cpu().numpy()
    a, b = a.reshape(batch, M, K), b.reshape(batch, N, K)
    for i in range(batch):
        want = oracle.tzgemm_f64(a[i], b[i], alpha=1.1)
        assert np.abs(got[i] - want).max() <= 1e-3 * K
