"""im2col and the fp32 -> fp16 cast through the C ABI against the CPU checker (B200 only): bit-exact."""
import numpy as np
import pytest

from helpers import to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [
    (3, 9, 7, 3, 3, 1, 1, 2, 1, 1, 1),
    (4, 16, 16, 3, 3, 1, 1, 1, 1, 1, 1),
    (2, 11, 13, 5, 3, 2, 0, 2, 3, 1, 2),
    (64, 56, 56, 3, 3, 1, 1, 1, 1, 1, 1),        # a VGG16 conv3 block at batch 1
    (3, 224, 224, 3, 3, 1, 1, 1, 1, 1, 1),       # VGG16 conv1_1
    (8, 14, 14, 1, 1, 0, 0, 1, 1, 1, 1),
])
def test_im2col_bit_exact(cuda, oracle, cfg):
    from tacker_b200 import ops

    c, h, w, kh, kw, ph, pw, sh, sw, dh, dw = cfg
    im = oracle.uniform_f32(c * h * w, 31, -1.0, 1.0).reshape(c, h, w)
    want = oracle.im2col_f32(im, kh, kw, ph, pw, sh, sw, dh, dw)
    d_im = to_dev(cuda, im)
    d_col = cuda.full(want.shape, float("nan"), dtype=cuda.float32, device="cuda")
    ops.im2col_f32(d_im.data_ptr(), c, h, w, kh, kw, ph, pw, sh, sw, dh, dw, d_col.data_ptr())
    cuda.cuda.synchronize()
    assert oracle.bit_mismatches(d_col.cpu().numpy(), want) == 0


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 1 << 20, (1 << 20) + 3])
def test_cast_bit_exact(cuda, oracle, n):
    from tacker_b200 import ops

    x = oracle.normal_f32(n, 5, 0.0, 30.0)
    x[:: 97] *= 1e-6
    if n > 10:
        x[7] = 70000.0
        x[9] = -1e-9
    d_in = to_dev(cuda, x)
    d_out = cuda.zeros(n, dtype=cuda.float16, device="cuda")
    ops.convert_fp32_to_fp16(d_out.data_ptr(), d_in.data_ptr(), n)
    cuda.cuda.synchronize()
    got = d_out.cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.f32_to_f16_bits(x))


def test_conv_shape_rule(cuda):
    from tacker_b200 import ops

    assert ops.conv_mnk([1, 64, 224, 224, 64, 64, 3, 3, 1, 1, 1, 1, 1, 1]) == (50176, 64, 576)
    assert ops.tzgemm_dims(50176, 64, 576) == (50176, 128, 512, 784 * 2)
