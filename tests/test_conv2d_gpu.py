"""GPU parity: conv2d (NHWC, weights [OC, KH, KW, IC]) against the CPU oracle -- bit-exact, since taps accumulate in
the same order with separate multiply and add -- and the reference's known answer."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_known_answer(gpu):
    x = np.arange(16, dtype=np.float32).reshape(1, 4, 4, 1)
    w = np.ones((1, 3, 3, 1), np.float32)
    b = np.zeros(1, np.float32)
    assert gpu.np_conv2d_f32(x, w, b, (1, 1), (0, 0))[0, 0, 0, 0] == 45.0     # test_conv2d_host.cpp:31-36
    assert gpu.np_conv2d_f32(x, w, b, (1, 1), (1, 1))[0, 1, 1, 0] == 45.0


@pytest.mark.parametrize("n,h,w,ic,oc,kh,kw,stride,pad", [
    (1, 5, 6, 3, 4, 3, 3, (1, 1), (1, 1)), (2, 9, 7, 2, 5, 3, 2, (2, 1), (0, 1)), (1, 8, 8, 4, 3, 1, 1, (1, 1), (0, 0)),
    (1, 7, 7, 1, 2, 5, 5, (2, 2), (2, 2)),
    (1, 224, 224, 3, 32, 3, 3, (2, 2), (1, 1)),      # MobileNetV2 stem (mobilenet_poc/mobilenetv2_full.sl:110-112)
    (1, 112, 112, 32, 16, 1, 1, (1, 1), (0, 0)),     # a pointwise layer of the same model (:511-513)
])
def test_against_oracle(gpu, oracle, n, h, w, ic, oc, kh, kw, stride, pad):
    rng = np.random.default_rng(h * 31 + ic)
    x = rng.standard_normal((n, h, w, ic)).astype(np.float32)
    wt = rng.standard_normal((oc, kh, kw, ic)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32)
    out = gpu.np_conv2d_f32(x, wt, b, stride, pad)
    ref = oracle.conv2d_f32(x, wt, b, stride, pad)
    assert out.shape == ref.shape
    assert np.array_equal(out, ref)


def test_errors(gpu):
    x = np.zeros((1, 2, 2, 1), np.float32)
    with pytest.raises(gpu.SimpGpuError):
        gpu.np_conv2d_f32(x, np.zeros((1, 3, 3, 1), np.float32), np.zeros(1, np.float32))   # kernel larger than the input
