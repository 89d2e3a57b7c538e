"""GPU parity: rmsnorm / softmax / silu / int8 quantise-dequantise vs the CPU oracle.

Tolerance: max relative error 1e-4 for f32 ops (the north-star bound), measured as
|gpu - ref| <= 1e-4 * max(|ref|, floor) with a small absolute floor for values near zero;
bit-exact for the integer results.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RTOL = 1e-4


def close(a, b, rtol=RTOL, floor=1e-6):
    return np.all(np.abs(a - b) <= rtol * np.maximum(np.abs(b), floor) + 1e-9)


@pytest.mark.parametrize("rows,n", [(1, 768), (1, 3200), (1, 4096), (7, 768), (64, 3200), (512, 4096), (4096, 768),
                                    (3, 4), (2, 1), (5, 770), (2, 8200), (1, 33), (3, 16384)])
def test_rmsnorm(gpu, oracle, rows, n):
    rng = np.random.default_rng(rows * 131 + n)
    x = rng.standard_normal((rows, n)).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(n + 5)).astype(np.float32)
    woff = 4 if n % 4 == 0 else 5
    dx, dw = gpu.DeviceBuffer.from_numpy(x), gpu.DeviceBuffer.from_numpy(w)
    dy = gpu.DeviceBuffer(x.nbytes)
    gpu.rmsnorm_f32(dx, dw, dy, rows, n, 1e-5, woff, n)
    y = dy.to_numpy(np.float32, (rows, n))
    ref = np.stack([oracle.rmsnorm(x[r], w, 1e-5, woff) for r in range(rows)])
    assert close(y, ref)


def test_rmsnorm_residual_fused(gpu, oracle):
    rng = np.random.default_rng(5)
    rows, n = 9, 3200
    x = rng.standard_normal((rows, n)).astype(np.float32)
    res = rng.standard_normal((rows, n)).astype(np.float32)
    w = np.ones(n, np.float32)
    dx, dr, dw = (gpu.DeviceBuffer.from_numpy(a) for a in (x, res, w))
    dy = gpu.DeviceBuffer(x.nbytes)
    gpu.rmsnorm_f32(dx, dw, dy, rows, n, 1e-5, 0, n, residual=dr)
    xs = x + res
    assert np.array_equal(dx.to_numpy(np.float32, (rows, n)), xs)
    ref = np.stack([oracle.rmsnorm(xs[r], w) for r in range(rows)])
    assert close(dy.to_numpy(np.float32, (rows, n)), ref)


def test_rmsnorm_known_answer(gpu):
    # examples/llama2/kernels/test_rmsnorm.sl:13-39: x=[1,2,3,4], w=1 -> y[0] = 1/sqrt(7.5+1e-5)
    dx = gpu.DeviceBuffer.from_numpy(np.array([1, 2, 3, 4], np.float32))
    dw = gpu.DeviceBuffer.from_numpy(np.ones(4, np.float32))
    dy = gpu.DeviceBuffer(16)
    gpu.rmsnorm_f32(dx, dw, dy, 1, 4)
    y = dy.to_numpy(np.float32, 4)
    assert abs(y[0] - 1 / np.sqrt(7.5 + 1e-5)) < 1e-4


@pytest.mark.parametrize("rows,n", [(1, 32), (1, 1), (12, 17), (12, 1024), (64, 4096), (4096, 32), (1024, 2048),
                                    (3, 1000), (2, 8196), (5, 333)])
def test_softmax(gpu, oracle, rows, n):
    rng = np.random.default_rng(rows * 7 + n)
    stride = n + (4 if n % 4 == 0 else 3)
    x = (3 * rng.standard_normal(rows * stride + 8)).astype(np.float32)
    off = 4 if n % 4 == 0 else 1
    dx = gpu.DeviceBuffer.from_numpy(x)
    dy = gpu.DeviceBuffer(x.nbytes)
    dy.zero()
    gpu.softmax_f32(dx, dy, rows, n, off, off, stride)
    y = dy.to_numpy(np.float32, x.size)
    ref = np.zeros_like(x)
    for r in range(rows):
        oracle.softmax(x, n, off + r * stride, off + r * stride, out=ref)
    assert close(y, ref, floor=1e-12)
    for r in range(rows):
        assert abs(y[off + r * stride: off + r * stride + n].sum() - 1) < 1e-4


def test_softmax_known_answer(gpu):
    # examples/llama2/kernels/test_softmax_host.cpp:34-38
    dx = gpu.DeviceBuffer.from_numpy(np.array([1, 2, 3, 4], np.float32))
    dy = gpu.DeviceBuffer(16)
    gpu.softmax_f32(dx, dy, 1, 4)
    e = np.exp(np.array([-3., -2., -1., 0.]))
    assert abs(dy.to_numpy(np.float32, 4)[0] - e[0] / e.sum()) < 1e-4


@pytest.mark.parametrize("n", [1, 3, 2048, 8640, 4096 * 768, 1000003])
@pytest.mark.parametrize("fused", [False, True])
def test_silu(gpu, oracle, n, fused):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32) * 3
    m = rng.standard_normal(n).astype(np.float32) if fused else None
    dx = gpu.DeviceBuffer.from_numpy(x)
    dm = gpu.DeviceBuffer.from_numpy(m) if fused else None
    dy = gpu.DeviceBuffer(x.nbytes)
    gpu.silu_f32(dx, dm, dy, n)
    assert close(dy.to_numpy(np.float32, n), oracle.silu(x, m), floor=1e-7)


def test_silu_known_answers(gpu):
    # test_silu_host.cpp:31-36 silu(1.0); test_swiglu_host.cpp:33-41 silu(0.5)*2
    dx = gpu.DeviceBuffer.from_numpy(np.array([1.0, 0.5], np.float32))
    dm = gpu.DeviceBuffer.from_numpy(np.array([1.0, 2.0], np.float32))
    dy = gpu.DeviceBuffer(8)
    gpu.silu_f32(dx, dm, dy, 2)
    y = dy.to_numpy(np.float32, 2)
    assert abs(y[0] - 1 / (1 + np.exp(-1.0))) < 1e-4
    assert abs(y[1] - 2 * 0.5 / (1 + np.exp(-0.5))) < 1e-4


@pytest.mark.parametrize("n", [1, 5, 4096, 100001])
@pytest.mark.parametrize("clamp", [True, False])
def test_quantize_i8(gpu, oracle, n, clamp):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * (1.5 if clamp else 0.4)).astype(np.float32)
    x[:: 7] = np.round(x[:: 7] * 127) / 127  # values on the truncation boundary
    dx = gpu.DeviceBuffer.from_numpy(x)
    dy = gpu.DeviceBuffer(max(n, 16))
    gpu.quantize_i8(dx, dy, n, 127.0, clamp)
    assert np.array_equal(dy.to_numpy(np.int8, n), oracle.quantize_i8(x, 127.0, clamp))


@pytest.mark.parametrize("n", [1, 6, 3200, 70001])
def test_dequantize_i32(gpu, oracle, n):
    rng = np.random.default_rng(n)
    a = rng.integers(-2**31, 2**31 - 1, n, dtype=np.int64).astype(np.int32)
    da = gpu.DeviceBuffer.from_numpy(a)
    dy = gpu.DeviceBuffer(max(4 * n, 16))
    gpu.dequantize_i32(da, dy, n, 65536.0)
    assert np.array_equal(dy.to_numpy(np.float32, n), oracle.dequantize_i32(a, 65536.0))


def test_empty_and_bad_arguments(gpu):
    gpu.silu_f32(None, None, None, 0)
    gpu.rmsnorm_f32(None, None, None, 0, 0)
    with pytest.raises(gpu.SimpGpuError):
        gpu.silu_f32(None, None, None, 8)
    with pytest.raises(gpu.SimpGpuError):
        gpu.softmax_f32(None, None, 1, -1)
