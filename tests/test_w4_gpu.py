"""GPU parity: matmul_quant / dequant_w4 vs the CPU oracle.

Tolerance (north star): relative error 1e-3 for W4.  Two readings are asserted: against sum_k |w_k * x_k| of the
row, and the stricter max|out - ref| <= 1e-3 * max|ref| over the whole result (the one the model tests use).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def make(rng, total, gs, symmetric):
    w = (0.02 * rng.standard_normal(total)).astype(np.float32)
    if symmetric:
        g = w.reshape(-1, gs)
        scale = (np.abs(g).max(axis=1) / 7.0).astype(np.float32)
        scale[scale < 1e-8] = 1e-8
        q = np.clip(np.rint(g / scale[:, None]), -8, 7).astype(np.int32) + 8
        q = q.reshape(-1)
        qw = (q[0::2] | (q[1::2] << 4)).astype(np.uint8)
        return qw, scale, None
    import oracle
    return oracle.quantize_w4(w, gs)


def row_scale(oracle, qw, sc, zr, x, rows, cols, gs, offset):
    zr_ = zr if zr is not None else (-8 * sc).astype(np.float32)
    w = oracle.dequant_w4(qw, sc, zr_, offset, rows * cols, gs).reshape(rows, cols)
    return np.abs(w.astype(np.float64)) @ np.abs(x.astype(np.float64)) + 1e-30


@pytest.mark.parametrize("rows,cols,gs", [(3200, 3200, 64), (8640, 3200, 64), (3200, 8640, 64), (1536, 1536, 128),
                                          (100, 256, 32), (7, 128, 128), (33, 1024, 256), (9600, 3200, 32),
                                          # chunk counts that leave a partial 128-weight span; enough rows for 32-row tiles
                                          (50, 160, 32), (40, 224, 32), (12000, 512, 64), (20001, 1024, 128)])
@pytest.mark.parametrize("symmetric", [True, False])
def test_matmul_w4_per_matrix(gpu, oracle, rows, cols, gs, symmetric):
    rng = np.random.default_rng(rows + cols + gs)
    offset = 2 * gs * 5  # a second matrix inside the shared byte array
    qw, sc, zr = make(rng, offset + rows * cols, gs, symmetric)
    x = rng.standard_normal(cols).astype(np.float32)
    d = [gpu.DeviceBuffer.from_numpy(a) if a is not None else None for a in (qw, sc, zr, x)]
    dout = gpu.DeviceBuffer(rows * 4)
    gpu.matmul_w4(d[0], d[1], d[2], d[3], dout, rows, cols, gs, offset, scale_mode=1)
    out = dout.to_numpy(np.float32, rows)
    ref = oracle.matmul_quant(qw, sc, zr, x, rows, cols, gs, offset, scale_mode=1, threads=0)
    err = np.abs(out.astype(np.float64) - ref) / row_scale(oracle, qw, sc, zr, x, rows, cols, gs, offset)
    assert err.max() <= 1e-3, err.max()
    top = np.max(np.abs(out - ref)) / (np.max(np.abs(ref)) + 1e-30)
    print(f"w4 {rows}x{cols} gs {gs} sym {symmetric}: max error / row scale = {err.max():.2e}, / max|ref| = {top:.2e}")
    assert top <= 1e-3, top


@pytest.mark.parametrize("rows,cols,gs,offset", [(1536, 1536, 128, 0), (64, 1536, 128, 1536 * 1536), (10, 200, 64, 0),
                                                 (9, 320, 32, 64), (5, 8640, 128, 0), (6, 130, 128, 1)])
def test_matmul_w4_reference_mode(gpu, oracle, rows, cols, gs, offset):
    """scale_mode 0 reproduces the lowering literally, including its group quirks."""
    rng = np.random.default_rng(rows + cols)
    total = offset + rows * cols + 256
    qw, sc, zr = oracle.quantize_w4((0.02 * rng.standard_normal(total)).astype(np.float32), gs)
    x = rng.standard_normal(cols).astype(np.float32)
    d = [gpu.DeviceBuffer.from_numpy(a) for a in (qw, sc, zr, x)]
    dout = gpu.DeviceBuffer(rows * 4)
    gpu.matmul_w4(d[0], d[1], d[2], d[3], dout, rows, cols, gs, offset, scale_mode=0)
    out = dout.to_numpy(np.float32, rows)
    ref = oracle.matmul_quant(qw, sc, zr, x, rows, cols, gs, offset, scale_mode=0)
    scale = np.abs(ref).max() + 1e-30
    assert np.max(np.abs(out - ref)) <= 1e-3 * scale


def test_dequant_w4_range(gpu, oracle):
    rng = np.random.default_rng(3)
    qw, sc, zr = oracle.quantize_w4(rng.standard_normal(4096).astype(np.float32), 128)
    d = [gpu.DeviceBuffer.from_numpy(a) for a in (qw, sc, zr)]
    dout = gpu.DeviceBuffer(1000 * 4)
    gpu.dequant_w4(d[0], d[1], d[2], 37, 1000, 128, dout)
    assert np.array_equal(dout.to_numpy(np.float32, 1000), oracle.dequant_w4(qw, sc, zr, 37, 1000, 128))


def test_bad_arguments(gpu):
    with pytest.raises(gpu.SimpGpuError):
        gpu.matmul_w4(1, 1, None, 1, 1, 4, 100, 64, 0, scale_mode=1)  # cols % gs != 0
    with pytest.raises(gpu.SimpGpuError):
        gpu.matmul_w4(1, 1, None, 1, 1, 4, 128, 0, 0, scale_mode=0)  # gs == 0
