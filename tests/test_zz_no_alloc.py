"""GPU test of simp_gpu_matmul_w4_noalloc, the W4 GEMV variant for callers that cannot allocate device
memory (its packed-input scratch is a fixed array inside the library, not the growable arena).

It is called through the C-ABI twice in a row with different inputs -- the array is shared and keeps the
previous call's contents, so the second call proves nothing stale leaks through -- and each result is
compared with the regular entry point's on the same inputs (same kernels, so the W4 tolerance of 1e-3 is
met with a wide margin).  The file name sorts last so that, if this addition ever fails, a run that stops at
the first failure has already covered everything else.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(gpu, rng, rows, cols, gs, symmetric):
    q = rng.integers(0, 256, rows * cols // 2, dtype=np.uint8)
    sc = (0.005 + 0.01 * rng.random(rows * cols // gs)).astype(np.float32)
    zr = None if symmetric else (-0.08 * rng.random(rows * cols // gs)).astype(np.float32)
    x = rng.standard_normal(cols).astype(np.float32)
    d = [gpu.DeviceBuffer.from_numpy(a) if a is not None else None for a in (q, sc, zr, x)]
    ref_out, new_out = gpu.DeviceBuffer(rows * 4), gpu.DeviceBuffer(rows * 4)
    zp = d[2].ptr if d[2] is not None else None
    gpu.matmul_w4(d[0], d[1], d[2], d[3], ref_out, rows, cols, gs, 0, scale_mode=1)
    gpu.check(gpu.lib().simp_gpu_matmul_w4_noalloc(d[0].ptr, d[1].ptr, zp, d[3].ptr, new_out.ptr, rows, cols, gs, 0, 1))
    a, b = ref_out.to_numpy(np.float32, rows), new_out.to_numpy(np.float32, rows)
    assert np.all(np.isfinite(b))
    assert np.max(np.abs(a - b)) <= 1e-3 * np.max(np.abs(a))


def test_two_calls_in_a_row_match_the_regular_entry_point(gpu):
    rng = np.random.default_rng(2024)
    _case(gpu, rng, 3200, 8640, 64, True)    # fills most of the built-in scratch
    _case(gpu, rng, 1000, 3200, 64, False)   # shorter input right after: stale tail must not matter
    _case(gpu, rng, 96, 16384, 128, True)    # exactly the maximum


def test_rejects_what_it_cannot_hold(gpu):
    d = gpu.DeviceBuffer(64)
    rc = gpu.lib().simp_gpu_matmul_w4_noalloc(d.ptr, d.ptr, None, d.ptr, d.ptr, 4, 16384 + 64, 64, 0, 1)
    assert rc != 0 and b"exceeds" in gpu.lib().simp_gpu_last_error()
