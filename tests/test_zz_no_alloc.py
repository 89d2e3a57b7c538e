"""GPU test of simp_gpu_matmul_w4_noalloc, the W4 GEMV entry point for callers that may not allocate device
memory when they call the library (a serving process whose own pool took the whole memory budget at start-up,
or code running where the CUDA runtime forbids allocation).  The W4 kernels keep everything they stage in
shared memory, so the entry point has no scratch in global memory; what it adds is that it never initialises
the library on demand and that it refuses rows longer than its documented limit.

It is called through the C-ABI several times in a row with different shapes, and each result is compared
both with the regular entry point's on the same inputs (same kernels: equal to rounding) and with the CPU oracle
(the W4 tolerance of 1e-3 against the largest output).  The file name sorts last so that, if this addition
ever fails, a run that stops at the first failure has already covered everything else.
"""
import ctypes as C

import numpy as np
import pytest

import oracle

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
    want = oracle.matmul_quant(q, sc, zr, x, rows, cols, gs, 0, scale_mode=1, threads=0)
    err = np.max(np.abs(b - want)) / np.max(np.abs(want))
    print(f"w4_noalloc {rows}x{cols} gs {gs}: max error vs oracle / max|oracle| = {err:.2e}")
    assert err <= 1e-3


def test_two_calls_in_a_row_match_the_regular_entry_point(gpu):
    rng = np.random.default_rng(2024)
    _case(gpu, rng, 3200, 8640, 64, True)
    _case(gpu, rng, 1000, 3200, 64, False)   # a shorter input right after a longer one
    _case(gpu, rng, 96, 16384, 128, True)    # exactly the maximum row length
    _case(gpu, rng, 40, 16384, 32, False)    # too long for the shared-memory pipeline: the general kernel


def test_rejects_what_it_cannot_hold(gpu):
    d = gpu.DeviceBuffer(64)
    rc = gpu.lib().simp_gpu_matmul_w4_noalloc(d.ptr, d.ptr, None, d.ptr, d.ptr, 4, 16384 + 64, 64, 0, 1)
    assert rc != 0 and b"exceeds" in gpu.lib().simp_gpu_last_error()
