"""GPU parity of the reference-facing layer: host-pointer entry points (simp_host_*) and the memref-ABI shims
(simp_rt_*) a compiled .sl kernel would call, checked against the CPU oracle on host arrays.  Also the
resident-operand registry."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
i64 = C.c_int64


def memref1(a, off=0):
    """(allocated, aligned, offset, size, stride) of a contiguous 1-D numpy array."""
    p = C.c_void_p(a.ctypes.data)
    return [p, p, i64(off), i64(a.size), i64(1)]


def memref2(a):
    p = C.c_void_p(a.ctypes.data)
    return [p, p, i64(0), i64(a.shape[0]), i64(a.shape[1]), i64(a.shape[1]), i64(1)]


def test_shim_rmsnorm_softmax_silu(gpu, oracle):
    L = gpu.lib()
    rng = np.random.default_rng(0)
    n = 768
    x = rng.standard_normal(n).astype(np.float32)
    w = (1 + 0.02 * rng.standard_normal(3 * n)).astype(np.float32)
    y = np.zeros(n, np.float32)
    gpu.check(L.simp_rt_rmsnorm_f32(*memref1(x), *memref1(w), *memref1(y), i64(n), C.c_float(1e-5), i64(n)))
    assert np.allclose(y, oracle.rmsnorm(x, w, 1e-5, n), rtol=1e-4, atol=1e-6)
    att = (3 * rng.standard_normal(4 * 64)).astype(np.float32)
    soft = np.zeros_like(att)
    gpu.check(L.simp_rt_softmax_f32(*memref1(att), *memref1(soft), i64(37), i64(64), i64(64)))
    ref = np.zeros_like(att)
    oracle.softmax(att, 37, 64, 64, out=ref)
    assert np.allclose(soft, ref, rtol=1e-4, atol=1e-9)
    h = rng.standard_normal(2048).astype(np.float32)
    hs = np.zeros_like(h)
    gpu.check(L.simp_rt_silu_f32(*memref1(h), *memref1(hs), i64(2048)))
    assert np.allclose(hs, oracle.silu(h), rtol=1e-4, atol=1e-7)


def test_shim_matmul_accumulates_with_offsets(gpu, oracle):
    # the stories110M call shape: matmul(wq, xb, q, 768, 768, 1, layer_offset, 0, 0) on a zeroed q
    L = gpu.lib()
    rng = np.random.default_rng(1)
    dim, layer = 768, 2
    wq = (0.02 * rng.standard_normal(3 * dim * dim)).astype(np.float32)
    xb = rng.standard_normal(dim).astype(np.float32)
    q = np.full(dim, 0.5, np.float32)
    ref = q.copy()
    oracle.matmul_f32(wq, layer * dim * dim, xb, 0, ref, 0, dim, dim, 1)
    gpu.check(L.simp_rt_matmul_f32(*memref1(wq), *memref1(xb), *memref1(q), i64(dim), i64(dim), i64(1),
                                   i64(layer * dim * dim), i64(0), i64(0)))
    assert np.max(np.abs(q - ref)) <= 1e-4 * np.max(np.abs(ref))


def test_shim_matmul_quant_is_the_op_as_lowered(gpu, oracle):
    L = gpu.lib()
    rng = np.random.default_rng(2)
    rows, cols, gs = 64, 1536, 128
    qw, sc, zr = oracle.quantize_w4((0.02 * rng.standard_normal(2 * rows * cols)).astype(np.float32), gs)
    x = rng.standard_normal(cols).astype(np.float32)
    out = np.zeros(rows, np.float32)
    off = rows * cols  # second matrix: the lowering still reads matrix 0's scales
    gpu.check(L.simp_rt_matmul_quant(*memref1(qw.view(np.int8)), *memref1(sc), *memref1(zr), *memref1(x), *memref1(out),
                                     i64(rows), i64(cols), i64(gs), i64(off)))
    ref = oracle.matmul_quant(qw, sc, zr, x, rows, cols, gs, off, scale_mode=0)
    assert np.max(np.abs(out - ref)) <= 1e-3 * np.max(np.abs(ref))


@pytest.mark.parametrize("nt", [False, True])
def test_shim_tensor_matmul_i8(gpu, oracle, nt):
    L = gpu.lib()
    rng = np.random.default_rng(3)
    M, K, N = 192, 320, 272
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (N, K) if nt else (K, N), dtype=np.int8)
    Cm = np.zeros((M, N), np.int32)
    fn = L.simp_rt_tensor_matmul_nt_i8 if nt else L.simp_rt_tensor_matmul_i8
    gpu.check(fn(*memref2(A), *memref2(B), *memref2(Cm)))
    assert np.array_equal(Cm, oracle.tensor_matmul_i8(A, B, b_transposed=nt))
    # a shape mismatch is an error status, not a crash
    assert fn(*memref2(A), *memref2(B[:-1]), *memref2(Cm)) != 0


def test_shim_tensor_matmul_f32_known_answer(gpu):
    # tests/test_tensor_matmul.sl:4-65 -> C[0,0] = 22
    L = gpu.lib()
    A = (np.arange(12, dtype=np.float32) + 1).reshape(4, 3)
    B = (np.arange(6, dtype=np.float32) + 1).reshape(3, 2)
    Cm = np.full((4, 2), -1, np.float32)
    gpu.check(L.simp_rt_tensor_matmul_f32(*memref2(A), *memref2(B), *memref2(Cm)))
    assert Cm[0, 0] == 22.0 and np.array_equal(Cm, A @ B)


def test_host_gemm_chunked_pipeline_and_registered_weights(gpu, oracle):
    rng = np.random.default_rng(4)
    M, K, N = 2500, 512, 1024  # > 8 MB of C: several row chunks, ragged last chunk
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    Bt = rng.integers(-128, 128, (N, K), dtype=np.int8)
    ref = oracle.tensor_matmul_i8(A, Bt, b_transposed=True)
    assert np.array_equal(gpu.host_tensor_matmul_i8(A, Bt, b_transposed=True), ref)
    gpu.check(gpu.lib().simp_gpu_register_host(Bt.ctypes.data, Bt.nbytes))
    try:
        Bt_host_copy = Bt.copy()
        Bt[...] = 0  # resident copy is used: changing the host array after registration has no effect
        assert np.array_equal(gpu.host_tensor_matmul_i8(A, Bt, b_transposed=True), ref)
        Bt[...] = Bt_host_copy
    finally:
        gpu.check(gpu.lib().simp_gpu_unregister_host(Bt.ctypes.data))
    assert gpu.lib().simp_gpu_unregister_host(Bt.ctypes.data) != 0


@pytest.mark.parametrize("nt", [False, True])
@pytest.mark.parametrize("a_dtype", [np.uint8, np.int8])
def test_host_gemm_blocked_pipeline(gpu, oracle, nt, a_dtype):
    """Large host-to-host products are cut into row chunks x column blocks of C (uploads ordered so that the first block
    leaves early): ragged last row chunk, both layouts of B, pageable and pinned host buffers."""
    rng = np.random.default_rng(14)
    M, K, N = 2100, 4096, 4096   # 16 MB of B: 9 row chunks (the last one ragged) x 4 column blocks
    lo, hi = (0, 256) if a_dtype == np.uint8 else (-128, 128)
    A = rng.integers(lo, hi, (M, K)).astype(a_dtype)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    Bg = np.ascontiguousarray(B.T) if nt else B
    ref = oracle.tensor_matmul_i8(A, Bg, b_transposed=nt)
    assert np.array_equal(gpu.host_tensor_matmul_i8(A, Bg, b_transposed=nt), ref)
    Ap, Bp, Cp = gpu.pinned_empty(A.shape, A.dtype), gpu.pinned_empty(Bg.shape, Bg.dtype), gpu.pinned_empty((M, N), np.int32)
    Ap[...] = A
    Bp[...] = Bg
    Cp[...] = -1
    assert np.array_equal(gpu.host_tensor_matmul_i8(Ap, Bp, out=Cp, b_transposed=nt), ref)


def test_cpp_host_driver(gpu):
    """The C++ host (GpuKernelRunner / ProfiledGpuKernelRunner) loads the library, runs and verifies a GEMM."""
    import os
    import subprocess
    from simplang_b200 import build as b
    exe = b.build_host()
    r = subprocess.run([exe, gpu.LIB_PATH, "256", "512", "384", "5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "verification passed" in r.stdout and "GIOP/s" in r.stdout
    r = subprocess.run([exe, os.path.join(os.path.dirname(gpu.LIB_PATH), "missing.so")], capture_output=True, text=True)
    assert r.returncode == 1 and "Failed to load library" in r.stderr


def test_record_and_replay(gpu, oracle):
    """A recorded sequence of device-pointer calls replays with the results of the direct calls."""
    rng = np.random.default_rng(5)
    M, K, N = 96, 256, 160
    A = rng.integers(0, 256, (M, K), dtype=np.uint8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(B)
    dC = gpu.DeviceBuffer(M * N * 4)
    x = rng.standard_normal(4096).astype(np.float32)
    dx, dy = gpu.DeviceBuffer.from_numpy(x), gpu.DeviceBuffer(x.nbytes)
    # run once first (first calls of an op family set kernel attributes, which a recording may not do)
    gpu.matmul_i8(dA, dB, dC, M, K, N, a_unsigned=True, b_transposed=False)
    gpu.silu_f32(dx, None, dy, x.size)
    gpu.check(gpu.lib().simp_gpu_memset(dC.ptr, 0, dC.nbytes))
    gpu.check(gpu.lib().simp_gpu_memset(dy.ptr, 0, dy.nbytes))
    gpu.sync()
    with gpu.Recording() as rec:
        gpu.matmul_i8(dA, dB, dC, M, K, N, a_unsigned=True, b_transposed=False)
        gpu.silu_f32(dx, None, dy, x.size)
    gpu.sync()
    assert not dC.to_numpy(np.int32, (M, N)).any()      # recording does not execute
    rec.replay(3)
    gpu.sync()
    assert np.array_equal(dC.to_numpy(np.int32, (M, N)), oracle.tensor_matmul_i8(A, B))
    ref = oracle.silu(x)
    assert np.max(np.abs(dy.to_numpy(np.float32, x.shape) - ref)) <= 1e-4 * np.max(np.abs(ref))
    rec.close()
