"""GPU parity: simp.matmul / tensor_matmul on f32 vs the CPU oracle.

Tolerance (north star): max relative error 1e-4.  Two readings are asserted: against the row's scale
sum_p |A[i,p]*B[p,j]| (the natural bound for a dot product whose summation order differs), and the stricter
max|out - ref| <= 1e-4 * max|ref| over the whole result (skipped only for results of fewer than 16 elements,
where one cancelling dot product decides max|ref|).  Both against an f64 product and the sequential-f32 oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def check(gpu_out, A, B, ref32):
    A64, B64 = A.astype(np.float64), B.astype(np.float64)
    exact = A64 @ B64
    scale = np.abs(A64) @ np.abs(B64) + 1e-30
    assert np.max(np.abs(gpu_out - exact) / scale) <= 1e-4
    assert np.max(np.abs(gpu_out - ref32) / scale) <= 1e-4
    top = np.max(np.abs(exact))
    e64, e32 = np.max(np.abs(gpu_out - exact)) / (top + 1e-30), np.max(np.abs(gpu_out - ref32)) / (top + 1e-30)
    print(f"f32 matmul {A.shape}x{B.shape}: max error / max|ref| = {e64:.2e} (f64), {e32:.2e} (f32 oracle)")
    if exact.size >= 16:
        assert e64 <= 1e-4 and e32 <= 1e-4


@pytest.mark.parametrize("m,k", [(768, 768), (2048, 768), (768, 2048), (32000, 768), (3200, 8640), (5, 12), (33, 770),
                                 (1, 4), (100, 3)])
@pytest.mark.parametrize("accumulate", [True, False])
def test_gemv(gpu, oracle, m, k, accumulate):
    rng = np.random.default_rng(m + k)
    aoff, coff = 8, 3
    A = (0.02 * rng.standard_normal(aoff + m * k)).astype(np.float32)
    x = rng.standard_normal(k).astype(np.float32)
    c0 = rng.standard_normal(coff + m).astype(np.float32)
    dA, dx, dC = (gpu.DeviceBuffer.from_numpy(a) for a in (A, x, c0))
    gpu.matmul_f32(dA, aoff, dx, 0, dC, coff, m, k, 1, accumulate=accumulate)
    out = dC.to_numpy(np.float32, coff + m)
    assert np.array_equal(out[:coff], c0[:coff])
    ref = c0.copy()
    if not accumulate:
        ref[coff:] = 0
    oracle.matmul_f32(A, aoff, x, 0, ref, coff, m, k, 1, threads=0)
    base = c0[coff:] if accumulate else 0
    Am = A[aoff:].reshape(m, k)
    check((out[coff:] - base)[:, None], Am, x[:, None], (ref[coff:] - base)[:, None])


@pytest.mark.parametrize("m,k,n", [(64, 64, 64), (100, 37, 53), (4, 3, 2), (2, 2, 2), (512, 768, 96), (1, 300, 200),
                                   # skinny left operand: the k-split streaming kernel (m <= 64, n % 4 == 0, n >= 512, k >= 256)
                                   (8, 2048, 2048), (64, 512, 1024), (5, 300, 512), (17, 1000, 516), (8, 2048, 8192)])
@pytest.mark.parametrize("b_t", [False, True])
def test_gemm_tile(gpu, oracle, m, k, n, b_t):
    rng = np.random.default_rng(m * k + n)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    Bg = np.ascontiguousarray(B.T) if b_t else B
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(Bg)
    dC = gpu.DeviceBuffer(m * n * 4)
    gpu.matmul_f32(dA, 0, dB, 0, dC, 0, m, k, n, accumulate=False, b_transposed=b_t)
    out = dC.to_numpy(np.float32, (m, n))
    check(out, A, B, oracle.tensor_matmul_f32(A, Bg, b_transposed=b_t))


@pytest.mark.parametrize("m,k,n", [(512, 768, 2304), (300, 520, 516), (1024, 1024, 1024), (128, 4096, 128), (2048, 64, 2048),
                                   (256, 16384, 128),
                                   # fewer tiles than CTA pairs: the K chunks of a tile go to different pairs (split K)
                                   (256, 8192, 512), (256, 2048, 256)])
@pytest.mark.parametrize("b_t", [False, True])
@pytest.mark.parametrize("accumulate", [False, True])
def test_gemm_tensor_core(gpu, oracle, m, k, n, b_t, accumulate):
    """GEMM-sized shapes run as 3 x TF32 on the tensor cores (operands split into two TF32 planes each): edge tiles in m
    and n, k that is not a multiple of the 32-float K block, B in both layouts, and C += through the TMA reduce-add.
    The error must stay at f32 level -- a plain TF32 product would be ~1e-3."""
    rng = np.random.default_rng(m + 3 * k + 7 * n)
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    C0 = rng.standard_normal((m, n)).astype(np.float32)
    Bg = np.ascontiguousarray(B.T) if b_t else B
    dA, dB, dC = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(Bg), gpu.DeviceBuffer.from_numpy(C0)
    gpu.matmul_f32(dA, 0, dB, 0, dC, 0, m, k, n, accumulate=accumulate, b_transposed=b_t)
    out = dC.to_numpy(np.float32, (m, n))
    if accumulate:
        out = out - C0
    check(out, A, B, oracle.tensor_matmul_f32(A, Bg, b_transposed=b_t))
    exact = A.astype(np.float64) @ B.astype(np.float64)
    assert np.max(np.abs(out - exact)) / np.max(np.abs(exact)) <= 2e-5


def test_skinny_accumulates_like_simp_matmul(gpu, oracle):
    """simp.matmul semantics (C += A . B) on the k-split kernel."""
    rng = np.random.default_rng(9)
    m, k, n = 8, 1024, 768
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = (0.05 * rng.standard_normal((k, n))).astype(np.float32)
    C0 = rng.standard_normal((m, n)).astype(np.float32)
    dA, dB, dC = (gpu.DeviceBuffer.from_numpy(a) for a in (A, B, C0))
    gpu.matmul_f32(dA, 0, dB, 0, dC, 0, m, k, n, accumulate=True)
    out = dC.to_numpy(np.float32, (m, n))
    check(out - C0, A, B, oracle.tensor_matmul_f32(A, B))


def test_known_answers(gpu):
    # tests/mlir/integration/test_matmul_simple.sl:24-27: [[1,2],[3,4]] x [[5,6],[7,8]] -> C[0,0] = 19
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(B)
    dC = gpu.DeviceBuffer(16)
    dC.zero()
    gpu.matmul_f32(dA, 0, dB, 0, dC, 0, 2, 2, 2, accumulate=True)
    assert dC.to_numpy(np.float32, (2, 2))[0, 0] == 19.0
    # tests/test_tensor_matmul.sl:4-65: A[i,j] = i*3+j+1 (4x3), B[i,j] = i*2+j+1 (3x2) -> C[0,0] = 22
    A = (np.arange(12, dtype=np.float32) + 1).reshape(4, 3)
    B = (np.arange(6, dtype=np.float32) + 1).reshape(3, 2)
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(B)
    dC = gpu.DeviceBuffer(32)
    gpu.matmul_f32(dA, 0, dB, 0, dC, 0, 4, 3, 2, accumulate=False)
    assert dC.to_numpy(np.float32, (4, 2))[0, 0] == 22.0


@pytest.mark.parametrize("batch,m,k,n", [(3, 8, 2048, 512), (5, 33, 70, 41), (1, 64, 64, 64), (12, 16, 64, 16),
                                         (2, 256, 512, 512)])
@pytest.mark.parametrize("b_t", [False, True])
def test_batched_tensor_matmul(gpu, oracle, batch, m, k, n, b_t):
    """3-D tensor_matmul (linalg.batch_matmul, ConvertSimpToMemRef.cpp:3286-3291): every batch entry equals the 2-D op."""
    rng = np.random.default_rng(batch * 1000 + m * k + n)
    A = rng.standard_normal((batch, m, k)).astype(np.float32)
    B = rng.standard_normal((batch, k, n)).astype(np.float32)
    Bg = np.ascontiguousarray(B.transpose(0, 2, 1)) if b_t else B
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(Bg)
    dC = gpu.DeviceBuffer(batch * m * n * 4)
    gpu.check(gpu.lib().simp_gpu_matmul_f32_batched(dA.ptr, dB.ptr, dC.ptr, batch, m, k, n, int(b_t)))
    out = dC.to_numpy(np.float32, (batch, m, n))
    for b in range(batch):
        check(out[b], A[b], B[b], oracle.tensor_matmul_f32(A[b], Bg[b], b_transposed=b_t))
