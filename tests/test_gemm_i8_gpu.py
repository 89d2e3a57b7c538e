"""GPU parity: tensor_matmul on i8 -> i32, bit-exact against the CPU oracle.

Covers both signedness modes (s8 x s8 = the op; u8 x s8 = raw vpdpbusd), both B layouts, tile-aligned
and ragged shapes (TMA edge tiles, the dp4a kernel for rows that are not 16-byte multiples), extremes
and i32 wrap-around, the reference's deterministic fill, and linearity at a size too large for the
CPU oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rand(rng, shape, unsigned):
    if unsigned:
        return rng.integers(0, 256, shape, dtype=np.int64).astype(np.uint8)
    return rng.integers(-128, 128, shape, dtype=np.int64).astype(np.int8)


SHAPES = [(128, 128, 256), (128, 256, 256), (256, 512, 512), (1024, 1024, 1024), (512, 3200, 9600),
          (100, 64, 48), (130, 144, 272), (1, 128, 256), (4, 4, 4), (1, 1, 1), (65, 63, 67), (300, 1000, 500),
          (129, 2048, 257), (384, 8640, 3200)]


@pytest.mark.parametrize("M,K,N", SHAPES)
@pytest.mark.parametrize("a_unsigned", [False, True])
@pytest.mark.parametrize("b_t", [False, True])
def test_matmul_i8(gpu, oracle, M, K, N, a_unsigned, b_t):
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    A = rand(rng, (M, K), a_unsigned)
    B = rand(rng, (N, K) if b_t else (K, N), False)
    out = gpu.np_matmul_i8(A, B, b_transposed=b_t)
    ref = oracle.tensor_matmul_i8(A, B, b_transposed=b_t)
    bad = np.argwhere(out != ref)
    assert bad.size == 0, f"{len(bad)} mismatches, first at {bad[:5].tolist()}"


@pytest.mark.parametrize("M,K,N,b_t", [(650, 384, 7952, False), (650, 384, 7952, True), (1280, 256, 4864, False)])
def test_hybrid_stream_k_ragged(gpu, oracle, monkeypatch, M, K, N, b_t):
    """More tiles than SMs with a partial last wave and ragged edges, split forced on: the full waves are stored
    as whole tiles, the tiles of the last wave are zeroed and reduce-added from K ranges."""
    monkeypatch.setenv("SIMP_GEMM_I8_STREAMK", "1")
    monkeypatch.setenv("SIMP_GEMM_I8_KERNEL", "1cta")
    rng = np.random.default_rng(M + N)
    A = rand(rng, (M, K), True)
    B = rand(rng, (N, K) if b_t else (K, N), False)
    out = gpu.np_matmul_i8(A, B, b_transposed=b_t)
    ref = oracle.tensor_matmul_i8(A, B, b_transposed=b_t)
    bad = np.argwhere(out != ref)
    assert bad.size == 0, f"{len(bad)} mismatches, first at {bad[:5].tolist()}"


def test_extremes_and_wraparound(gpu, oracle):
    # 255*127 and 255*-128 products (test_vnni_correctness.cpp:118-160) and i32 wrap (:248-277):
    # K = 131072 of 255 * -128 overflows int32 and must wrap, not saturate.
    M, K, N = 128, 131072, 256
    A = np.full((M, K), 255, np.uint8)
    B = np.full((N, K), -128, np.int8)
    B[1::2] = 127
    out = gpu.np_matmul_i8(A, B, b_transposed=True)
    e0 = np.int64(255) * -128 * K
    e1 = np.int64(255) * 127 * K
    wrap = lambda v: np.int64((int(v) + 2**31) % 2**32 - 2**31)
    assert np.all(out[:, 0::2] == wrap(e0)) and np.all(out[:, 1::2] == wrap(e1))


def test_reference_fill_checksum(gpu, oracle):
    # bench_int8_matmul_omp_runner.cpp:36-64: A[i,j] = ((i*N+j)%127)-64, B[j,i] = A[i,j]; checksum of C.
    N = 1024
    idx = np.arange(N * N, dtype=np.int64).reshape(N, N)
    A = ((idx % 127) - 64).astype(np.int8)
    B = np.ascontiguousarray(A.T)
    out = gpu.np_matmul_i8(A, B)
    assert oracle.checksum_i32(out) == 1100912128  # value produced by the reference's scalar loop
    assert np.array_equal(out, oracle.tensor_matmul_i8(A, B))


def test_linearity_large(gpu):
    # 4096^3 is beyond what the scalar oracle finishes quickly: check (A1 + A2).B == A1.B + A2.B (mod 2^32)
    # with A1 + A2 kept inside int8, and a sampled exact check of rows.
    n = 4096
    rng = np.random.default_rng(11)
    A1 = rng.integers(-60, 60, (n, n), dtype=np.int64).astype(np.int8)
    A2 = rng.integers(-60, 60, (n, n), dtype=np.int64).astype(np.int8)
    B = rng.integers(-128, 128, (n, n), dtype=np.int64).astype(np.int8)
    c1 = gpu.np_matmul_i8(A1, B)
    c2 = gpu.np_matmul_i8(A2, B)
    c12 = gpu.np_matmul_i8((A1 + A2).astype(np.int8), B)
    assert np.array_equal((c1.astype(np.int64) + c2).astype(np.int32), c12)
    rows = [0, 1, 127, 128, 2049, 4095]
    exact = A1[rows].astype(np.int64) @ B.astype(np.int64)
    assert np.array_equal(c1[rows], exact.astype(np.int32))


def test_16384_cube_sampled_rows_exact(gpu):
    """The largest cube of the sweep (16384^3, u8 x s8, B as [K, N]): too large for the CPU oracle as a whole, so rows
    and columns are sampled -- every 2048-column slice gets 4 of the rows checked bit for bit against an exact product
    (partial sums stay below 2^53, so a float64 BLAS product of the sample is exact)."""
    S = 16384
    rng = np.random.default_rng(16384)
    A = rng.integers(0, 256, (S, S), dtype=np.uint8)
    B = rng.integers(-128, 128, (S, S), dtype=np.int8)
    dA, dB = gpu.DeviceBuffer.from_numpy(A), gpu.DeviceBuffer.from_numpy(B)
    dC = gpu.DeviceBuffer(S * S * 4)
    gpu.matmul_i8(dA, dB, dC, S, S, S, a_unsigned=True, b_transposed=False)
    gpu.sync()
    for s in range(S // 2048):
        rows = sorted(int(r) for r in rng.choice(S, 4, replace=False)) + [0, S - 1][s % 2:s % 2 + 1]
        cols = slice(s * 2048, (s + 1) * 2048)
        exact = (A[rows].astype(np.float64) @ B[:, cols].astype(np.float64)).astype(np.int64).astype(np.int32)
        got = np.empty((len(rows), 2048), np.int32)
        for i, r in enumerate(rows):
            gpu.check(gpu.lib().simp_gpu_download(got[i].ctypes.data, dC.ptr + 4 * (r * S + s * 2048), 4 * 2048))
        bad = np.argwhere(got != exact)
        assert bad.size == 0, f"slice {s}: {len(bad)} mismatches, first at {bad[:3].tolist()}"
