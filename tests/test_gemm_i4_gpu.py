"""GPU parity: tensor_matmul on packed signed i4 -> i16, bit-exact against the CPU oracle, against the reference's
own checksums on its deterministic fill, and through i16 wrap-around."""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K,N", [(32, 32, 32), (128, 128, 128), (1, 1, 1), (3, 5, 7), (17, 33, 18), (100, 250, 70),
                                   (256, 384, 512), (64, 4096, 48)])
def test_matmul_i4(gpu, oracle, M, K, N):
    rng = np.random.default_rng(M * 5 + K * 3 + N)
    A = rng.integers(-8, 8, (M, K))
    B = rng.integers(-8, 8, (K, N))
    Ap, Bp = oracle.pack_i4(A), oracle.pack_i4(B)
    out = gpu.np_matmul_i4(Ap, Bp, M, K, N)
    ref = oracle.tensor_matmul_i4(Ap, Bp, M, K, N)
    assert np.array_equal(out, ref)


def test_reference_fill_checksums(gpu, oracle):
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "golden.json")))["int4_fill_checksums"]["values"]
    for n_s, expect in g.items():
        n = int(n_s)
        i, j = np.meshgrid(np.arange(n), np.arange(n), indexing="ij")
        A = ((i * n + j) % 15) - 7
        out = gpu.np_matmul_i4(oracle.pack_i4(A), oracle.pack_i4(A.T.copy()), n, n, n)
        assert int(np.sum(out.astype(np.int64))) == expect, n


def test_i16_wraparound(gpu):
    # K = 2048 products of (-8) * (-8) = 64 sum to 131072 = 2 * 65536: the low 16 bits are 0; 7 * (-8) wraps negative
    K = 2048
    A = np.full((4, K), -8)
    B = np.full((K, 6), -8)
    B[:, 1] = 7
    from oracle import pack_i4
    out = gpu.np_matmul_i4(pack_i4(A), pack_i4(B), 4, K, 6)
    exact = (A.astype(np.int64) @ B.astype(np.int64))
    assert np.array_equal(out, exact.astype(np.int16))
    assert out[0, 0] == 0 and out[0, 1] == np.array([-8 * 7 * K], np.int64).astype(np.int16)[0]
