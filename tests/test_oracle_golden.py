"""CPU tests: the oracle against the golden vectors (known answers transcribed from the reference's own
tests, and outputs of the reference's own compiled VNNI kernels stored in tests/golden/golden.json),
and -- when oracle/_ref is present and the CPU has AVX512-VNNI -- directly against those kernels."""
import hashlib
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "golden.json")) as f:
    GOLD = json.load(f)


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("ka", GOLD["known_answers"], ids=lambda k: k["op"] + str(k.get("b", "")))
def test_known_answers(oracle, ka):
    op = ka["op"]
    f32 = lambda v: np.array(v, np.float32)
    if op == "rmsnorm":
        got = oracle.rmsnorm(f32(ka["x"]), f32(ka["w"]), ka["eps"])[ka["index"]]
    elif op == "softmax":
        got = oracle.softmax(f32(ka["x"]))[ka["index"]]
    elif op == "silu":
        got = oracle.silu(f32(ka["x"]))[ka["index"]]
    elif op == "swiglu":
        got = oracle.silu(f32(ka["x"]), f32(ka["mul"]))[ka["index"]]
    elif op == "matmul_f32":
        A, B = f32(ka["A"]), f32(ka["B"])
        C = np.zeros(A.shape[0] * B.shape[1], np.float32)
        oracle.matmul_f32(A.ravel(), 0, B.ravel(), 0, C, 0, A.shape[0], A.shape[1], B.shape[1])
        got = C.reshape(A.shape[0], -1)[tuple(ka["index"])]
    elif op == "tensor_matmul_f64":
        got = oracle.tensor_matmul_f64(np.array(ka["A"]), np.array(ka["B"]))[tuple(ka["index"])]
    elif op == "vpdpbusd":
        A = np.full((1, 4), ka["a"], np.uint8)
        B = np.full((4, 1), ka["b"], np.int8)
        assert oracle.tensor_matmul_i8(A, B)[0, 0] == ka["expect_lane"]
        return
    assert abs(float(got) - ka["expect"]) <= ka["atol"] + 1e-12


def test_fill_checksum(oracle):
    n = 1024
    idx = np.arange(n * n, dtype=np.int64).reshape(n, n)
    A = ((idx % 127) - 64).astype(np.int8)
    C = oracle.tensor_matmul_i8(A, np.ascontiguousarray(A.T))
    assert oracle.checksum_i32(C) == GOLD["fill_checksum_1024"]["value"]


@pytest.mark.parametrize("g", GOLD["ref_int8"], ids=lambda g: f"{g.get('n', g.get('M'))}")
def test_oracle_matches_stored_reference_outputs(oracle, g):
    rng = np.random.default_rng(g["seed"])
    if "n" in g:
        M = N = K = g["n"]
    else:
        M, N, K = g["M"], g["N"], g["K"]
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    Bt = rng.integers(-128, 128, (N, K), dtype=np.int8)
    C = oracle.tensor_matmul_i8(A, Bt, b_transposed=True)
    assert digest(C) == g["sha256"]
    assert oracle.checksum_i32(C) == g["checksum"]
    # and the [K,N] form of the op gives the same matrix
    assert np.array_equal(oracle.tensor_matmul_i8(A, np.ascontiguousarray(Bt.T)), C)


def test_oracle_against_compiled_reference_kernels(oracle):
    if oracle.ref("multicore") is None:
        pytest.skip("oracle/_ref not built or no AVX512-VNNI on this CPU")
    rng = np.random.default_rng(9)
    A = rng.integers(-128, 128, (512, 512), dtype=np.int8)
    Bt = rng.integers(-128, 128, (512, 512), dtype=np.int8)
    assert np.array_equal(oracle.ref_vnni_square(A, Bt), oracle.tensor_matmul_i8(A, Bt, b_transposed=True))
    A = rng.integers(-128, 128, (7, 320), dtype=np.int8)
    Bt = rng.integers(-128, 128, (33, 320), dtype=np.int8)
    assert np.array_equal(oracle.ref_vnni_mnk(A, Bt, threads=2), oracle.tensor_matmul_i8(A, Bt, b_transposed=True))
    assert oracle.ref("vnnitest").simp_ref_vnni_selftest() == 0  # the reference's own 9 vpdpbusd tests


def test_unsigned_form_and_wraparound(oracle):
    # u8 x s8 (raw vpdpbusd) and modulo-2^32 accumulation (test_vnni_correctness.cpp:248-277)
    K = 70000
    A = np.full((1, K), 255, np.uint8)
    B = np.full((K, 1), 127, np.int8)
    exact = 255 * 127 * K
    assert oracle.tensor_matmul_i8(A, B)[0, 0] == ((exact + 2**31) % 2**32) - 2**31
    As = np.full((1, 4), -1, np.int8)
    assert oracle.tensor_matmul_i8(As, np.ones((4, 1), np.int8))[0, 0] == -4
    assert oracle.tensor_matmul_i8(As.view(np.uint8), np.ones((4, 1), np.int8))[0, 0] == 4 * 255


def test_matmul_accumulates_and_offsets(oracle):
    rng = np.random.default_rng(0)
    A = rng.standard_normal(5 + 6 * 7).astype(np.float32)
    B = rng.standard_normal(2 + 7 * 3).astype(np.float32)
    C0 = rng.standard_normal(4 + 6 * 3).astype(np.float32)
    C = C0.copy()
    oracle.matmul_f32(A, 5, B, 2, C, 4, 6, 7, 3)
    want = C0[4:].reshape(6, 3) + A[5:].reshape(6, 7).astype(np.float64) @ B[2:].reshape(7, 3)
    assert np.allclose(C[4:].reshape(6, 3), want, rtol=1e-5, atol=1e-5)
    assert np.array_equal(C[:4], C0[:4])


def test_w4_quirks(oracle):
    rng = np.random.default_rng(1)
    rows, cols, gs = 4, 256, 128
    w = rng.standard_normal(2 * rows * cols).astype(np.float32)
    qw, sc, zr = oracle.quantize_w4(w, gs)
    x = rng.standard_normal(cols).astype(np.float32)
    # w = q*scale + zero, low nibble = even index
    deq = oracle.dequant_w4(qw, sc, zr, 0, w.size, gs)
    q0 = qw[0] & 15
    assert deq[0] == np.float32(q0) * sc[0] + zr[0]
    assert np.max(np.abs(deq - w)) <= sc.max() * 0.51
    # the reference ignores `offset` in the scale index: matrix 1 read with matrix 0's scales
    off = rows * cols
    ref_mode = oracle.matmul_quant(qw, sc, zr, x, rows, cols, gs, off, scale_mode=0)
    q = np.zeros(off, np.float32)
    for i in range(off):
        b = qw[(off + i) >> 1]
        q[i] = (b >> 4) if (off + i) & 1 else (b & 15)
    wrong = (q.reshape(rows, cols) * np.repeat(sc[: off // gs], gs).reshape(rows, cols)
             + np.repeat(zr[: off // gs], gs).reshape(rows, cols))
    assert np.allclose(ref_mode, wrong @ x, rtol=1e-4, atol=1e-4)
    # per-matrix mode is the true product
    pm = oracle.matmul_quant(qw, sc, zr, x, rows, cols, gs, off, scale_mode=1)
    assert np.allclose(pm, deq[off:].reshape(rows, cols) @ x, rtol=1e-4, atol=1e-4)


def test_quantize_i8_truncates_toward_zero(oracle):
    x = np.array([0.999 / 127, -0.999 / 127, 1.5 / 127, -1.5 / 127, 2.0, -2.0], np.float32)
    assert oracle.quantize_i8(x).tolist() == [0, 0, 1, -1, 127, -128]
    assert oracle.dequantize_i32(np.array([65536, -32768], np.int32)).tolist() == [1.0, -0.5]


def test_llama_forward_runs_and_is_causal(oracle):
    cfg = dict(dim=64, hidden_dim=128, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=50, seq_len=16)
    rng = np.random.default_rng(0)
    d, h, L, V = cfg["dim"], cfg["hidden_dim"], cfg["n_layers"], cfg["vocab_size"]
    mk = lambda *s: (0.05 * rng.standard_normal(s)).astype(np.float32)
    t = dict(token_embedding=mk(V, d), rms_att_w=np.ones((L, d), np.float32), rms_ffn_w=np.ones((L, d), np.float32),
             rms_final_w=np.ones(d, np.float32), wcls=mk(V, d), wq=mk(L, d, d), wk=mk(L, d, d), wv=mk(L, d, d),
             wo=mk(L, d, d), w1=mk(L, h, d), w2=mk(L, d, h), w3=mk(L, h, d))
    m = oracle.Llama(cfg, t, threads=1)
    l0 = m.forward(3, 0).copy()
    l1 = m.forward(7, 1).copy()
    assert np.all(np.isfinite(l0)) and np.all(np.isfinite(l1)) and not np.array_equal(l0, l1)
    m2 = oracle.Llama(cfg, t, threads=2)
    assert np.allclose(m2.forward(3, 0), l0, rtol=1e-5, atol=1e-6)
    with pytest.raises(ValueError):
        m.forward(0, 16)
