"""Generates tests/golden/golden.json.

Two kinds of vectors:
  * known answers transcribed from the reference's own tests (file:line given per entry);
  * outputs of the reference's own compiled CPU kernels (oracle/_ref, built from the reference
    checkout by oracle/Makefile) on seeded inputs, stored as checksums plus sampled entries.
Run in the build container (needs the reference checkout and AVX512-VNNI):
    python tests/golden/make_golden.py
"""
import ctypes
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    oracle.build(with_ref=True)
    g = {"known_answers": [], "ref_int8": []}
    ka = g["known_answers"]
    ka.append({"op": "rmsnorm", "src": "examples/llama2/kernels/test_rmsnorm.sl:13-39; test_rmsnorm_host.cpp:39-44",
               "x": [1, 2, 3, 4], "w": [1, 1, 1, 1], "eps": 1e-5, "index": 0, "expect": float(1 / np.sqrt(7.5 + 1e-5)),
               "atol": 1e-4})
    e = np.exp(np.array([1., 2., 3., 4.]) - 4)
    ka.append({"op": "softmax", "src": "examples/llama2/kernels/test_softmax_host.cpp:34-38", "x": [1, 2, 3, 4],
               "index": 0, "expect": float(e[0] / e.sum()), "atol": 1e-4})
    ka.append({"op": "silu", "src": "examples/llama2/kernels/test_silu_host.cpp:31-36", "x": [1.0], "index": 0,
               "expect": float(1 / (1 + np.exp(-1.0))), "atol": 1e-4})
    ka.append({"op": "swiglu", "src": "examples/llama2/kernels/test_swiglu_host.cpp:33-41", "x": [0.5], "mul": [2.0],
               "index": 0, "expect": float(0.5 / (1 + np.exp(-0.5)) * 2.0), "atol": 1e-4})
    ka.append({"op": "matmul_f32", "src": "tests/mlir/integration/test_matmul_simple.sl:24-27; test_matmul_runner.cpp:37-39",
               "A": [[1, 2], [3, 4]], "B": [[5, 6], [7, 8]], "index": [0, 0], "expect": 19.0, "atol": 0})
    ka.append({"op": "tensor_matmul_f64", "src": "tests/test_tensor_matmul.sl:4-65; runner :39-62",
               "A": (np.arange(12) + 1.0).reshape(4, 3).tolist(), "B": (np.arange(6) + 1.0).reshape(3, 2).tolist(),
               "index": [0, 0], "expect": 22.0, "atol": 0})
    # vpdpbusd extremes (simptensor/tests/test_vnni_correctness.cpp:118-160): every lane 4*255*127 and 4*255*-128
    ka.append({"op": "vpdpbusd", "src": "simptensor/tests/test_vnni_correctness.cpp:118-160", "a": 255, "b": 127,
               "expect_lane": 129540})
    ka.append({"op": "vpdpbusd", "src": "simptensor/tests/test_vnni_correctness.cpp:118-160", "a": 255, "b": -128,
               "expect_lane": -130560})

    # reference's scalar checksum on its deterministic fill (bench_int8_matmul_omp_runner.cpp:36-64)
    L = oracle.ref("omprunner")
    L.simp_ref_scalar_checksum_1024.restype = ctypes.c_int32
    g["fill_checksum_1024"] = {"src": "simptensor/benchmarks/bench_int8_matmul_omp_runner.cpp:36-64",
                               "value": int(L.simp_ref_scalar_checksum_1024())}
    # reference VNNI kernels on seeded inputs (seed = size), s8 x s8 with B pre-transposed
    for n in (64, 256, 1024):
        rng = np.random.default_rng(n)
        A = rng.integers(-128, 128, (n, n), dtype=np.int8)
        Bt = rng.integers(-128, 128, (n, n), dtype=np.int8)
        C = oracle.ref_vnni_square(A, Bt, multicore=True)
        g["ref_int8"].append({"kernel": "vnni_matmul_multicore (bench_int8_matmul_multicore.cpp:88-132)", "n": n,
                              "seed": n, "sha256": digest(C), "checksum": oracle.checksum_i32(C),
                              "samples": {f"{i},{j}": int(C[i, j]) for i, j in ((0, 0), (n // 2, n // 3), (n - 1, n - 1))}})
    for (M, N, K) in ((1, 2048, 2048), (5, 192, 128), (512, 640, 3200)):
        rng = np.random.default_rng(M * 1000 + K)
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        Bt = rng.integers(-128, 128, (N, K), dtype=np.int8)
        C = oracle.ref_vnni_mnk(A, Bt, threads=1)
        g["ref_int8"].append({"kernel": "vnni_matmul_i8 (bench_qkv_only_runner.cpp:43-70)", "M": M, "N": N, "K": K,
                              "seed": M * 1000 + K, "sha256": digest(C), "checksum": oracle.checksum_i32(C)})
    # tensor_gather known answers (simptensor/tests/test_scatter_gather.sl:8-147; expected values in
    # simptensor/tests/test_scatter_gather_host.cpp:61-68): source = 1..n in row-major order unless given
    def seq(*shape):
        return (np.arange(int(np.prod(shape))) + 1.0).reshape(shape).tolist()
    g["gather_known_answers"] = [
        {"src": "test_scatter_gather.sl:9-15", "source": [float(v) for v in range(10)], "indices": [0, 3, 7, 2], "axis": 0,
         "sum_at": [[0], [1], [2], [3]], "expect": 12.0},
        {"src": "test_scatter_gather.sl:18-24", "source": [10.0 * (v + 1) for v in range(8)], "indices": [7, 2, 0], "axis": 0,
         "sum_at": [[0], [1], [2]], "expect": 120.0},
        {"src": "test_scatter_gather.sl:27-42", "source": seq(5, 3), "indices": [4, 1, 0], "axis": 0,
         "sum_at": [[0, 0], [1, 1], [2, 2]], "expect": 21.0},
        {"src": "test_scatter_gather.sl:45-58", "source": seq(3, 5), "indices": [4, 1], "axis": 1,
         "sum_at": [[0, 0], [1, 1], [2, 0]], "expect": 27.0},
        {"src": "test_scatter_gather.sl:61-80", "source": seq(4, 2, 3), "indices": [3, 0], "axis": 0,
         "sum_at": [[0, 0, 0], [1, 1, 2]], "expect": 25.0},
        {"src": "test_scatter_gather.sl:83-100", "source": seq(2, 4, 3), "indices": [3, 0], "axis": 1,
         "sum_at": [[0, 0, 0], [1, 1, 2]], "expect": 25.0},
        {"src": "test_scatter_gather.sl:103-118", "source": seq(2, 3, 5), "indices": [4, 1, 0], "axis": 2,
         "sum_at": [[0, 0, 0], [1, 2, 1]], "expect": 32.0},
        {"src": "test_scatter_gather.sl:121-147", "source": seq(2, 2, 3, 4), "indices": [2, 0], "axis": 2,
         "sum_at": [[0, 0, 0, 0], [1, 1, 1, 3]], "expect": 49.0},
    ]
    # reference's own i4 x i4 -> i16 references on the ((i*N+j)%15)-7 fill (bench_int4_matmul_runner.cpp:34-148)
    g["int4_fill_checksums"] = {"src": "simptensor/benchmarks/bench_int4_matmul_runner.cpp:34-148 "
                                       "(scalar_matmul_int4<N>, packed_matmul_int4<N>)", "values": {}}
    for n in (32, 64, 128, 256, 384, 512, 768, 1024):
        sc, pk = oracle.ref_int4_checksums(n)
        assert sc == pk
        g["int4_fill_checksums"]["values"][str(n)] = sc
    with open(os.path.join(HERE, "golden.json"), "w") as f:
        json.dump(g, f, indent=1)
    print("wrote golden.json")


if __name__ == "__main__":
    main()
