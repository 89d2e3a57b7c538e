// bench_int8_gemm_host.cpp -- C++ host for the int8 GEMM of libsimp_gpu.so, the GPU counterpart of the
// reference's prefill-matmul host (simptensor/benchmarks/bench_prefill_matmul_runner.cpp:25-120): same seeded
// inputs (std::mt19937, seeds 1 and 2), a scalar [M,K].[N,K]^T verification on the host for small shapes,
// warm-up + timed iterations, GIOP/s = 2*M*N*K / t.
//
//   bench_int8_gemm_host <path/to/libsimp_gpu.so> [M K N] [iterations]
//
// Exit code 0 when the run (and, for shapes up to 2^31 MACs, the verification) succeeded.
#include <cstdio>
#include <cstdlib>
#include <random>

#include "gpu_kernel_runner.hpp"

static void init_random_i8(std::vector<int8_t>& v, int seed) {
  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> dist(-128, 127);
  for (auto& x : v) x = int8_t(dist(rng));
}

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: %s <libsimp_gpu.so> [M K N] [iterations]\n", argv[0]);
    return 2;
  }
  const int64_t M = argc > 4 ? std::atoll(argv[2]) : 512, K = argc > 4 ? std::atoll(argv[3]) : 2048,
                N = argc > 4 ? std::atoll(argv[4]) : 2048;
  const size_t iters = argc > 5 ? std::atoll(argv[5]) : 20;
  try {
    simp_gpu::GpuKernelRunner runner;
    runner.loadLibrary(argv[1]);
    auto matmul = runner.sym<int (*)(const void*, const int8_t*, int32_t*, int64_t, int64_t, int64_t, int, int)>(
        "simp_gpu_matmul_i8");
    std::vector<int8_t> A(M * K), Bt(N * K);
    init_random_i8(A, 1);
    init_random_i8(Bt, 2);
    void* dA = runner.alloc(A.size());
    void* dB = runner.alloc(Bt.size());
    void* dC = runner.alloc(size_t(M) * N * 4);
    runner.upload(dA, A.data(), A.size());
    runner.upload(dB, Bt.data(), Bt.size());
    runner.sync();
    simp_gpu::ProfiledGpuKernelRunner prof(runner, 3, iters, true);
    const double us = prof.runBenchmark("tensor_matmul_nt i8", [&] {
      runner.check(matmul(dA, static_cast<const int8_t*>(dB), static_cast<int32_t*>(dC), M, K, N, 0, 1),
                   "simp_gpu_matmul_i8");
    });
    prof.printStatistics();
    std::printf("M=%lld K=%lld N=%lld: %.2f us, %.1f GIOP/s\n", (long long)M, (long long)K, (long long)N, us,
                2.0 * double(M) * double(N) * double(K) / (us * 1e-6) / 1e9);
    int bad = 0;
    if (double(M) * double(N) * double(K) <= 2147483648.0) {
      std::vector<int32_t> C(size_t(M) * N);
      runner.download(C.data(), dC, C.size() * 4);
      for (int64_t i = 0; i < M && bad < 5; ++i)
        for (int64_t j = 0; j < N; ++j) {
          int32_t ref = 0;
          for (int64_t k = 0; k < K; ++k) ref += int32_t(A[i * K + k]) * int32_t(Bt[j * K + k]);
          if (ref != C[i * N + j] && bad++ < 5)
            std::printf("MISMATCH [%lld,%lld]: expected %d got %d\n", (long long)i, (long long)j, ref, C[i * N + j]);
        }
      std::printf(bad ? "verification FAILED\n" : "verification passed (bit-exact)\n");
    }
    runner.free(dA);
    runner.free(dB);
    runner.free(dC);
    return bad ? 1 : 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "Error: %s\n", e.what());
    return 1;
  }
}
