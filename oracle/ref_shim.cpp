// ref_shim.cpp -- builds the reference's OWN CPU code for the int8 path into
// small shared objects under oracle/_ref/, straight from the reference checkout.
//
// TEST INFRASTRUCTURE ONLY (see simp_oracle.cpp).  No reference source is copied:
// each unit #includes one reference file where it lies (the include path is the
// reference project root, given by the Makefile) with its main() renamed, and
// exports a few C entry points that call the reference's functions unmodified.
// One unit per shared object because the reference files define clashing globals.
//
//   REF_UNIT_MULTICORE : simptensor/benchmarks/bench_int8_matmul_multicore.cpp
//                        -> vnni_matmul_multicore<N>, vnni_matmul_single_thread<N> (:38-132)
//   REF_UNIT_QKV       : simptensor/benchmarks/bench_qkv_only_runner.cpp
//                        -> vnni_matmul_i8(A, B_T, C, M, N, K) (:43-70)
//   REF_UNIT_VNNITEST  : simptensor/tests/test_vnni_correctness.cpp
//                        -> scalar_vpdpbusd_reference / vnni_vpdpbusd (:28-59) and its 9 tests
//   REF_UNIT_OMPRUNNER : simptensor/benchmarks/bench_int8_matmul_omp_runner.cpp
//                        -> scalar_matmul_checksum() (:36-64)
//   REF_UNIT_INT4RUNNER: simptensor/benchmarks/bench_int4_matmul_runner.cpp
//                        -> scalar_matmul_int4<N>() (:34-68), packed_matmul_int4<N>() (:74-148)
#include <cstdint>
#define REF_API extern "C" __attribute__((visibility("default")))

#if defined(REF_UNIT_MULTICORE)
#define main simp_ref_multicore_main
#include "simptensor/benchmarks/bench_int8_matmul_multicore.cpp"
#undef main
// s8 x s8 -> s32, A [N,N], B_T [N,N] (B transposed), N % 64 == 0 (the K loop drops tails).
REF_API int simp_ref_vnni_square(const int8_t* A, const int8_t* B_T, int32_t* C, int N,
                                 int multicore) {
#define REF_CASE(n)                                       \
  case n:                                                 \
    if (multicore) vnni_matmul_multicore<n>(A, B_T, C);   \
    else vnni_matmul_single_thread<n>(A, B_T, C);         \
    return 0;
  switch (N) {
    REF_CASE(64) REF_CASE(128) REF_CASE(256) REF_CASE(512) REF_CASE(1024) REF_CASE(2048)
    REF_CASE(4096) REF_CASE(8192)
    default: return -1;
  }
#undef REF_CASE
}
#endif

#if defined(REF_UNIT_QKV)
#define main simp_ref_qkv_main
#include "simptensor/benchmarks/bench_qkv_only_runner.cpp"
#undef main
#include <algorithm>
// s8 x s8 -> s32, A [M,K], B_T [N,K], K % 64 == 0.  Rows are split into chunks of a
// multiple of 4 (the kernel's row tile) and each chunk is one unmodified call.
REF_API int simp_ref_vnni_mnk(int8_t* A, int8_t* B_T, int32_t* C, int M, int N, int K,
                              int threads) {
  if (K % 64 != 0) return -1;
  if (threads <= 1) {
    vnni_matmul_i8(A, B_T, C, M, N, K);
    return 0;
  }
  const int chunk = std::max(4, ((M + threads - 1) / threads + 3) / 4 * 4);
  const int nchunks = (M + chunk - 1) / chunk;
#pragma omp parallel for num_threads(threads) schedule(static)
  for (int c = 0; c < nchunks; ++c) {
    const int r0 = c * chunk, r1 = std::min(M, r0 + chunk);
    vnni_matmul_i8(A + size_t(r0) * K, B_T, C + size_t(r0) * N, r1 - r0, N, K);
  }
  return 0;
}
#endif

#if defined(REF_UNIT_VNNITEST)
#define main simp_ref_vnnitest_main
#include "simptensor/tests/test_vnni_correctness.cpp"
#undef main
REF_API void simp_ref_vpdpbusd(const uint8_t* a, const int8_t* b, const int32_t* acc,
                               int32_t* result, int use_vnni) {
  if (use_vnni) vnni_vpdpbusd(a, b, acc, result);
  else scalar_vpdpbusd_reference(a, b, acc, result);
}
// Runs the reference's own 9 VNNI-vs-scalar tests; 0 = all passed.
REF_API int simp_ref_vnni_selftest() { return simp_ref_vnnitest_main(); }
#endif

#if defined(REF_UNIT_OMPRUNNER)
#define main simp_ref_omprunner_main
#include "simptensor/benchmarks/bench_int8_matmul_omp_runner.cpp"
#undef main
// Checksum of the scalar s8 x s8 product on the ((i*N+j)%127)-64 fill, N = 1024.
REF_API int32_t simp_ref_scalar_checksum_1024() { return scalar_matmul_checksum(); }
#endif

#if defined(REF_UNIT_INT4RUNNER)
#define main simp_ref_int4runner_main
#include "simptensor/benchmarks/bench_int4_matmul_runner.cpp"
#undef main
// Checksums of the i4 x i4 -> i16 product on the ((i*N+j)%15)-7 fill (B[j,i] = A[i,j]): the scalar reference and
// the packed-storage reference of the runner.  Returns 0 and writes both, or -1 for a size it does not instantiate.
REF_API int simp_ref_int4_checksums(int N, int32_t* scalar, int32_t* packed) {
#define REF_CASE(n) case n: *scalar = scalar_matmul_int4<n>(); *packed = packed_matmul_int4<n>(); return 0;
  switch (N) {
    REF_CASE(32) REF_CASE(64) REF_CASE(128) REF_CASE(256) REF_CASE(384) REF_CASE(512) REF_CASE(768) REF_CASE(1024)
    default: return -1;
  }
#undef REF_CASE
}
#endif
