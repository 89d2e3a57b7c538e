// gemm_i4.cu -- tensor_matmul on packed signed i4 operands, i16 result
// (TensorMatMulOpLowering, packed-i4 branch, src/mlir/lowering/ConvertSimpToMemRef.cpp:2953-3133).
//
// The reference unpacks both operands to i8 (sign-extending each nibble; A along K, B along N, transposing B on
// the way), runs an i8 x i8 -> i32 contraction and truncates to i16.  Here the same three steps run on the
// device: two unpack kernels (one thread per packed byte, outputs padded with zeros to 16-byte row pitches so
// the TMA tiles of the GEMM can address them; B keeps its [K, N] orientation, which the tensor cores read
// through an MN-major descriptor), the tcgen05 int8 GEMM (exact i32), and a narrowing kernel that keeps the
// low 16 bits.  The i32 sums are exact, so the result equals the reference's for every shape.
#include "common.cuh"

namespace simp {

int gemm_i8_run(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N, int a_unsigned,
                int b_transposed, int32_t* const* peer_c, int n_peers, int64_t ldc, int64_t col_offset, int self_rank = 0);

// src: [rows, ceil(cols / 2)] bytes, low nibble = even column.  dst: [rows_p, cols_p] s8, zero outside [rows, cols).
__global__ void unpack_i4_kernel(const uint8_t* __restrict__ src, int8_t* __restrict__ dst, int64_t rows, int64_t cols,
                                 int64_t rows_p, int64_t cols_p) {
  const int64_t pairs_p = cols_p >> 1;
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows_p * pairs_p) return;
  const int64_t r = idx / pairs_p, cp = idx - r * pairs_p;
  int lo = 0, hi = 0;
  if (r < rows && 2 * cp < cols) {
    const uint8_t b = src[r * ((cols + 1) >> 1) + cp];
    lo = b & 15;
    lo = lo >= 8 ? lo - 16 : lo;
    if (2 * cp + 1 < cols) {
      hi = (b >> 4) & 15;
      hi = hi >= 8 ? hi - 16 : hi;
    }
  }
  *reinterpret_cast<char2*>(dst + r * cols_p + 2 * cp) = make_char2(char(lo), char(hi));
}
// C16[i, j] = low 16 bits of C32[i, j] (C32 has row pitch ld)
__global__ void narrow_i32_i16_kernel(const int32_t* __restrict__ c32, int16_t* __restrict__ c16, int64_t M, int64_t N,
                                      int64_t ld) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= M * N) return;
  const int64_t i = idx / N, j = idx - i * N;
  c16[idx] = int16_t(uint16_t(uint32_t(c32[i * ld + j]) & 0xffffu));
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_gpu_matmul_i4(const uint8_t* A_packed, const uint8_t* B_packed, int16_t* C, int64_t M, int64_t K,
                                int64_t N) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(M >= 0 && K >= 0 && N >= 0, SIMP_ERR_ARG, "matmul_i4: negative size");
  if (M == 0 || N == 0) return SIMP_OK;
  SIMP_REQUIRE(A_packed && B_packed && C, SIMP_ERR_ARG, "matmul_i4: null pointer");
  cudaStream_t st = ctx().stream;
  if (K == 0) {
    SIMP_CUDA(cudaMemsetAsync(C, 0, size_t(M) * size_t(N) * 2, st));
    return SIMP_OK;
  }
  const int64_t Kp = (K + 15) & ~int64_t(15), Np = (N + 15) & ~int64_t(15);
  int8_t* a8 = static_cast<int8_t*>(scratch(size_t(M) * Kp, 8));
  int8_t* b8 = static_cast<int8_t*>(scratch(size_t(Kp) * Np, 9));
  int32_t* c32 = static_cast<int32_t*>(scratch(size_t(M) * Np * 4, 10));
  if (!(a8 && b8 && c32)) return scratch_failed("matmul_i4 (unpacked operands)");
  auto blocks = [](int64_t n) { return unsigned((n + 255) / 256); };
  unpack_i4_kernel<<<blocks(M * (Kp / 2)), 256, 0, st>>>(A_packed, a8, M, K, M, Kp);
  unpack_i4_kernel<<<blocks(Kp * (Np / 2)), 256, 0, st>>>(B_packed, b8, K, N, Kp, Np);
  SIMP_LAUNCH_CHECK();
  if (int rc = gemm_i8_run(a8, b8, c32, M, Kp, Np, /*a_unsigned=*/0, /*b_transposed=*/0, nullptr, 0, Np, 0)) return rc;
  narrow_i32_i16_kernel<<<blocks(M * N), 256, 0, st>>>(c32, C, M, N, Np);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
