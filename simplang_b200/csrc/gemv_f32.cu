// gemv_f32.cu -- simp.matmul / tensor_matmul on f32.
//
// n == 1 (every projection of the f32 LLaMA models, examples/llama2/stories110M.sl:77-83,
// 174, 199-244) is a bandwidth-bound streaming GEMV: each warp (or W cooperating warps for
// short matrices) streams one row of A with 128-bit no-allocate loads, all loads of a step
// issued before the first use, multiplies with x from L1 and reduces with shuffles.  Tensor
// cores are not used: at one right-hand side the op is 0.5 flop/byte.
// Other shapes run a 64x64 FFMA tile kernel (plain f32 FMA, never TF32).
// Semantics: MatMulOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:1890-1913, accumulates)
// and TensorMatMulOpLowering f32 (ConvertSimpToMemRef.cpp:2926-2933, 3280-3291, fresh result).
#include "common.cuh"
#include "gemv_f32_core.cuh"

namespace simp {

// Any alignment, n == 1: one warp per row, scalar loads.
__global__ void __launch_bounds__(256) gemv_f32_any_kernel(const float* __restrict__ A, const float* __restrict__ x,
                                                           float* __restrict__ C, int64_t m, int64_t k,
                                                           int accumulate) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * 8 + warp;
  if (row >= m) return;
  const float* a = A + row * k;
  float acc = 0.0f;
  for (int64_t i = lane; i < k; i += 32) acc = fmaf(a[i], x[i], acc);
  acc = warp_sum(acc);
  if (lane == 0) C[row] = accumulate ? C[row] + acc : acc;
}

// General shapes: 64x64 output tile, K step 16, 256 threads x (4x4) micro-tile, FFMA.
// B is [k,n] (b_t == 0) or [n,k] (b_t == 1).  Scalar, bounds-checked loads: any alignment.
// blockIdx.z = batch index of the 3-D form (strides m*k, k*n, m*n; linalg.batch_matmul).
__global__ void __launch_bounds__(256) gemm_f32_tile_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                            float* __restrict__ C, int64_t m, int64_t k, int64_t n,
                                                            int accumulate, int b_t) {
  __shared__ float As[16][64 + 4];
  __shared__ float Bs[16][64 + 4];
  A += int64_t(blockIdx.z) * m * k;
  B += int64_t(blockIdx.z) * k * n;
  C += int64_t(blockIdx.z) * m * n;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = int64_t(blockIdx.y) * 64, n0 = int64_t(blockIdx.x) * 64;
  float acc[4][4] = {};
  for (int64_t p0 = 0; p0 < k; p0 += 16) {
    for (int e = threadIdx.x; e < 64 * 16; e += 256) {
      {  // A tile: element (r, c) with c fastest in memory
        const int r = e >> 4, c = e & 15;
        const int64_t gi = m0 + r, gp = p0 + c;
        As[c][r] = (gi < m && gp < k) ? A[gi * k + gp] : 0.0f;
      }
      if (b_t) {
        const int r = e >> 4, c = e & 15;  // r: n index, c: k index (k fastest in memory)
        const int64_t gj = n0 + r, gp = p0 + c;
        Bs[c][r] = (gj < n && gp < k) ? B[gj * k + gp] : 0.0f;
      } else {
        const int c = e >> 6, r = e & 63;  // r: n index (fastest in memory), c: k index
        const int64_t gj = n0 + r, gp = p0 + c;
        Bs[c][r] = (gj < n && gp < k) ? B[gp * n + gj] : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 16; ++p) {
      float a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = As[p][ty * 4 + u];
        b[u] = Bs[p][tx * 4 + u];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(a[u], b[v], acc[u][v]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int64_t gi = m0 + ty * 4 + u, gj = n0 + tx * 4 + v;
      if (gi < m && gj < n) {
        float* c = C + gi * n + gj;
        *c = accumulate ? *c + acc[u][v] : acc[u][v];
      }
    }
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_gpu_matmul_f32(const float* A, int64_t aoff, const float* B, int64_t boff, float* C,
                                 int64_t coff, int64_t m, int64_t k, int64_t n, int accumulate,
                                 int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(m >= 0 && k >= 0 && n >= 0 && aoff >= 0 && boff >= 0 && coff >= 0, SIMP_ERR_ARG,
               "matmul_f32: negative size or offset");
  if (m == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(A && B && C, SIMP_ERR_ARG, "matmul_f32: null pointer");
  cudaStream_t st = ctx().stream;
  const float* a = A + aoff;
  const float* b = B + boff;
  float* c = C + coff;
  if (k == 0) {
    if (!accumulate) SIMP_CUDA(cudaMemsetAsync(c, 0, size_t(m) * size_t(n) * sizeof(float), st));
    return SIMP_OK;
  }
  if (n == 1) {
    const bool vec = (k % 4 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(b) & 15u) == 0) && k / 4 <= 0x7fffffff;
    if (vec) {
      GemvArgs g{};
      g.seg[0] = GemvSeg{a, c, int(m)};
      g.nseg = 1;
      g.k4 = int(k / 4);
      g.x = b;
      SIMP_REQUIRE(m <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_f32: too many rows");
      if (int rc = accumulate ? gemv_f32_launch<GEMV_ACCUM>(g, st, ctx().sm_count)
                              : gemv_f32_launch<GEMV_STORE>(g, st, ctx().sm_count))
        return rc;
    } else {
      const int64_t grid = cdiv(m, 8);
      SIMP_REQUIRE(grid <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_f32: too many rows");
      gemv_f32_any_kernel<<<int(grid), 256, 0, st>>>(a, b, c, m, k, accumulate);
    }
  } else {
    const int64_t gx = cdiv(n, 64), gy = cdiv(m, 64);
    SIMP_REQUIRE(gx <= 0x7fffffff && gy <= 65535, SIMP_ERR_SHAPE, "matmul_f32: shape too large for the tile kernel");
    gemm_f32_tile_kernel<<<dim3(unsigned(gx), unsigned(gy)), 256, 0, st>>>(a, b, c, m, k, n, accumulate,
                                                                         b_transposed);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

// Batched (3-D) tensor_matmul on f32: C[b] = A[b] . B[b] for b < batch, A [batch, m, k], B [batch, k, n] (or
// [batch, n, k] with b_transposed), C [batch, m, n] fresh -- the linalg.batch_matmul case of TensorMatMulOpLowering
// (src/mlir/lowering/ConvertSimpToMemRef.cpp:3286-3291).  One launch of the tile kernel with the batch in grid.z.
SIMP_API int simp_gpu_matmul_f32_batched(const float* A, const float* B, float* C, int64_t batch, int64_t m, int64_t k,
                                         int64_t n, int b_transposed) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(batch >= 0 && m >= 0 && k >= 0 && n >= 0, SIMP_ERR_ARG, "matmul_f32_batched: negative size");
  if (batch == 0 || m == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(A && B && C, SIMP_ERR_ARG, "matmul_f32_batched: null pointer");
  cudaStream_t st = ctx().stream;
  if (k == 0) {
    SIMP_CUDA(cudaMemsetAsync(C, 0, size_t(batch) * size_t(m) * size_t(n) * sizeof(float), st));
    return SIMP_OK;
  }
  const int64_t gx = cdiv(n, 64), gy = cdiv(m, 64);
  SIMP_REQUIRE(gx <= 0x7fffffff && gy <= 65535 && batch <= 65535, SIMP_ERR_SHAPE,
               "matmul_f32_batched: shape too large for the tile kernel");
  gemm_f32_tile_kernel<<<dim3(unsigned(gx), unsigned(gy), unsigned(batch)), 256, 0, st>>>(A, B, C, m, k, n, 0, b_transposed);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
