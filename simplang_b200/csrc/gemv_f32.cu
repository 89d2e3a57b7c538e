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
#include <algorithm>

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

// Skinny left operand (m <= 64 rows; the prefill of a few tokens, examples/llama2/llama32_1b_fp32_prefill.sl:47-60:
// f32<8, 2048> x f32<2048, 2048>): the op streams B once and is bound by that stream, not by arithmetic.  B is
// [k, n] row-major, so a thread owns four neighbouring columns (one 16-byte load per row of B, coalesced across the
// block) and up to SK_ROWS rows of A, whose values it reads from shared memory as broadcasts.  The k range is cut
// into `splits` slices over grid.y so that every SM streams a share; slice s writes its partial [m, n] block to
// scratch and gemm_f32_skinny_reduce adds the slices in slice order (fixed order: run-to-run identical results).
constexpr int SK_ROWS = 8;
constexpr int SK_THREADS = 128;
constexpr int SK_KCHUNK = 64;   // rows of B per shared-memory refill of the A panel
__global__ void __launch_bounds__(SK_THREADS) gemm_f32_skinny_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                                     float* __restrict__ part, int m, int k, int n,
                                                                     int k_per_split) {
  __shared__ float As[SK_ROWS][SK_KCHUNK];
  const int j = (int(blockIdx.x) * SK_THREADS + int(threadIdx.x)) * 4;   // first of this thread's four columns
  const int k0 = int(blockIdx.y) * k_per_split, k1 = min(k, k0 + k_per_split);
  const int r0 = int(blockIdx.z) * SK_ROWS, nr = min(SK_ROWS, m - r0);
  float acc[SK_ROWS][4];
#pragma unroll
  for (int r = 0; r < SK_ROWS; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.0f;
  for (int p0 = k0; p0 < k1; p0 += SK_KCHUNK) {
    const int pc = min(SK_KCHUNK, k1 - p0);
    __syncthreads();
    for (int e = threadIdx.x; e < SK_ROWS * SK_KCHUNK; e += SK_THREADS) {
      const int r = e / SK_KCHUNK, c = e - r * SK_KCHUNK;
      As[r][c] = (r < nr && c < pc) ? A[int64_t(r0 + r) * k + p0 + c] : 0.0f;
    }
    __syncthreads();
    if (j < n) {
#pragma unroll 4
      for (int c = 0; c < pc; ++c) {
        const float4 b = ld_stream_f4(B + int64_t(p0 + c) * n + j);
#pragma unroll
        for (int r = 0; r < SK_ROWS; ++r) {
          const float a = As[r][c];
          acc[r][0] = fmaf(a, b.x, acc[r][0]);
          acc[r][1] = fmaf(a, b.y, acc[r][1]);
          acc[r][2] = fmaf(a, b.z, acc[r][2]);
          acc[r][3] = fmaf(a, b.w, acc[r][3]);
        }
      }
    }
  }
  if (j < n) {
    float* dst = part + (int64_t(blockIdx.y) * m + r0) * n + j;
#pragma unroll
    for (int r = 0; r < SK_ROWS; ++r)
      if (r < nr) *reinterpret_cast<float4*>(dst + int64_t(r) * n) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
  }
}
__global__ void __launch_bounds__(256) gemm_f32_skinny_reduce(const float* __restrict__ part, float* __restrict__ C, int64_t mn,
                                                              int splits, int accumulate) {
  const int64_t i = (int64_t(blockIdx.x) * 256 + threadIdx.x) * 4;
  if (i >= mn) return;
  float4 s = *reinterpret_cast<const float4*>(part + i);
  for (int q = 1; q < splits; ++q) {
    const float4 t = *reinterpret_cast<const float4*>(part + int64_t(q) * mn + i);
    s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
  }
  float4* c = reinterpret_cast<float4*>(C + i);
  if (accumulate) {
    const float4 o = *c;
    s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
  }
  *c = s;
}

}  // namespace simp

namespace simp {
int gemm_f32_tc_run(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int accumulate,
                    int b_transposed);
}
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
  } else if (!b_transposed && m <= 64 && n % 4 == 0 && n >= 512 && k >= 256 && k <= 0x7fffffff && n <= 0x7fffffff &&
             ((reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0) {
    // skinny left operand: stream B once, k split over the SMs, partial blocks in library scratch
    const int col_blocks = int(cdiv(n / 4, SK_THREADS)), row_blocks = int(cdiv(m, SK_ROWS));
    int splits = int(cdiv(int64_t(ctx().sm_count) * 2, int64_t(col_blocks) * row_blocks));
    splits = int(std::max<int64_t>(1, std::min<int64_t>(splits, k / 64)));
    const int k_per_split = int(cdiv(cdiv(k, splits), 4) * 4);
    splits = int(cdiv(k, k_per_split));
    float* part = static_cast<float*>(scratch(size_t(splits) * size_t(m) * size_t(n) * 4, 12));
    if (!part) return scratch_failed("matmul_f32 (k-slice partial sums)");
    gemm_f32_skinny_kernel<<<dim3(unsigned(col_blocks), unsigned(splits), unsigned(row_blocks)), SK_THREADS, 0, st>>>(
        a, b, part, int(m), int(k), int(n), k_per_split);
    gemm_f32_skinny_reduce<<<unsigned(cdiv(m * n / 4, 256)), 256, 0, st>>>(part, c, m * n, splits, accumulate);
  } else {
    // GEMM-sized shapes: 3 x TF32 on the tensor cores (gemm_f32_tc.cu); everything else: the FFMA tile kernel
    const int tc = gemm_f32_tc_run(a, b, c, m, k, n, accumulate, b_transposed);
    if (tc < 0) return tc;
    if (tc == 1) {
      const int64_t gx = cdiv(n, 64), gy = cdiv(m, 64);
      SIMP_REQUIRE(gx <= 0x7fffffff && gy <= 65535, SIMP_ERR_SHAPE, "matmul_f32: shape too large for the tile kernel");
      gemm_f32_tile_kernel<<<dim3(unsigned(gx), unsigned(gy)), 256, 0, st>>>(a, b, c, m, k, n, accumulate,
                                                                           b_transposed);
    }
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
  // GEMM-sized matrices: one tensor-core GEMM per batch entry (the split planes live in library scratch, reused in
  // stream order)
  {
    const int first = gemm_f32_tc_run(A, B, C, m, k, n, 0, b_transposed);
    if (first < 0) return first;
    if (first == 0) {
      for (int64_t i = 1; i < batch; ++i) {
        const int rc = gemm_f32_tc_run(A + i * m * k, B + i * k * n, C + i * m * n, m, k, n, 0, b_transposed);
        if (rc != 0) return rc < 0 ? rc : set_error(SIMP_ERR_CUDA, "matmul_f32_batched: scratch lost between batch entries");
      }
      return SIMP_OK;
    }
  }
  const int64_t gx = cdiv(n, 64), gy = cdiv(m, 64);
  SIMP_REQUIRE(gx <= 0x7fffffff && gy <= 65535 && batch <= 65535, SIMP_ERR_SHAPE,
               "matmul_f32_batched: shape too large for the tile kernel");
  gemm_f32_tile_kernel<<<dim3(unsigned(gx), unsigned(gy), unsigned(batch)), 256, 0, st>>>(A, B, C, m, k, n, 0, b_transposed);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
