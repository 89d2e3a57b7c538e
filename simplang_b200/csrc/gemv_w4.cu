// gemv_w4.cu -- matmul_quant: out[rows] = W4[rows,cols] . x[cols]   (batch-1 decode GEMV)
//
// Semantics: MatMulQuantOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:3906-4005):
// two 4-bit weights per byte, low nibble = even flat index, w = q*scale + zero with one
// (scale, zero) pair per group of `gs` consecutive row-major weights.
//
// Streaming kernel (bandwidth-bound, no tensor cores -- one right-hand side is 4 flop/byte):
//   * x is staged once per block in shared memory, 32-float chunks padded to 36 floats so the
//     128-bit reads of 8 neighbouring lanes fall in distinct banks;
//   * each lane streams 16 bytes (32 weights, one chunk) per load with ld.global.nc
//     L1::no_allocate, 4 chunk-steps x R rows of loads issued before the first use;
//   * a nibble becomes a float without an int->float conversion: the byte (q | 0x80) is placed
//     by one PRMT into bits 16..23 of 0x3F00'0000, giving 1 + q/128 exactly; one FFMA per
//     weight accumulates sum((1+q/128)*x), and the chunk sum S = sum(x) (computed once per
//     chunk, shared by the R rows) is removed afterwards:
//         sum(q*x) = 128*(dot - S);   out += scale*sum(q*x) + zero*S;
//   * rows are reduced with warp shuffles in a fixed order (deterministic results).
// The general kernel follows the lowering's index arithmetic literally, for every
// (gs, cols, offset, scale_mode) the fast path does not take.
#include "common.cuh"

namespace simp {

__device__ __forceinline__ uint4 ldg_nc_u4(const uint4* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}

// dot of one 32-bit word (8 nibbles) with 8 floats, weights encoded as 1 + q/128.
__device__ __forceinline__ float dot8_w4(uint32_t v, const float* __restrict__ xr, float d) {
  const uint32_t lo = (v & 0x0F0F0F0Fu) | 0x80808080u;         // weights 0,2,4,6 in bytes 0..3
  const uint32_t hi = ((v >> 4) & 0x0F0F0F0Fu) | 0x80808080u;  // weights 1,3,5,7
  d = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7044)), xr[0], d);
  d = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7044)), xr[1], d);
  d = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7144)), xr[2], d);
  d = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7144)), xr[3], d);
  d = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7244)), xr[4], d);
  d = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7244)), xr[5], d);
  d = fmaf(__uint_as_float(__byte_perm(lo, 0x3F000000u, 0x7344)), xr[6], d);
  d = fmaf(__uint_as_float(__byte_perm(hi, 0x3F000000u, 0x7344)), xr[7], d);
  return d;
}

constexpr int W4_WARPS = 8;
constexpr int W4_XPAD = 36;  // floats per staged 32-float chunk

// qw points at the first byte of the matrix (offset already applied, 16-byte aligned);
// sc/zr point at the first group of the matrix.  cols % 32 == 0, gs = 32 << log2_cpg.
template <int R>
__global__ void __launch_bounds__(W4_WARPS * 32)
    w4_gemv_kernel(const uint8_t* __restrict__ qw, const float* __restrict__ sc, const float* __restrict__ zr,
                   const float* __restrict__ x, float* __restrict__ out, int rows, int cols, int log2_cpg,
                   int groups_per_row, int passes) {
  extern __shared__ __align__(16) float xs[];
  const int nchunks = cols >> 5;
  for (int i = threadIdx.x; i < (cols >> 2); i += blockDim.x) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(x) + i);
    *reinterpret_cast<float4*>(xs + (i >> 3) * W4_XPAD + (i & 7) * 4) = v;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_it = (nchunks + 31) >> 5;
  const int64_t row_u4 = cols >> 5;  // uint4 per row
  for (int pass = 0; pass < passes; ++pass) {
    const int row0 = (blockIdx.x * passes + pass) * (W4_WARPS * R) + warp * R;
    if (row0 >= rows) break;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int it0 = 0; it0 < n_it; it0 += 4) {
      uint4 wv[4][R];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + ((it0 + u) << 5);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          if (c < nchunks && row0 + r < rows)
            wv[u][r] = ldg_nc_u4(reinterpret_cast<const uint4*>(qw) + int64_t(row0 + r) * row_u4 + c);
          else
            wv[u][r] = make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + ((it0 + u) << 5);
        if (c < nchunks) {
          float xr[32];
          const float4* xp = reinterpret_cast<const float4*>(xs + c * W4_XPAD);
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float4 v = xp[t];
            xr[4 * t + 0] = v.x; xr[4 * t + 1] = v.y; xr[4 * t + 2] = v.z; xr[4 * t + 3] = v.w;
          }
          float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            s0 += xr[t]; s1 += xr[8 + t]; s2 += xr[16 + t]; s3 += xr[24 + t];
          }
          const float S = (s0 + s1) + (s2 + s3);
          const int g = c >> log2_cpg;
#pragma unroll
          for (int r = 0; r < R; ++r) {
            if (row0 + r < rows) {
              const float d0 = dot8_w4(wv[u][r].x, xr + 0, 0.f);
              const float d1 = dot8_w4(wv[u][r].y, xr + 8, 0.f);
              const float d2 = dot8_w4(wv[u][r].z, xr + 16, 0.f);
              const float d3 = dot8_w4(wv[u][r].w, xr + 24, 0.f);
              // per-word (dot - s) keeps the cancellation local to 8 terms
              const float qx = ((d0 - s0) + (d1 - s1)) + ((d2 - s2) + (d3 - s3));
              const int64_t sidx = int64_t(row0 + r) * groups_per_row + g;
              const float s = __ldg(sc + sidx);
              const float z = zr ? __ldg(zr + sidx) : -8.0f * s;
              acc[r] = fmaf(s, 128.0f * qx, fmaf(z, S, acc[r]));
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && row0 + r < rows) out[row0 + r] = v;
    }
  }
}

// The lowering, literally: any gs / cols / offset; scale_mode 0 visits 128 weights per group
// and ignores `offset` in the scale index, scale_mode 1 visits gs weights and adds it.
__global__ void __launch_bounds__(256)
    w4_gemv_general_kernel(const uint8_t* __restrict__ qw, const float* __restrict__ sc, const float* __restrict__ zr,
                           const float* __restrict__ x, float* __restrict__ out, int64_t rows, int64_t cols,
                           int64_t gs, int64_t offset, int scale_mode) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = int64_t(blockIdx.x) * 8 + warp;
  if (row >= rows) return;
  const int64_t row_off = row * cols;
  const int64_t ngroups = cols / gs;
  const int64_t span = scale_mode == 0 ? 128 : gs;
  const int64_t sbase = (scale_mode == 0 ? row_off : offset + row_off) / gs;
  float acc = 0.0f;
  for (int64_t g = 0; g < ngroups; ++g) {
    const float s = sc[sbase + g];
    const float z = zr ? zr[sbase + g] : __fmul_rn(-8.0f, s);
    for (int64_t e = lane; e < span; e += 32) {
      const int64_t kk = g * gs + e;
      if (kk < cols) {
        const int64_t idx = offset + row_off + kk;
        const uint32_t b = qw[idx >> 1];
        const uint32_t q = (idx & 1) ? (b >> 4) : (b & 15u);
        const float w = __fadd_rn(__fmul_rn(float(q), s), z);
        acc = fmaf(w, x[kk], acc);
      }
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[row] = acc;
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_gpu_matmul_w4(const uint8_t* qw, const float* sc, const float* zr, const float* x, float* out,
                                int64_t rows, int64_t cols, int64_t gs, int64_t offset, int scale_mode) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(rows >= 0 && cols >= 0 && offset >= 0, SIMP_ERR_ARG, "matmul_w4: negative size or offset");
  SIMP_REQUIRE(gs > 0, SIMP_ERR_ARG, "matmul_w4: group_size must be positive");
  SIMP_REQUIRE(scale_mode == 0 || scale_mode == 1, SIMP_ERR_ARG, "matmul_w4: scale_mode must be 0 or 1");
  if (rows == 0) return SIMP_OK;
  SIMP_REQUIRE(qw && sc && x && out, SIMP_ERR_ARG, "matmul_w4: null pointer");
  SIMP_REQUIRE(scale_mode == 0 || cols % gs == 0, SIMP_ERR_SHAPE,
               "matmul_w4: scale_mode 1 needs cols %% group_size == 0 (cols %lld, gs %lld)", (long long)cols,
               (long long)gs);
  cudaStream_t st = ctx().stream;
  // Fast path: chunked streaming kernel.
  int log2_cpg = -1;
  for (int s = 0; s <= 5; ++s)
    if (gs == (int64_t(32) << s)) log2_cpg = s;
  const bool mode_ok = scale_mode == 1 ? (offset % gs == 0) : (gs == 128);
  const uint8_t* base = qw + offset / 2;
  const bool fast = log2_cpg >= 0 && mode_ok && cols > 0 && cols % gs == 0 && cols <= 16384 && offset % 32 == 0 &&
                    ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) &&
                    ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) && rows <= 0x7fffffff;
  if (fast) {
    const int64_t soff = scale_mode == 1 ? offset / gs : 0;
    const float* scp = sc + soff;
    const float* zrp = zr ? zr + soff : nullptr;
    const int gpr = int(cols / gs);
    const size_t smem = size_t(cols / 32) * W4_XPAD * sizeof(float);
    constexpr int R = 2;
    const int rows_per_pass = W4_WARPS * R;
    // several passes per block amortise the staging of x once the grid covers the GPU twice over
    int passes = 1;
    while (passes < 8 && cdiv(rows, int64_t(rows_per_pass) * passes * 2) >= int64_t(ctx().sm_count) * 2) passes *= 2;
    const int64_t grid = cdiv(rows, int64_t(rows_per_pass) * passes);
    static bool attr_set = false;
    if (!attr_set) {
      SIMP_CUDA(cudaFuncSetAttribute(w4_gemv_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
      attr_set = true;
    }
    w4_gemv_kernel<R><<<int(grid), W4_WARPS * 32, smem, st>>>(base, scp, zrp, x, out, int(rows), int(cols),
                                                             log2_cpg, gpr, passes);
  } else {
    if (cols == 0) {
      SIMP_CUDA(cudaMemsetAsync(out, 0, size_t(rows) * sizeof(float), st));
      return SIMP_OK;
    }
    const int64_t grid = cdiv(rows, 8);
    SIMP_REQUIRE(grid <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_w4: too many rows");
    w4_gemv_general_kernel<<<int(grid), 256, 0, st>>>(qw, sc, zr, x, out, rows, cols, gs, offset, scale_mode);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
