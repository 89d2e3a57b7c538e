// gemv_w4.cu -- matmul_quant entry point: out[rows] = W4[rows,cols] . x[cols]   (batch-1 decode GEMV)
//
// Semantics: MatMulQuantOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:3906-4005).
// The streaming kernel and the packed-activation format live in w4_core.cuh (every block packs x in its
// own shared memory: no scratch in global memory); this file holds the two entry points and the general
// kernel that follows the lowering's index arithmetic literally for every (gs, cols, offset,
// scale_mode) the streaming kernel does not take.
#include "common.cuh"
#include "w4_core.cuh"

namespace simp {

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

namespace {
// Body shared by both entry points (`who` names the caller in error texts).  Neither path allocates: the
// streaming kernel stages everything in shared memory and the general kernel reads the operands in place.
int matmul_w4_run(const char* who, const uint8_t* qw, const float* sc, const float* zr, const float* x, float* out,
                  int64_t rows, int64_t cols, int64_t gs, int64_t offset, int scale_mode) {
  SIMP_REQUIRE(rows >= 0 && cols >= 0 && offset >= 0, SIMP_ERR_ARG, "%s: negative size or offset", who);
  SIMP_REQUIRE(gs > 0, SIMP_ERR_ARG, "%s: group_size must be positive", who);
  SIMP_REQUIRE(scale_mode == 0 || scale_mode == 1, SIMP_ERR_ARG, "%s: scale_mode must be 0 or 1", who);
  if (rows == 0) return SIMP_OK;
  SIMP_REQUIRE(qw && sc && x && out, SIMP_ERR_ARG, "%s: null pointer", who);
  SIMP_REQUIRE(scale_mode == 0 || cols % gs == 0, SIMP_ERR_SHAPE,
               "%s: scale_mode 1 needs cols %% group_size == 0 (cols %lld, gs %lld)", who, (long long)cols, (long long)gs);
  cudaStream_t st = ctx().stream;
  int log2_cpg = -1;
  for (int s = 0; s <= 5; ++s)
    if (gs == (int64_t(32) << s)) log2_cpg = s;
  const bool mode_ok = scale_mode == 1 ? (offset % gs == 0) : (gs == 128);
  const uint8_t* base = qw + offset / 2;
  const int64_t soff = scale_mode == 1 ? offset / gs : 0;
  const bool sc_aligned = ((reinterpret_cast<uintptr_t>(sc + soff) & 15u) == 0) &&
                          (!zr || (reinterpret_cast<uintptr_t>(zr + soff) & 15u) == 0);
  bool fast = sc_aligned && log2_cpg >= 0 && mode_ok && cols > 0 && cols % gs == 0 && cols <= 16384 && offset % 32 == 0 &&
              ((reinterpret_cast<uintptr_t>(base) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
              rows <= 0x7fffffff;
  // the packed input plus two stages of the smallest (8-row) tile must fit in shared memory; very long rows with
  // small groups and zeros (16384 columns, groups of 32) do not, and take the general kernel
  if (fast && w4_packed_bytes(cols) + 2 * w4_stage_bytes(int(cols), int(cols / gs), 1, zr != nullptr, 8) > W4_SMEM_LIMIT)
    fast = false;
  if (fast) {
    W4Args a{};
    a.seg[0] = W4Seg{base, sc + soff, zr ? zr + soff : nullptr, out, int(rows)};
    a.nseg = 1;
    a.cols = int(cols);
    a.log2_cpg = log2_cpg;
    a.groups_per_row = int(cols / gs);
    a.x = x;
    a.res = nullptr;
    return w4_launch<W4_STORE>(a, st, ctx().sm_count);
  }
  if (cols == 0) {
    SIMP_CUDA(cudaMemsetAsync(out, 0, size_t(rows) * sizeof(float), st));
    return SIMP_OK;
  }
  const int64_t grid = cdiv(rows, 8);
  SIMP_REQUIRE(grid <= 0x7fffffff, SIMP_ERR_SHAPE, "%s: too many rows", who);
  w4_gemv_general_kernel<<<int(grid), 256, 0, st>>>(qw, sc, zr, x, out, rows, cols, gs, offset, scale_mode);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
}  // namespace

SIMP_API int simp_gpu_matmul_w4(const uint8_t* qw, const float* sc, const float* zr, const float* x, float* out,
                                int64_t rows, int64_t cols, int64_t gs, int64_t offset, int scale_mode) {
  if (int rc = ensure_ready()) return rc;
  return matmul_w4_run("matmul_w4", qw, sc, zr, x, out, rows, cols, gs, offset, scale_mode);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of simp_gpu_matmul_w4.
//
// Some hosts may not allocate device memory when they call into this library: a serving process
// that hands its whole memory budget to its own pool at start-up (a later cudaMalloc then fails or
// fragments the pool), or code running where the CUDA runtime forbids allocation altogether.
// The W4 kernels need no scratch in global memory (the streaming kernel packs the input vector in every
// block's shared memory, the general kernel reads the operands in place), so what distinguishes this entry
// point is what it refuses to do: it never initialises the library on demand (initialisation allocates the
// stream and the status words) and it takes at most W4_NOALLOC_MAX_COLS columns, the documented limit of
// the interface.
constexpr int64_t W4_NOALLOC_MAX_COLS = 16384;

SIMP_API int simp_gpu_matmul_w4_noalloc(const uint8_t* qw, const float* sc, const float* zr, const float* x,
                                        float* out, int64_t rows, int64_t cols, int64_t gs, int64_t offset,
                                        int scale_mode) {
  SIMP_REQUIRE(ctx().ready, SIMP_ERR_STATE,
               "matmul_w4_noalloc: call simp_gpu_init first (initialisation allocates; this entry point must not)");
  SIMP_REQUIRE(cols <= W4_NOALLOC_MAX_COLS, SIMP_ERR_SHAPE,
               "matmul_w4_noalloc: cols %lld exceeds the limit of this entry point (%lld); use simp_gpu_matmul_w4",
               (long long)cols, (long long)W4_NOALLOC_MAX_COLS);
  return matmul_w4_run("matmul_w4_noalloc", qw, sc, zr, x, out, rows, cols, gs, offset, scale_mode);
}
