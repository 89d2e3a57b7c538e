// gemv_f32_core.cuh -- streaming f32 GEMV shared by simp_gpu_matmul_f32 (n == 1) and the decode driver.
//
// out[rows] (+)= A[rows,k] . x[k] for up to three matrices that share x (the q/k/v projections of one
// layer), or the fused SwiGLU pair out = silu(W1.x) * (W3.x) (examples/llama2/stories110M.sl:199-212).
// Each warp (or W cooperating warps for short matrices) streams one row with 128-bit no-allocate
// loads, all 8 loads of a step issued before the first use; x comes from L1.  No tensor cores: one
// right-hand side is 0.5 flop/byte, the kernel is HBM-bound.  The reduction tree is fixed for a
// given (k, W), so results are run-to-run identical.
#pragma once
#include "common.cuh"

namespace simp {

constexpr int GEMV_WARPS = 8;  // warps per block

struct GemvSeg {
  const float* A;  // first element of the matrix, rows 16-byte aligned
  float* out;
  int rows;
};
enum GemvMode { GEMV_STORE = 0, GEMV_ACCUM = 1 /* out += dot */, GEMV_GATE_UP = 2 };
struct GemvArgs {
  GemvSeg seg[3];
  int nseg;
  int k4;              // k / 4
  const float* x;
  int blocks_start[4]; // first block of each segment
};

__device__ __forceinline__ float gemv_row_partial(const float4* __restrict__ a, const float4* __restrict__ xv, int c0,
                                                  int c1, int lane) {
  float acc = 0.0f;
  int i = c0 + lane;
  for (; i + 7 * 32 < c1; i += 8 * 32) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ld_stream_f4(a + i + u * 32);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float4 b = __ldg(xv + i + u * 32);
      acc = fmaf(v[u].x, b.x, acc); acc = fmaf(v[u].y, b.y, acc);
      acc = fmaf(v[u].z, b.z, acc); acc = fmaf(v[u].w, b.w, acc);
    }
  }
  float4 v[8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
    if (i + u * 32 < c1) v[u] = ld_stream_f4(a + i + u * 32);
#pragma unroll
  for (int u = 0; u < 8; ++u)
    if (i + u * 32 < c1) {
      const float4 b = __ldg(xv + i + u * 32);
      acc = fmaf(v[u].x, b.x, acc); acc = fmaf(v[u].y, b.y, acc);
      acc = fmaf(v[u].z, b.z, acc); acc = fmaf(v[u].w, b.w, acc);
    }
  return acc;
}

// W warps share a row (W in {1,2,4,8}); partials are combined in warp order through shared memory.
template <int W, int MODE>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_f32_kernel(const GemvArgs a) {
  __shared__ float part[2][GEMV_WARPS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ROWS = GEMV_WARPS / W;
  int s = 0;
  if (MODE != GEMV_GATE_UP)
    while (s + 1 < a.nseg && int(blockIdx.x) >= a.blocks_start[s + 1]) ++s;
  const int rows = a.seg[s].rows;
  const int row = (int(blockIdx.x) - a.blocks_start[s]) * ROWS + warp / W;
  const int kp = warp % W;
  const int chunk = (a.k4 + W - 1) / W;
  const int c0 = kp * chunk;
  const int c1 = min(a.k4, c0 + chunk);
  const float4* xv = reinterpret_cast<const float4*>(a.x);
  float acc0 = 0.0f, acc1 = 0.0f;
  if (row < rows) {
    acc0 = gemv_row_partial(reinterpret_cast<const float4*>(a.seg[s].A) + int64_t(row) * a.k4, xv, c0, c1, lane);
    if (MODE == GEMV_GATE_UP)
      acc1 = gemv_row_partial(reinterpret_cast<const float4*>(a.seg[1].A) + int64_t(row) * a.k4, xv, c0, c1, lane);
  }
  acc0 = warp_sum(acc0);
  if (MODE == GEMV_GATE_UP) acc1 = warp_sum(acc1);
  if (W > 1) {
    if (lane == 0) {
      part[0][warp] = acc0;
      part[1][warp] = acc1;
    }
    __syncthreads();
    if (kp == 0 && lane == 0) {
      acc0 = part[0][warp];
      acc1 = part[1][warp];
#pragma unroll
      for (int u = 1; u < W; ++u) {
        acc0 += part[0][warp + u];
        acc1 += part[1][warp + u];
      }
    }
  }
  if (lane == 0 && kp == 0 && row < rows) {
    float* o = a.seg[s].out + row;
    if (MODE == GEMV_STORE) *o = acc0;
    if (MODE == GEMV_ACCUM) *o = *o + acc0;
    if (MODE == GEMV_GATE_UP) *o = (acc0 / (1.0f + expf(-acc0))) * acc1;
  }
}

// Picks W so that short matrices still put ~16 warps on every SM, fills the block bookkeeping, launches.
template <int MODE>
inline int gemv_f32_launch(GemvArgs a, cudaStream_t st, int sm_count) {
  int64_t total_rows = 0;
  const int nseg = MODE == GEMV_GATE_UP ? 1 : a.nseg;
  for (int s = 0; s < nseg; ++s) total_rows += a.seg[s].rows;
  if (total_rows == 0) return SIMP_OK;
  const int64_t want = int64_t(sm_count) * 16;
  int W = 1;
  while (W < 8 && total_rows * W * (MODE == GEMV_GATE_UP ? 2 : 1) < want && a.k4 / (W * 2) >= 64) W *= 2;
  const int rows_per_block = GEMV_WARPS / W;
  int blocks = 0;
  for (int s = 0; s < nseg; ++s) {
    a.blocks_start[s] = blocks;
    blocks += (a.seg[s].rows + rows_per_block - 1) / rows_per_block;
  }
  a.blocks_start[nseg] = blocks;
  switch (W) {
    case 1: gemv_f32_kernel<1, MODE><<<blocks, GEMV_WARPS * 32, 0, st>>>(a); break;
    case 2: gemv_f32_kernel<2, MODE><<<blocks, GEMV_WARPS * 32, 0, st>>>(a); break;
    case 4: gemv_f32_kernel<4, MODE><<<blocks, GEMV_WARPS * 32, 0, st>>>(a); break;
    default: gemv_f32_kernel<8, MODE><<<blocks, GEMV_WARPS * 32, 0, st>>>(a); break;
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

// ---- decode variant ---------------------------------------------------------------------------
// Same streaming GEMV, arranged for a chain of small dependent launches: the first batch of weight
// loads is issued before waiting for the producer of x (programmatic dependent launch), x is staged
// in shared memory, and the preceding rmsnorm can be folded into that staging
// (x := (x / sqrt(mean(x^2) + eps)) * norm_w, the arithmetic of RMSNormOpLowering).
struct GemvDecArgs {
  GemvSeg seg[3];
  int nseg;
  int k4;
  const float* x;
  const float* norm_w;  // nullptr: no rmsnorm prologue
  float eps;
  int blocks_start[4];
};

template <int W, int MODE>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_f32_dec_kernel(const GemvDecArgs a) {
  extern __shared__ __align__(16) float xs_f32[];
  __shared__ float part[2][GEMV_WARPS];
  __shared__ float red[33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int ROWS = GEMV_WARPS / W;
  constexpr int NM = MODE == GEMV_GATE_UP ? 2 : 1;
  int s = 0;
  if (MODE != GEMV_GATE_UP)
    while (s + 1 < a.nseg && int(blockIdx.x) >= a.blocks_start[s + 1]) ++s;
  const int rows = a.seg[s].rows;
  const int row = (int(blockIdx.x) - a.blocks_start[s]) * ROWS + warp / W;
  const int kp = warp % W;
  const int chunk = (a.k4 + W - 1) / W;
  const int c0 = kp * chunk;
  const int c1 = min(a.k4, c0 + chunk);
  const float4* ap[NM];
#pragma unroll
  for (int m = 0; m < NM; ++m)
    ap[m] = reinterpret_cast<const float4*>(a.seg[MODE == GEMV_GATE_UP ? m : s].A) + int64_t(row < rows ? row : 0) * a.k4;
  float4 v[NM][8];
  auto load = [&](int i) {
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (row < rows && i + u * 32 < c1) v[m][u] = ld_stream_f4(ap[m] + i + u * 32);
  };
  int i = c0 + lane;
  load(i);
  pdl_launch_dependents();
  pdl_wait();
  const int k = a.k4 * 4;
  if (a.norm_w) {
    float ss = 0.0f;
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const float t = a.x[j];
      xs_f32[j] = t;
      ss += t * t;
    }
    ss = block_sum(ss, red);
    const float r = sqrtf(ss / float(k) + a.eps);
    for (int j = threadIdx.x; j < k; j += blockDim.x) xs_f32[j] = (xs_f32[j] / r) * a.norm_w[j];
  } else {
    for (int j = threadIdx.x; j < a.k4; j += blockDim.x)
      reinterpret_cast<float4*>(xs_f32)[j] = reinterpret_cast<const float4*>(a.x)[j];
  }
  __syncthreads();
  const float4* xv = reinterpret_cast<const float4*>(xs_f32);
  float acc[NM];
#pragma unroll
  for (int m = 0; m < NM; ++m) acc[m] = 0.0f;
  bool first = true;
  for (; i < c1; i += 8 * 32) {
    if (!first) load(i);
    first = false;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (row < rows && i + u * 32 < c1) {
        const float4 b = xv[i + u * 32];
#pragma unroll
        for (int m = 0; m < NM; ++m) {
          acc[m] = fmaf(v[m][u].x, b.x, acc[m]); acc[m] = fmaf(v[m][u].y, b.y, acc[m]);
          acc[m] = fmaf(v[m][u].z, b.z, acc[m]); acc[m] = fmaf(v[m][u].w, b.w, acc[m]);
        }
      }
  }
  float acc0 = warp_sum(acc[0]);
  float acc1 = NM == 2 ? warp_sum(acc[NM - 1]) : 0.0f;
  if (W > 1) {
    if (lane == 0) {
      part[0][warp] = acc0;
      part[1][warp] = acc1;
    }
    __syncthreads();
    if (kp == 0 && lane == 0) {
      acc0 = part[0][warp];
      acc1 = part[1][warp];
#pragma unroll
      for (int u = 1; u < W; ++u) {
        acc0 += part[0][warp + u];
        acc1 += part[1][warp + u];
      }
    }
  }
  if (lane == 0 && kp == 0 && row < rows) {
    float* o = a.seg[s].out + row;
    if (MODE == GEMV_STORE) *o = acc0;
    if (MODE == GEMV_ACCUM) *o = *o + acc0;
    if (MODE == GEMV_GATE_UP) *o = (acc0 / (1.0f + expf(-acc0))) * acc1;
  }
}

template <int MODE>
inline int gemv_f32_dec_launch(GemvDecArgs a, cudaStream_t st, int sm_count, bool pdl) {
  int64_t total_rows = 0;
  const int nseg = MODE == GEMV_GATE_UP ? 1 : a.nseg;
  for (int s = 0; s < nseg; ++s) total_rows += a.seg[s].rows;
  if (total_rows == 0) return SIMP_OK;
  const int64_t want = int64_t(sm_count) * 16;
  int W = 1;
  while (W < 8 && total_rows * W * (MODE == GEMV_GATE_UP ? 2 : 1) < want && a.k4 / (W * 2) >= 64) W *= 2;
  const int rows_per_block = GEMV_WARPS / W;
  int blocks = 0;
  for (int s = 0; s < nseg; ++s) {
    a.blocks_start[s] = blocks;
    blocks += (a.seg[s].rows + rows_per_block - 1) / rows_per_block;
  }
  a.blocks_start[nseg] = blocks;
  const size_t smem = size_t(a.k4) * 16;
  cudaError_t e;
  switch (W) {
    case 1: e = launch_kernel(gemv_f32_dec_kernel<1, MODE>, dim3(blocks), dim3(GEMV_WARPS * 32), smem, st, pdl, a); break;
    case 2: e = launch_kernel(gemv_f32_dec_kernel<2, MODE>, dim3(blocks), dim3(GEMV_WARPS * 32), smem, st, pdl, a); break;
    case 4: e = launch_kernel(gemv_f32_dec_kernel<4, MODE>, dim3(blocks), dim3(GEMV_WARPS * 32), smem, st, pdl, a); break;
    default: e = launch_kernel(gemv_f32_dec_kernel<8, MODE>, dim3(blocks), dim3(GEMV_WARPS * 32), smem, st, pdl, a); break;
  }
  if (e != cudaSuccess) return set_error(SIMP_ERR_CUDA, "gemv_f32_dec launch failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

}  // namespace simp
