// w4_core.cuh -- streaming W4 GEMV shared by the matmul_quant entry point and the decode driver.
//
// out[rows] = W4[rows,cols] . x[cols], two 4-bit weights per byte (low nibble = even flat index),
// w = q*scale + zero per group of gs consecutive weights (MatMulQuantOpLowering,
// src/mlir/lowering/ConvertSimpToMemRef.cpp:3906-4005).
//
// The kernel is HBM-bound only if the per-weight instruction count stays near one, so the
// activations are first packed (w4_pack_x_kernel) into 16-bit block floating point: per chunk of
// 32 inputs a scale sx = max|x|/32767 and x16 = rint(x/sx) split into a signed high byte and an
// unsigned low byte, laid out so that one masked weight word (4 nibbles as 4 bytes) meets 4 input
// bytes in one dp4a.  Per 8 weights: 3 logic ops + 4 dp4a, exact integer accumulation; per chunk
// one int->float conversion and one FMA with scale*sx.  Rounding x to 16 bits inside each chunk
// bounds the error of a term by 1.5e-5 * max|x_chunk| * |w| -- two orders below the 1e-3
// tolerance of the W4 path, and independent of outliers elsewhere in x.
//
// Packed layout, per chunk c (80 bytes, 5 x uint4): words wd = 0..3 cover inputs 32c+8wd .. +7:
//   uint4 wd = { XH_even, XH_odd, XL_even, XL_odd }  (even/odd = the inputs paired with the low /
//   high nibbles of the weight word), then uint4 meta = { sx, sum(x) f32, sum(x16) i32, 0 }.
// The 80-byte stride makes the 128-bit shared-memory reads of 8 neighbouring lanes conflict-free.
#pragma once
#include "common.cuh"

namespace simp {

constexpr int W4_WARPS = 8;
constexpr int W4_CHUNK_U4 = 5;  // uint4 per packed chunk

inline size_t w4_packed_bytes(int64_t cols) { return size_t(cols / 32) * W4_CHUNK_U4 * 16; }

// One warp per 32-input chunk.  `x` may be produced by a fused prologue: see w4_pack_value().
__device__ __forceinline__ void w4_pack_chunk(float xv, int lane, uint8_t* chunk_bytes) {
  const float amax = warp_max(fabsf(xv));
  const float inv = amax > 0.0f ? 32767.0f / amax : 0.0f;
  int x16 = __float2int_rn(xv * inv);
  x16 = max(-32767, min(32767, x16));
  const int xh = x16 >> 8;    // signed high byte, floor
  const int xl = x16 & 255;   // unsigned low byte: x16 == xh*256 + xl
  const int wd = lane >> 3, j = lane & 7;
  const int pos = wd * 16 + (j & 1) * 4 + (j >> 1);
  chunk_bytes[pos] = uint8_t(xh);
  chunk_bytes[pos + 8] = uint8_t(xl);
  const float sumx = warp_sum(xv);
  int sum16 = x16;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum16 += __shfl_xor_sync(0xffffffffu, sum16, o);
  if (lane == 0) {
    uint4 meta;
    meta.x = __float_as_uint(amax > 0.0f ? amax / 32767.0f : 0.0f);
    meta.y = __float_as_uint(sumx);
    meta.z = uint32_t(sum16);
    meta.w = 0;
    *reinterpret_cast<uint4*>(chunk_bytes + 64) = meta;
  }
}

static __global__ void __launch_bounds__(256) w4_pack_x_kernel(const float* __restrict__ x, uint8_t* __restrict__ xp,
                                                        int nchunks) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= nchunks) return;
  w4_pack_chunk(x[warp * 32 + lane], lane, xp + size_t(warp) * (W4_CHUNK_U4 * 16));
}

__device__ __forceinline__ uint4 ldg_nc_u4(const uint4* p) {
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(p));
  return v;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {  // unsigned a bytes x signed b bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// sum_j q_j * x16_j over one 32-weight chunk: weights `w` (4 words), packed inputs `xq` (4 uint4).
__device__ __forceinline__ int w4_chunk_dot(const uint4& w, const uint4* xq) {
  int ah = 0;
  uint32_t al = 0;
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t lo = ws[wd] & 0x0F0F0F0Fu;
    const uint32_t hi = (ws[wd] >> 4) & 0x0F0F0F0Fu;
    ah = dp4a_us(lo, xq[wd].x, ah);
    ah = dp4a_us(hi, xq[wd].y, ah);
    al = dp4a_uu(lo, xq[wd].z, al);
    al = dp4a_uu(hi, xq[wd].w, al);
  }
  return ah * 256 + int(al);
}

// One matrix segment of a launch.  All segments share cols / group size / the packed input.
struct W4Seg {
  const uint8_t* qw;   // first byte of the matrix (16-byte aligned)
  const float* sc;     // first group scale of the matrix
  const float* zr;     // first group zero, or nullptr (symmetric: zero = -8*scale)
  float* out;
  int rows;
};
enum W4Mode { W4_STORE = 0, W4_ADD = 1, W4_GATE_UP = 2 };
struct W4Args {
  W4Seg seg[3];
  int nseg;
  int cols, log2_cpg, groups_per_row;
  const uint8_t* xp;     // packed input
  const float* res;      // W4_ADD: out[i] = res[i] + dot   (segment 0 only)
  int total_groups;      // row groups over all segments (W4_GATE_UP: over segment 0)
  int seg_group_start[4];
};

constexpr int W4_R = 2;                       // rows per warp per pass
constexpr int W4_ROWS_PER_GROUP = W4_WARPS * W4_R;

template <int MODE>
__global__ void __launch_bounds__(W4_WARPS * 32, 3) w4_gemv_kernel(const W4Args a) {
  extern __shared__ __align__(16) uint4 xs[];
  const int nchunks = a.cols >> 5;
  for (int i = threadIdx.x; i < nchunks * W4_CHUNK_U4; i += blockDim.x)
    xs[i] = __ldg(reinterpret_cast<const uint4*>(a.xp) + i);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_it = (nchunks + 31) >> 5;
  const int64_t row_u4 = nchunks;  // uint4 of weights per row
  constexpr int NM = MODE == W4_GATE_UP ? 2 : 1;  // matrices streamed together
  for (int grp = blockIdx.x; grp < a.total_groups; grp += gridDim.x) {
    int s = 0;
    if (MODE != W4_GATE_UP) {
      while (s + 1 < a.nseg && grp >= a.seg_group_start[s + 1]) ++s;
    }
    const int row0 = (grp - a.seg_group_start[s]) * W4_ROWS_PER_GROUP + warp * W4_R;
    const int rows = a.seg[s].rows;
    if (row0 >= rows) continue;
    float acc[NM][W4_R];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int r = 0; r < W4_R; ++r) acc[m][r] = 0.0f;
    constexpr int U = MODE == W4_GATE_UP ? 2 : 4;  // chunk-steps whose loads are issued together
    for (int it0 = 0; it0 < n_it; it0 += U) {
      uint4 wv[U][NM][W4_R];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = lane + ((it0 + u) << 5);
#pragma unroll
        for (int m = 0; m < NM; ++m)
#pragma unroll
          for (int r = 0; r < W4_R; ++r) {
            const W4Seg& sg = a.seg[MODE == W4_GATE_UP ? m : s];
            if (c < nchunks && row0 + r < rows)
              wv[u][m][r] = ldg_nc_u4(reinterpret_cast<const uint4*>(sg.qw) + int64_t(row0 + r) * row_u4 + c);
            else
              wv[u][m][r] = make_uint4(0, 0, 0, 0);
          }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = lane + ((it0 + u) << 5);
        if (c < nchunks) {
          uint4 xq[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) xq[t] = xs[c * W4_CHUNK_U4 + t];
          const uint4 meta = xs[c * W4_CHUNK_U4 + 4];
          const float sx = __uint_as_float(meta.x), sumx = __uint_as_float(meta.y);
          const int sum16 = int(meta.z);
          const int g = c >> a.log2_cpg;
#pragma unroll
          for (int m = 0; m < NM; ++m)
#pragma unroll
            for (int r = 0; r < W4_R; ++r) {
              if (row0 + r < rows) {
                const W4Seg& sg = a.seg[MODE == W4_GATE_UP ? m : s];
                const int tot = w4_chunk_dot(wv[u][m][r], xq);
                const int64_t sidx = int64_t(row0 + r) * a.groups_per_row + g;
                const float scale = __ldg(sg.sc + sidx);
                if (sg.zr == nullptr) {
                  acc[m][r] = fmaf(float(tot - 8 * sum16) * sx, scale, acc[m][r]);
                } else {
                  acc[m][r] = fmaf(float(tot) * sx, scale, fmaf(__ldg(sg.zr + sidx), sumx, acc[m][r]));
                }
              }
            }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < W4_R; ++r) {
      float v0 = warp_sum(acc[0][r]);
      float v1 = NM == 2 ? warp_sum(acc[NM - 1][r]) : 0.0f;
      if (lane == 0 && row0 + r < rows) {
        if (MODE == W4_STORE) a.seg[s].out[row0 + r] = v0;
        if (MODE == W4_ADD) a.seg[s].out[row0 + r] = a.res[row0 + r] + v0;
        if (MODE == W4_GATE_UP) a.seg[0].out[row0 + r] = (v0 / (1.0f + expf(-v0))) * v1;
      }
    }
  }
}

// Fills the group bookkeeping and launches.  All pointers are device pointers.
template <int MODE>
inline int w4_launch(W4Args a, cudaStream_t st, int sm_count) {
  int g = 0;
  const int nseg_groups = MODE == W4_GATE_UP ? 1 : a.nseg;
  for (int s = 0; s < nseg_groups; ++s) {
    a.seg_group_start[s] = g;
    g += (a.seg[s].rows + W4_ROWS_PER_GROUP - 1) / W4_ROWS_PER_GROUP;
  }
  a.seg_group_start[nseg_groups] = g;
  a.total_groups = g;
  if (g == 0) return SIMP_OK;
  const size_t smem = w4_packed_bytes(a.cols);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(w4_gemv_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr_set = true;
  }
  const int cap = sm_count * 3;
  const int grid = g < cap ? g : cap;
  w4_gemv_kernel<MODE><<<grid, W4_WARPS * 32, smem, st>>>(a);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

}  // namespace simp
