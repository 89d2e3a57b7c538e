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
#include "sm100_ptx.cuh"

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

// Packs x (optionally x[i]*mul[i], the next rmsnorm's weight) chunk by chunk; ss_out (optional) receives the
// sum of squares of the unscaled x per chunk -- the deterministic partials of that rmsnorm.
static __global__ void __launch_bounds__(256) w4_pack_x_kernel(const float* __restrict__ x, uint8_t* __restrict__ xp,
                                                               int nchunks, const float* __restrict__ mul,
                                                               float* __restrict__ ss_out) {
  pdl_launch_dependents();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  // the norm weights never change: requested before waiting for the producer of x (they miss in L2 once per layer)
  const float mw = (mul && warp < nchunks) ? __ldg(mul + warp * 32 + lane) : 1.0f;
  pdl_wait();
  if (warp >= nchunks) return;
  const float v = x[warp * 32 + lane];
  w4_pack_chunk(mul ? v * mw : v, lane, xp + size_t(warp) * (W4_CHUNK_U4 * 16));
  if (ss_out) {
    const float q = warp_sum(v * v);
    if (lane == 0) ss_out[warp] = q;
  }
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
  // four independent accumulation chains (high/low byte x low/high nibble) keep the dp4a pipe fed
  int ah0 = 0, ah1 = 0;
  uint32_t al0 = 0, al1 = 0;
  const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t lo = ws[wd] & 0x0F0F0F0Fu;
    const uint32_t hi = (ws[wd] >> 4) & 0x0F0F0F0Fu;
    ah0 = dp4a_us(lo, xq[wd].x, ah0);
    ah1 = dp4a_us(hi, xq[wd].y, ah1);
    al0 = dp4a_uu(lo, xq[wd].z, al0);
    al1 = dp4a_uu(hi, xq[wd].w, al1);
  }
  return (ah0 + ah1) * 256 + int(al0 + al1);
}

// One matrix segment of a launch.  All segments share cols / group size / the packed input.
struct W4Seg {
  const uint8_t* qw;   // first byte of the matrix (16-byte aligned)
  const float* sc;     // first group scale of the matrix (16-byte aligned)
  const float* zr;     // first group zero, or nullptr (symmetric: zero = -8*scale)
  float* out;          // f32 result rows
  int rows;
};
enum W4Mode { W4_STORE = 0, W4_ADD = 1, W4_GATE_UP = 2 };
struct W4Args {
  W4Seg seg[3];
  int nseg;
  int cols, log2_cpg, groups_per_row;
  const uint8_t* xp;       // packed input
  // Deferred rmsnorm of the input: when ss_part != nullptr the packed input holds x[i]*w_norm[i] and every
  // dot product is multiplied by 1/sqrt(sum(ss_part[0..n_ss)) / ss_div + eps).
  const float* ss_part;
  int n_ss;
  float ss_div, eps;
  const float* res;        // W4_ADD: out[i] = res[i] + dot (segment 0 only)
  int total_tiles;         // row tiles over all segments (W4_GATE_UP: over segment 0)
  int* status;             // device error word for bounded waits
  int seg_tile_start[4];
};

// Shared-memory footprint of one pipeline stage: 8*RW rows of every streamed matrix with their scales (+zeros).
inline size_t w4_stage_bytes(int cols, int groups_per_row, int nm, bool zeros, int rw) {
  return size_t(nm) * size_t(8 * rw) * (size_t(cols / 2) + size_t(groups_per_row) * 4 * (zeros ? 2 : 1));
}

// Streaming kernel.  A block owns tiles of 8*RW consecutive rows; a tile is fetched by ONE bulk async copy
// per matrix (cp.async.bulk global -> shared, completion on an mbarrier; rows of a row-major matrix are
// contiguous) plus one for its scales, two tiles in flight.  The copies of the first two tiles are issued
// before the kernel waits for the producer of its input vector, so under programmatic dependent launch
// the weights of the next projection are already streaming while the previous kernel finishes.
// Warps then read weights, scales and the packed input from shared memory only; warp w owns rows
// w*RW .. w*RW+RW-1 of the tile, lanes split the 32-weight chunks, one shuffle reduction per row.
template <int MODE, int RW>
__global__ void __launch_bounds__(W4_WARPS * 32, 3) w4_gemv_kernel(const W4Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float sh_inv_r;
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ int abort_flag;
  constexpr int NM = MODE == W4_GATE_UP ? 2 : 1;
  constexpr int S_ROWS = 8 * RW;
  const int nchunks = a.cols >> 5;
  const int row_bytes = a.cols >> 1;
  const int sc_row = a.groups_per_row;  // floats of scale per row
  const bool has_z = a.seg[0].zr != nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_it = (nchunks + 31) >> 5;
  const size_t xs_bytes = size_t(nchunks) * (W4_CHUNK_U4 * 16);
  const size_t mat_w = size_t(S_ROWS) * row_bytes, mat_s = size_t(S_ROWS) * sc_row * 4;
  const size_t mat_bytes = mat_w + mat_s * (has_z ? 2 : 1);
  const size_t stage_bytes = mat_bytes * NM;
  uint4* xs = reinterpret_cast<uint4*>(smem);
  auto stage_ptr = [&](int st, int m) { return smem + xs_bytes + st * stage_bytes + m * mat_bytes; };

  const int my_steps = int(blockIdx.x) < a.total_tiles ? (a.total_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  auto locate = [&](int q, int& s, int& row0, int& rows) {
    const int tile = int(blockIdx.x) + q * int(gridDim.x);
    s = 0;
    if (MODE != W4_GATE_UP)
      while (s + 1 < a.nseg && tile >= a.seg_tile_start[s + 1]) ++s;
    row0 = (tile - a.seg_tile_start[s]) * S_ROWS;
    rows = a.seg[s].rows;
  };
  // Requests tile q.  Full tiles: one elected thread issues bulk copies; a ragged last tile is copied with
  // plain loads by every thread (bulk copies need 16-byte multiples) and published by the same barrier.
  auto issue = [&](int q) {
    if (q >= my_steps) return;
    int s, row0, rows;
    locate(q, s, row0, rows);
    const int st = q & 1;
    const int vr = min(S_ROWS, rows - row0);
    const uint32_t bar = ptx::smem_u32(&bars[st]);
    if (vr == S_ROWS) {
      if (threadIdx.x == 0) {
        ptx::mbar_arrive_expect_tx(bar, uint32_t(stage_bytes));
#pragma unroll
        for (int m = 0; m < NM; ++m) {
          const W4Seg& sg = a.seg[MODE == W4_GATE_UP ? m : s];
          uint8_t* dst = stage_ptr(st, m);
          ptx::bulk_load(ptx::smem_u32(dst), sg.qw + size_t(row0) * row_bytes, uint32_t(mat_w), bar);
          ptx::bulk_load(ptx::smem_u32(dst + mat_w), sg.sc + size_t(row0) * sc_row, uint32_t(mat_s), bar);
          if (has_z) ptx::bulk_load(ptx::smem_u32(dst + mat_w + mat_s), sg.zr + size_t(row0) * sc_row, uint32_t(mat_s), bar);
        }
      }
    } else {
#pragma unroll
      for (int m = 0; m < NM; ++m) {
        const W4Seg& sg = a.seg[MODE == W4_GATE_UP ? m : s];
        uint8_t* dst = stage_ptr(st, m);
        const uint4* src = reinterpret_cast<const uint4*>(sg.qw + size_t(row0) * row_bytes);
        for (int i = threadIdx.x; i < vr * (row_bytes >> 4); i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = src[i];
        for (int i = threadIdx.x; i < vr * sc_row; i += blockDim.x) {
          reinterpret_cast<float*>(dst + mat_w)[i] = sg.sc[size_t(row0) * sc_row + i];
          if (has_z) reinterpret_cast<float*>(dst + mat_w + mat_s)[i] = sg.zr[size_t(row0) * sc_row + i];
        }
      }
      __syncthreads();
      if (threadIdx.x == 0) ptx::mbar_arrive(bar);
    }
  };

  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bars[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&bars[1]), 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // Weights never change: the first two tiles are requested before waiting for the producer of the input.
  issue(0);
  issue(1);
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < nchunks * W4_CHUNK_U4; i += blockDim.x)
    xs[i] = __ldg(reinterpret_cast<const uint4*>(a.xp) + i);
  if (warp == 0) {
    float inv_r = 1.0f;
    if (a.ss_part) {
      float ss = 0.0f;
      for (int i = lane; i < a.n_ss; i += 32) ss += a.ss_part[i];
      ss = warp_sum(ss);
      inv_r = 1.0f / sqrtf(ss / a.ss_div + a.eps);
    }
    if (lane == 0) sh_inv_r = inv_r;
  }
  __syncthreads();
  const float inv_r = sh_inv_r;

  for (int q = 0; q < my_steps; ++q) {
    int s, row0, rows;
    locate(q, s, row0, rows);
    const int st = q & 1;
    if (!ptx::mbar_wait(ptx::smem_u32(&bars[st]), uint32_t(q >> 1) & 1u, &abort_flag, a.status, 10)) break;
    float acc[NM][RW];
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int r = 0; r < RW; ++r) acc[m][r] = 0.0f;
    const int wr0 = warp * RW;  // first row of this warp inside the tile
    if (row0 + wr0 < rows) {
      for (int it = 0; it < n_it; ++it) {
        const int c = lane + (it << 5);
        if (c < nchunks) {
          uint4 xq[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) xq[t] = xs[c * W4_CHUNK_U4 + t];
          const uint4 meta = xs[c * W4_CHUNK_U4 + 4];
          const float sx = __uint_as_float(meta.x), sumx = __uint_as_float(meta.y);
          const int sum16 = int(meta.z);
          const int g = c >> a.log2_cpg;
#pragma unroll
          for (int m = 0; m < NM; ++m) {
            const uint8_t* base = stage_ptr(st, m);
#pragma unroll
            for (int r = 0; r < RW; ++r) {
              if (row0 + wr0 + r < rows) {
                const uint4 w = *reinterpret_cast<const uint4*>(base + size_t(wr0 + r) * row_bytes + size_t(c) * 16);
                const int tot = w4_chunk_dot(w, xq);
                const float scale = reinterpret_cast<const float*>(base + mat_w)[(wr0 + r) * sc_row + g];
                if (!has_z) {
                  acc[m][r] = fmaf(float(tot - 8 * sum16) * sx, scale, acc[m][r]);
                } else {
                  const float z = reinterpret_cast<const float*>(base + mat_w + mat_s)[(wr0 + r) * sc_row + g];
                  acc[m][r] = fmaf(float(tot) * sx, scale, fmaf(z, sumx, acc[m][r]));
                }
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
      const float v0 = warp_sum(acc[0][r]) * inv_r;
      const float v1 = NM == 2 ? warp_sum(acc[NM - 1][r]) * inv_r : 0.0f;
      const int row = row0 + wr0 + r;
      if (lane == 0 && row < rows) {
        if (MODE == W4_STORE) a.seg[s].out[row] = v0;
        if (MODE == W4_ADD) a.seg[s].out[row] = a.res[row] + v0;
        if (MODE == W4_GATE_UP) a.seg[0].out[row] = (v0 / (1.0f + expf(-v0))) * v1;
      }
    }
    __syncthreads();  // every warp is done with stage st before it is refilled
    issue(q + 2);
  }
}

// Fills the tile bookkeeping, sizes the stages and launches.  All pointers are device pointers.
template <int MODE>
inline int w4_launch(W4Args a, cudaStream_t st, int sm_count, bool pdl = false) {
  a.status = ctx().dev_status;
  constexpr int NM = MODE == W4_GATE_UP ? 2 : 1;
  const bool zeros = a.seg[0].zr != nullptr;
  const int nseg_tiles = MODE == W4_GATE_UP ? 1 : a.nseg;
  int64_t total_rows = 0;
  for (int s = 0; s < a.nseg; ++s) {
    const bool ok = (reinterpret_cast<uintptr_t>(a.seg[s].qw) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.seg[s].sc) & 15u) == 0 &&
                    (!zeros || (reinterpret_cast<uintptr_t>(a.seg[s].zr) & 15u) == 0) && ((a.seg[s].zr != nullptr) == zeros);
    if (!ok) return set_error(SIMP_ERR_SHAPE, "w4_gemv: weights, scales and zeros of every matrix must be 16-byte aligned");
    if (s < nseg_tiles) total_rows += a.seg[s].rows;
  }
  if (total_rows == 0) return SIMP_OK;
  // Rows per warp (tile = 8*RW rows).  More rows per tile reuse the packed input better (less shared-memory
  // traffic per weight); fewer keep every SM busy on the short matrices of batch-1 decode.  Two tiles must
  // fit in shared memory next to the packed input, with room for 2-3 blocks per SM.
  const size_t xs_bytes = w4_packed_bytes(a.cols);
  int rw = 4;
  while (rw > 1 && xs_bytes + 2 * w4_stage_bytes(a.cols, a.groups_per_row, NM, zeros, rw) > 74 * 1024) rw >>= 1;
  if (rw == 1 && xs_bytes + 2 * w4_stage_bytes(a.cols, a.groups_per_row, NM, zeros, 2) <= 112 * 1024) rw = 2;
  while (rw > 1 && total_rows / (8 * rw) < 2 * int64_t(sm_count)) rw >>= 1;
  const size_t smem = xs_bytes + 2 * w4_stage_bytes(a.cols, a.groups_per_row, NM, zeros, rw);
  if (smem > 220 * 1024) return set_error(SIMP_ERR_SHAPE, "w4_gemv: row too long for the shared-memory pipeline");
  int g = 0;
  for (int s = 0; s < nseg_tiles; ++s) {
    a.seg_tile_start[s] = g;
    g += (a.seg[s].rows + 8 * rw - 1) / (8 * rw);
  }
  a.seg_tile_start[nseg_tiles] = g;
  a.total_tiles = g;
  int per_sm = int((227 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
  const int cap = sm_count * per_sm;
  const int grid = g < cap ? g : cap;
  cudaError_t e;
#define W4_LAUNCH_RW(RWV)                                                                                   \
  do {                                                                                                      \
    static bool attr_set = false;                                                                           \
    if (!attr_set) {                                                                                        \
      cudaFuncSetAttribute(w4_gemv_kernel<MODE, RWV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); \
      attr_set = true;                                                                                      \
    }                                                                                                       \
    e = launch_kernel(w4_gemv_kernel<MODE, RWV>, dim3(grid), dim3(W4_WARPS * 32), smem, st, pdl, a);        \
  } while (0)
  if (rw == 4) W4_LAUNCH_RW(4);
  else if (rw == 2) W4_LAUNCH_RW(2);
  else W4_LAUNCH_RW(1);
#undef W4_LAUNCH_RW
  if (e != cudaSuccess) return set_error(SIMP_ERR_CUDA, "w4_gemv launch failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

}  // namespace simp
