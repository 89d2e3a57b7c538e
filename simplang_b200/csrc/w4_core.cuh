// w4_core.cuh -- streaming W4 GEMV shared by the matmul_quant entry point and the decode driver.
//
// out[rows] = W4[rows,cols] . x[cols], two 4-bit weights per byte (low nibble = even flat index),
// w = q*scale + zero per group of gs consecutive weights (MatMulQuantOpLowering,
// src/mlir/lowering/ConvertSimpToMemRef.cpp:3906-4005).
//
// The kernel is HBM-bound only if the per-weight instruction count stays well below one: lop3, shf, dp4a and
// the integer multiply-add share a pipe that issues 64 lane-operations per clock and SM, while HBM delivers ~50
// weights per clock and SM.  So every block first packs the activations (w4_pack_quarter) into 16-bit block floating
// point -- per chunk of 32 inputs a scale sx = max|x|/32512 and x16 = rint(x/sx) split into two signed bytes
// x16 = 256*xh + xl -- and the integer dot products run on the tensor cores as warp-level
// mma.sync.m16n8k32 (u8 nibbles x s8 input bytes -> s32): a GEMV has one column, so the eight columns of the
// B operand carry the high and low byte planes of four different 32-input chunks, each zero outside its own
// chunk.  One group of four MMAs then yields, for 16 rows, the exact integer dot product of four chunks, every
// lane holding one (row pair, chunk) result to scale by its group's scale.  Per 8 weights of a row: 3 logic ops
// (shared by 16 rows' worth of tensor work) instead of 3 logic ops + 4 dp4a.  Rounding x to 16 bits inside each
// chunk bounds the error of a term by 1.6e-5 * max|x_chunk| * |w| -- two orders below the 1e-3 tolerance of
// the W4 path, and independent of outliers elsewhere in x.
//
// Packed layout, per chunk c (80 bytes, 5 x uint4): bytes 0..31 the high plane, 32..63 the low plane, each as
// words j = 0..3 (inputs 32c+8j .. +7) of { 4 even inputs, 4 odd inputs } -- the inputs that meet the low / high
// nibbles of weight word j -- then uint4 meta = { sx, sum(x) f32, sum(x16) i32, 0 }.
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace simp {

constexpr int W4_WARPS = 8;
constexpr int W4_CHUNK_U4 = 5;  // uint4 per packed chunk
constexpr int W4_PACK_ROUNDS = 3;   // rounds of input loads a thread keeps in flight while packing

constexpr size_t W4_SMEM_LIMIT = 220 * 1024;   // dynamic shared memory a launch may ask for

inline size_t w4_packed_bytes(int64_t cols) { return size_t(cols / 32) * W4_CHUNK_U4 * 16; }

// Eight inputs of a chunk packed by one thread, the four threads of a chunk (adjacent lanes, j = lane & 3) sharing
// the maximum and the sums by two shuffles each: thread j produces word j of both byte planes.  Every block packs
// the whole vector for itself, so the pack must be short.  All 32 lanes of a warp must call this together;
// `active` = this thread's chunk exists.
__device__ __forceinline__ void w4_pack_quarter(const float (&v)[8], bool active, int j, uint8_t* chunk) {
  float amax = 0.0f, sumx = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    amax = fmaxf(amax, fabsf(v[i]));
    sumx += v[i];
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const float inv = amax > 0.0f ? 32512.0f / amax : 0.0f;
  int sum16 = 0;
  uint32_t xh[2] = {0u, 0u}, xl[2] = {0u, 0u};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    int x16 = __float2int_rn(v[e] * inv);
    x16 = max(-32512, min(32512, x16));
    sum16 += x16;
    const int h = (x16 + 128) >> 8;   // nearest multiple of 256, in [-127, 127]
    const int l = x16 - (h << 8);     // signed low byte, in [-128, 127]
    xh[e & 1] |= uint32_t(h & 255) << (8 * (e >> 1));
    xl[e & 1] |= uint32_t(l & 255) << (8 * (e >> 1));
  }
  sumx += __shfl_xor_sync(0xffffffffu, sumx, 1);
  sumx += __shfl_xor_sync(0xffffffffu, sumx, 2);
  sum16 += __shfl_xor_sync(0xffffffffu, sum16, 1);
  sum16 += __shfl_xor_sync(0xffffffffu, sum16, 2);
  if (active) {
    *reinterpret_cast<uint2*>(chunk + j * 8) = make_uint2(xh[0], xh[1]);
    *reinterpret_cast<uint2*>(chunk + 32 + j * 8) = make_uint2(xl[0], xl[1]);
    if (j == 0)
      *reinterpret_cast<uint4*>(chunk + 64) =
          make_uint4(__float_as_uint(amax > 0.0f ? amax / 32512.0f : 0.0f), __float_as_uint(sumx), uint32_t(sum16), 0u);
  }
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
  const float* x;          // input vector (cols floats, 32-byte aligned)
  // Fused rmsnorm of the input: with mul != nullptr the packed input holds x[i]*mul[i], and with norm != 0 every
  // dot product is multiplied by 1/sqrt(sum(x^2) / ss_div + eps).
  const float* mul;
  int norm;
  float ss_div, eps;
  const float* res;        // W4_ADD: out[i] = res[i] + dot (segment 0 only)
  // L2 prefetch on behalf of a later kernel: pf_len[0] rows of pf_row_bytes bytes from each of pf_base[0..1]
  // (nullptr: none)
  const int* pf_len;
  const uint8_t* pf_base[2];
  int pf_row_bytes;
  // L2 prefetch of the NEXT launch's weights (regions of nx_bytes[i] bytes at nx_base[i], 16-byte aligned; unused
  // entries have nx_bytes 0): every block requests a share right after its own tiles, so HBM keeps streaming
  // through this launch's wait for its input, its arithmetic and the launch gap.
  const uint8_t* nx_base[6];
  uint32_t nx_bytes[6];

  // Tensor parallel (tp.n > 1): x and res are arrays of tagged 64-bit words (see TpLL) that the kernel polls for
  // tag id_x / id_res; with id_out != 0 the rows of segment 0 (W4_GATE_UP: the gated rows) go, tagged id_out, into
  // every rank's copy of the output vector at byte offset out_off of the arena (this rank's slice) instead of `out`.
  TpLL tp;
  uint32_t id_x, id_res, id_out, out_off;
  int total_tiles;         // row tiles over all segments (W4_GATE_UP: over segment 0)
  int any_ragged;          // some segment's row count is not a multiple of the tile height (its last tile is copied
                           // with plain loads instead of bulk copies)
  int* status;             // device error word for bounded waits
  int seg_tile_start[4];
#ifdef SIMP_W4_TRACE
  unsigned long long* trace;   // instrumented builds: [gridDim.x][16] globaltimer marks of this launch, or nullptr
#endif
};

#ifdef SIMP_W4_TRACE
#define W4_MARK(k) do { if (a.trace && threadIdx.x == 0) a.trace[size_t(blockIdx.x) * 16 + (k)] = ptx::globaltimer_ns(); } while (0)
#else
#define W4_MARK(k) do { } while (0)
#endif

// Shared-memory footprint of one pipeline stage: TR rows of every streamed matrix with their scales (+zeros).
inline size_t w4_stage_bytes(int cols, int groups_per_row, int nm, bool zeros, int tr) {
  return size_t(nm) * size_t(tr) * (size_t(cols / 2) + size_t(groups_per_row) * 4 * (zeros ? 2 : 1));
}

// D (16 x 8, s32) += A (16 x 32 unsigned bytes, row-major fragments) * B (32 x 8 signed bytes, column fragments).
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Shared-memory view of one tile for w4_mma_spans: matrix m starts at base + m * mat_bytes and holds its rows
// (row_bytes each), then the rows' scales at +mat_w and, when has_z, the zeros at +mat_w+mat_s.
struct W4Tile {
  const uint8_t* base;
  size_t mat_bytes, mat_w, mat_s;
  int row_bytes, sc_row;
  bool has_z;
};

// One warp, 16 rows (HALF: 8 rows) starting at tile row `r0`, spans s0, s0+sstep, ... of 128 weights.
// In the warp's MMA lane (g, t) = (lane / 4, lane % 4) reads 16 bytes -- chunk 4s+t -- of rows g and g+8; MMA j
// multiplies word j of every lane's piece (low nibbles as the first 16 k-slots, high nibbles as the second) with a
// B operand whose column n is the byte plane (n & 1) of chunk 4s + n/2 and zero in the other chunks' k-slots:
// lanes with t == g/2 load those 32 bytes from the packed input, the others pass zeros.  After the four MMAs
// lane (g, t) holds the integer dot products of chunk 4s+t with rows g and g+8 (high plane in c0/c2, low plane
// in c1/c3), which it scales and adds to acc[m][0] (row g) and acc[m][1] (row g+8).
template <int NM, bool HALF>
__device__ __forceinline__ void w4_mma_spans(const W4Tile& tl, int r0, int vrows, const uint4* __restrict__ xs, int nchunks,
                                             int log2_cpg, int s0, int sstep, int lane, float (&acc)[NM][2]) {
  const int g = lane >> 2, t = lane & 3;
  const bool va = r0 + g < vrows, vb = !HALF && r0 + g + 8 < vrows;   // rows past the tile's last row read nothing
  const bool bsel = t == (g >> 1);
  const int plane = g & 1;
  const int nspans = (nchunks + 3) >> 2;
  if constexpr (!HALF) {
    // Lean loop for the common case (a whole 16-row slab, symmetric weights, whole spans): the same arithmetic in the
    // same order, with 32-bit shared-memory addresses that advance by a constant per span and nothing predicated
    // but the B operand.  A decode launch runs this loop a handful of times per warp, so its length in instructions
    // is what it costs.
    if (!tl.has_z && r0 + 16 <= vrows) {
      const int nfull = nchunks >> 2;
      const uint32_t tile = ptx::smem_u32(tl.base);
      uint32_t xa = ptx::smem_u32(xs) + uint32_t(4 * s0 + t) * (W4_CHUNK_U4 * 16);
      uint32_t wa_addr = tile + uint32_t(r0 + g) * uint32_t(tl.row_bytes) + uint32_t(4 * s0 + t) * 16u;
      const uint32_t sc_addr = tile + uint32_t(tl.mat_w) + uint32_t(r0 + g) * uint32_t(tl.sc_row) * 4u;
      const uint32_t xstep = uint32_t(sstep) * (4 * W4_CHUNK_U4 * 16), wstep = uint32_t(sstep) * 64u;
      const uint32_t wb_off = 8u * uint32_t(tl.row_bytes), sb_off = 8u * uint32_t(tl.sc_row) * 4u;
      const uint32_t xsel = uint32_t(plane) * 32u;
      uint4 xb0 = make_uint4(0, 0, 0, 0), xb1 = xb0;
      int s = s0;
      for (; s < nfull; s += sstep, xa += xstep, wa_addr += wstep) {
        const uint4 meta = ptx::lds128(xa + 64u);
        if (bsel) {
          xb0 = ptx::lds128(xa + xsel);
          xb1 = ptx::lds128(xa + xsel + 16u);
        }
        const float sx = __uint_as_float(meta.x);
        const int m8 = -8 * int(meta.z);
        const uint32_t grp4 = uint32_t((4 * s + t) >> log2_cpg) << 2;
#pragma unroll
        for (int m = 0; m < NM; ++m) {
          const uint32_t mo = uint32_t(m) * uint32_t(tl.mat_bytes);
          const uint4 wa = ptx::lds128(wa_addr + mo), wb = ptx::lds128(wa_addr + mo + wb_off);
          const float sa = ptx::lds_f32(sc_addr + mo + grp4), sb = ptx::lds_f32(sc_addr + mo + sb_off + grp4);
          int cc[4] = {0, 0, 0, 0};
          constexpr uint32_t MK = 0x0F0F0F0Fu;
          mma_u8s8(cc, wa.x & MK, wb.x & MK, (wa.x >> 4) & MK, (wb.x >> 4) & MK, xb0.x, xb0.y);
          mma_u8s8(cc, wa.y & MK, wb.y & MK, (wa.y >> 4) & MK, (wb.y >> 4) & MK, xb0.z, xb0.w);
          mma_u8s8(cc, wa.z & MK, wb.z & MK, (wa.z >> 4) & MK, (wb.z >> 4) & MK, xb1.x, xb1.y);
          mma_u8s8(cc, wa.w & MK, wb.w & MK, (wa.w >> 4) & MK, (wb.w >> 4) & MK, xb1.z, xb1.w);
          acc[m][0] = fmaf(float(cc[0] * 256 + cc[1] + m8) * sx, sa, acc[m][0]);
          acc[m][1] = fmaf(float(cc[2] * 256 + cc[3] + m8) * sx, sb, acc[m][1]);
        }
      }
      s0 = s;   // a ragged last span (cols % 128 != 0), if it is this warp's, goes through the general loop below
    }
  }
  for (int s = s0; s < nspans; s += sstep) {
    const int c = 4 * s + t;
    const bool valid = c < nchunks;
    uint4 xb0 = make_uint4(0, 0, 0, 0), xb1 = xb0, meta = xb0;
    if (valid) {
      meta = xs[c * W4_CHUNK_U4 + 4];
      if (bsel) {
        xb0 = xs[c * W4_CHUNK_U4 + plane * 2];
        xb1 = xs[c * W4_CHUNK_U4 + plane * 2 + 1];
      }
    }
    const float sx = __uint_as_float(meta.x), sumx = __uint_as_float(meta.y);
    const int m8 = -8 * int(meta.z);
    const int grp = c >> log2_cpg;
#pragma unroll
    for (int m = 0; m < NM; ++m) {
      const uint8_t* mb = tl.base + m * tl.mat_bytes;
      const uint8_t* wp = mb + size_t(r0 + g) * tl.row_bytes + size_t(c) * 16;
      uint4 wa = make_uint4(0, 0, 0, 0), wb = wa;
      if (valid && va) wa = *reinterpret_cast<const uint4*>(wp);
      if (valid && vb) wb = *reinterpret_cast<const uint4*>(wp + size_t(8) * tl.row_bytes);
      int cc[4] = {0, 0, 0, 0};
      constexpr uint32_t MK = 0x0F0F0F0Fu;
      mma_u8s8(cc, wa.x & MK, wb.x & MK, (wa.x >> 4) & MK, (wb.x >> 4) & MK, xb0.x, xb0.y);
      mma_u8s8(cc, wa.y & MK, wb.y & MK, (wa.y >> 4) & MK, (wb.y >> 4) & MK, xb0.z, xb0.w);
      mma_u8s8(cc, wa.z & MK, wb.z & MK, (wa.z >> 4) & MK, (wb.z >> 4) & MK, xb1.x, xb1.y);
      mma_u8s8(cc, wa.w & MK, wb.w & MK, (wa.w >> 4) & MK, (wb.w >> 4) & MK, xb1.z, xb1.w);
      const float* scp = reinterpret_cast<const float*>(mb + tl.mat_w) + (r0 + g) * tl.sc_row + grp;
      const float* zp = reinterpret_cast<const float*>(mb + tl.mat_w + tl.mat_s) + (r0 + g) * tl.sc_row + grp;
      if (valid && va) {
        const int tot = cc[0] * 256 + cc[1];
        if (!tl.has_z) acc[m][0] = fmaf(float(tot + m8) * sx, scp[0], acc[m][0]);
        else acc[m][0] = fmaf(float(tot) * sx, scp[0], fmaf(zp[0], sumx, acc[m][0]));
      }
      if (valid && vb) {
        const int tot = cc[2] * 256 + cc[3];
        if (!tl.has_z) acc[m][1] = fmaf(float(tot + m8) * sx, scp[8 * tl.sc_row], acc[m][1]);
        else acc[m][1] = fmaf(float(tot) * sx, scp[8 * tl.sc_row], fmaf(zp[8 * tl.sc_row], sumx, acc[m][1]));
      }
    }
  }
}

// Streaming kernel.  A block owns tiles of TR consecutive rows; a tile is fetched by ONE bulk async copy
// per matrix (cp.async.bulk global -> shared, completion on an mbarrier; rows of a row-major matrix are
// contiguous) plus one for its scales, NS tiles in flight.  The copies of the first NS tiles are issued
// before the kernel waits for the producer of its input vector, so under programmatic dependent launch
// the weights of the next projection are already streaming while the previous kernel finishes.  The input
// vector is then packed by every block for itself (no separate pack launch, no packed copy in global memory).
// Warps then read weights, scales and the packed input from shared memory only: a tile is TR/16 slabs of 16
// rows (TR == 8: one half-used slab), the NW warps split slabs x interleaved 128-weight spans, and the
// per-warp partial sums of a row meet in a small shared array.  NW = 8 with up to three blocks per SM; for rows so
// long that only 8-row tiles would fit that way, NW = 16 with 16-row tiles and one block per SM.
template <int MODE, int TR, int NW, int NS, bool BATCH, bool LL>
__global__ void __launch_bounds__(NW * 32, NW == 8 ? 3 : 1) w4_gemv_kernel(const W4Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float sh_ss[NW];
  __shared__ __align__(8) uint64_t bars[NS];
  __shared__ int abort_flag;
  constexpr int NM = MODE == W4_GATE_UP ? 2 : 1;
  constexpr int S_ROWS = TR;
  constexpr int SL = TR == 32 ? 2 : 1;      // slabs per tile
  constexpr int KP = NW / SL;               // warps that split the spans of one slab
  constexpr bool HALF = TR == 8;
  __shared__ float red[BATCH ? NS : 2][NM][KP][S_ROWS];
  W4_MARK(0);
  const int nchunks = a.cols >> 5;
  const int row_bytes = a.cols >> 1;
  const int sc_row = a.groups_per_row;  // floats of scale per row
  const bool has_z = a.seg[0].zr != nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t xs_bytes = size_t(nchunks) * (W4_CHUNK_U4 * 16);
  const size_t mat_w = size_t(S_ROWS) * row_bytes, mat_s = size_t(S_ROWS) * sc_row * 4;
  const size_t mat_bytes = mat_w + mat_s * (has_z ? 2 : 1);
  const size_t stage_bytes = mat_bytes * NM;
  uint4* xs = reinterpret_cast<uint4*>(smem);
  auto stage_ptr = [&](int st, int m) { return smem + xs_bytes + st * stage_bytes + m * mat_bytes; };

  const int my_steps = int(blockIdx.x) < a.total_tiles ? (a.total_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1 : 0;
  auto locate_tile = [&](int q, int& s, int& row0, int& rows) {
    const int tile = int(blockIdx.x) + q * int(gridDim.x);
    s = 0;
    if (MODE != W4_GATE_UP)
      while (s + 1 < a.nseg && tile >= a.seg_tile_start[s + 1]) ++s;
    row0 = (tile - a.seg_tile_start[s]) * S_ROWS;
    rows = a.seg[s].rows;
  };
  // Batched form: a block owns at most 2 * NS tiles; where they lie is worked out once (one thread per tile, while
  // the kernel has nothing else to do) and looked up afterwards -- every warp asks for every tile several times, and
  // in a decode launch 16 warps x a few dozen instructions per question is time on the critical path.
  __shared__ int t_seg[BATCH ? 2 * NS : 1], t_row0[BATCH ? 2 * NS : 1], t_rows[BATCH ? 2 * NS : 1];
  if (BATCH && int(threadIdx.x) < 2 * NS && int(threadIdx.x) < my_steps) {
    int s, row0, rows;
    locate_tile(int(threadIdx.x), s, row0, rows);
    t_seg[threadIdx.x] = s;
    t_row0[threadIdx.x] = row0;
    t_rows[threadIdx.x] = rows;
  }
  auto locate = [&](int q, int& s, int& row0, int& rows) {
    if (BATCH) {
      s = t_seg[q];
      row0 = t_row0[q];
      rows = t_rows[q];
    } else {
      locate_tile(q, s, row0, rows);
    }
  };
  // Requests of tiles.  A full tile is P = NM x (weights, scales[, zeros]) bulk copies onto the stage's barrier.
  // One thread accepts ~2.5 M bulk-copy requests per second whatever their size, so a round of tiles is spread
  // over the warps: request r of the round (tile r / P, piece r % P) is made by lane 0 of warp r % NW; the thread
  // with piece 0 also posts the stage's byte count (a copy that completes before that only drives the barrier's
  // byte count negative, which the barrier allows).  A ragged last tile (bulk copies need 16-byte multiples) is
  // copied with plain loads by the whole block and published on the same barrier.
  const int P = NM * (has_z ? 3 : 2);
  auto issue_round = [&](int q_first, int count) {
    for (int r = warp; r < count * P; r += NW) {
      const int q = q_first + r / P, piece = r % P;
      if (q >= my_steps || lane != 0) continue;
      int s, row0, rows;
      locate(q, s, row0, rows);
      if (rows - row0 < S_ROWS) continue;   // ragged: below
      const int st = q % NS;
      const uint32_t bar = ptx::smem_u32(&bars[st]);
      const int m = piece / (has_z ? 3 : 2), part = piece % (has_z ? 3 : 2);
      const W4Seg& sg = a.seg[MODE == W4_GATE_UP ? m : s];
      uint8_t* dst = stage_ptr(st, m);
      if (piece == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(stage_bytes));
      if (part == 0) ptx::bulk_load(ptx::smem_u32(dst), sg.qw + size_t(row0) * row_bytes, uint32_t(mat_w), bar);
      else if (part == 1) ptx::bulk_load(ptx::smem_u32(dst + mat_w), sg.sc + size_t(row0) * sc_row, uint32_t(mat_s), bar);
      else ptx::bulk_load(ptx::smem_u32(dst + mat_w + mat_s), sg.zr + size_t(row0) * sc_row, uint32_t(mat_s), bar);
    }
    if (a.any_ragged)
    for (int j = 0; j < count; ++j) {   // block-uniform
      const int q = q_first + j;
      if (q >= my_steps) break;
      int s, row0, rows;
      locate(q, s, row0, rows);
      const int vr = rows - row0;
      if (vr >= S_ROWS) continue;
      const int st = q % NS;
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
      if (threadIdx.x == 0) ptx::mbar_arrive(ptx::smem_u32(&bars[st]));
    }
  };

  // The norm weights never change either (they miss in L2 once per layer): they are requested FIRST, ahead of the
  // weight tiles in the memory system's queues, so that they are at hand when the input vector arrives.
  const int ntask = nchunks * 4;
  float ssl = 0.0f;
  float4 mv[W4_PACK_ROUNDS][2];
#pragma unroll
  for (int r = 0; r < W4_PACK_ROUNDS; ++r) {
    const int q = r * int(blockDim.x) + int(threadIdx.x);
    mv[r][0] = mv[r][1] = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    if (a.mul && q < ntask) {
      mv[r][0] = __ldg(reinterpret_cast<const float4*>(a.mul) + 2 * q);
      mv[r][1] = __ldg(reinterpret_cast<const float4*>(a.mul) + 2 * q + 1);
    }
  }
  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < NS; ++k) ptx::mbar_init(ptx::smem_u32(&bars[k]), 1);
    abort_flag = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();
  // Weights never change: the first NS tiles are requested before waiting for the producer of the input.
  constexpr bool ll = LL;                     // tensor parallel: tagged-word vectors (a.tp.n > 1)
  const uint32_t tbase = LL ? ll_tag_base(a.tp) : 0u;   // requested before the wait for the predecessor
  issue_round(0, NS);
  W4_MARK(1);
  pdl_launch_dependents();
  // Optional: bring a read-only region that a LATER kernel needs (the attention kernel's key / value rows of
  // earlier positions, evicted from L2 by a token's worth of weights) into L2 while this launch streams.
  if (warp == NW - 1 && lane < 6 && a.nx_bytes[lane] != 0 && (reinterpret_cast<uintptr_t>(a.nx_base[lane]) & 15u) == 0) {
    // this block's share of region `lane`, in 16-byte units; one request of at most 64 KB per loop trip
    const uint32_t units = a.nx_bytes[lane] >> 4;
    const uint32_t u0 = uint32_t(uint64_t(units) * blockIdx.x / gridDim.x), u1 = uint32_t(uint64_t(units) * (blockIdx.x + 1) / gridDim.x);
    for (uint32_t u = u0; u < u1; u += 4096) ptx::bulk_prefetch_l2(a.nx_base[lane] + size_t(u) * 16, (min(u1, u + 4096) - u) * 16);
  }
  if (a.pf_len) {
    const int n = __ldg(a.pf_len) * a.pf_row_bytes;   // bytes per region
    for (int o = (int(blockIdx.x) * int(blockDim.x) + int(threadIdx.x)) * 128; o < n; o += int(gridDim.x) * int(blockDim.x) * 128) {
      // real loads whose values are never used (a prefetch instruction is only a hint and did not help here)
      uint32_t d0, d1;
      asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(d0) : "l"(a.pf_base[0] + o) : "memory");
      asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(d1) : "l"(a.pf_base[1] + o) : "memory");
    }
  }
  // Pack the input vector into this block's shared memory, four threads per chunk, W4_PACK_ROUNDS rounds of
  // loads in flight together.
  pdl_wait();
  W4_MARK(2);
  const uint32_t tag_x = tbase + a.id_x;
  // (The arithmetic of a round exists once in the code: a kernel of a decode step runs every instruction only a
  // few times, so what it costs is largely fetching the instruction -- compact code beats unrolled code here.)
  for (int b0 = 0; b0 < ntask; b0 += W4_PACK_ROUNDS * int(blockDim.x)) {
    float4 xv[W4_PACK_ROUNDS][2];
#pragma unroll
    for (int r = 0; r < W4_PACK_ROUNDS; ++r) {
      const int q = b0 + r * int(blockDim.x) + int(threadIdx.x);
      xv[r][0] = xv[r][1] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      if (q < ntask && ll) {   // eight tagged words: all requested, then checked (a late one is polled)
        const ll_word* xw = reinterpret_cast<const ll_word*>(a.x) + 8 * q;
        ll_word w[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = ll_load_sys(xw + i);
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          f[i] = uint32_t(w[i] >> 32) == tag_x ? __uint_as_float(uint32_t(w[i])) : ll_spin(xw + i, tag_x, a.status, 80);
        xv[r][0] = make_float4(f[0], f[1], f[2], f[3]);
        xv[r][1] = make_float4(f[4], f[5], f[6], f[7]);
      } else if (q < ntask) {
        xv[r][0] = __ldcg(reinterpret_cast<const float4*>(a.x) + 2 * q);
        xv[r][1] = __ldcg(reinterpret_cast<const float4*>(a.x) + 2 * q + 1);
      }
      if (q < ntask) {
        if (b0 > 0 && a.mul) {
          mv[r][0] = __ldg(reinterpret_cast<const float4*>(a.mul) + 2 * q);
          mv[r][1] = __ldg(reinterpret_cast<const float4*>(a.mul) + 2 * q + 1);
        }
      }
    }
    static_assert(W4_PACK_ROUNDS == 3, "the rotation below is written for three rounds");
#pragma unroll 1
    for (int r = 0; r < W4_PACK_ROUNDS; ++r) {
      if (b0 + r * int(blockDim.x) >= ntask) break;   // uniform over the block: whole warps take part in the shuffles
      const int q = b0 + r * int(blockDim.x) + int(threadIdx.x);
      float v[8] = {xv[0][0].x, xv[0][0].y, xv[0][0].z, xv[0][0].w, xv[0][1].x, xv[0][1].y, xv[0][1].z, xv[0][1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) ssl = fmaf(v[i], v[i], ssl);
      v[0] *= mv[0][0].x; v[1] *= mv[0][0].y; v[2] *= mv[0][0].z; v[3] *= mv[0][0].w;
      v[4] *= mv[0][1].x; v[5] *= mv[0][1].y; v[6] *= mv[0][1].z; v[7] *= mv[0][1].w;
      w4_pack_quarter(v, q < ntask, q & 3, smem + size_t(q >> 2) * (W4_CHUNK_U4 * 16));
      // the next round's values move into place (register moves)
      xv[0][0] = xv[1][0]; xv[0][1] = xv[1][1]; xv[1][0] = xv[2][0]; xv[1][1] = xv[2][1];
      mv[0][0] = mv[1][0]; mv[0][1] = mv[1][1]; mv[1][0] = mv[2][0]; mv[1][1] = mv[2][1];
    }
  }
  if (a.norm) {
    ssl = warp_sum(ssl);
    if (lane == 0) sh_ss[warp] = ssl;
  }
  __syncthreads();
  float inv_r = 1.0f;
  // only the threads that will write results need the norm factor (the first S_ROWS per tile of a batch)
  if (a.norm && int(threadIdx.x) < (BATCH ? NS : 1) * S_ROWS) {
    float ss = 0.0f;
#pragma unroll
    for (int w = 0; w < NW; ++w) ss += sh_ss[w];
    inv_r = 1.0f / sqrtf(ss / a.ss_div + a.eps);
  }
  const int slab = warp % SL, kpart = warp / SL;
  W4_MARK(3);
  const int nspans = (nchunks + 3) >> 2;

  if constexpr (!BATCH) {
    // Streaming form (a block owns more tiles than there are stages): one tile at a time, the other stages in flight.
    for (int q = 0; q < my_steps; ++q) {
      int s, row0, rows;
      locate(q, s, row0, rows);
      const int st = q % NS, rb = q & 1;   // weight stage; buffer of the partial sums
      // residual rows are requested before the tile's arithmetic so that their latency is not paid in the epilogue
      float resid = 0.0f;
      if (MODE == W4_ADD && int(threadIdx.x) < S_ROWS && row0 + int(threadIdx.x) < rows)
        resid = ll ? ll_get(reinterpret_cast<const ll_word*>(a.res) + row0 + int(threadIdx.x), tbase + a.id_res, a.status, 82)
                   : __ldcg(a.res + row0 + int(threadIdx.x));
      if (!ptx::mbar_wait(ptx::smem_u32(&bars[st]), uint32_t(q / NS) & 1u, &abort_flag, a.status, 10)) break;
      float acc[NM][2];
#pragma unroll
      for (int m = 0; m < NM; ++m) acc[m][0] = acc[m][1] = 0.0f;
      W4Tile tl;
      tl.base = stage_ptr(st, 0);
      tl.mat_bytes = mat_bytes;
      tl.mat_w = mat_w;
      tl.mat_s = mat_s;
      tl.row_bytes = row_bytes;
      tl.sc_row = sc_row;
      tl.has_z = has_z;
      if (row0 + slab * 16 < rows) w4_mma_spans<NM, HALF>(tl, slab * 16, S_ROWS, xs, nchunks, a.log2_cpg, kpart, KP, lane, acc);
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int h = 0; h < (HALF ? 1 : 2); ++h) {
          float v = acc[m][h];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if ((lane & 3) == 0) red[rb][m][kpart][slab * 16 + (lane >> 2) + 8 * h] = v;
        }
      __syncthreads();  // partial sums published; every warp is done with stage st before it is refilled
      issue_round(q + NS, 1);
      if (threadIdx.x < S_ROWS) {
        const int row = row0 + int(threadIdx.x);
        float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
        for (int k = 0; k < KP; ++k) {
          v0 += red[rb][0][k][threadIdx.x];
          if (NM == 2) v1 += red[rb][NM - 1][k][threadIdx.x];
        }
        v0 *= inv_r;
        v1 *= inv_r;
        if (row < rows) {
          const float val = MODE == W4_STORE ? v0 : (MODE == W4_ADD ? resid + v0 : (v0 / (1.0f + expf(-v0))) * v1);
          if (ll && a.id_out != 0 && (MODE == W4_GATE_UP || s == 0)) ll_store_all(a.tp, a.out_off + uint32_t(row) * 8u, val, tbase + a.id_out);
          else a.seg[MODE == W4_GATE_UP ? 0 : s].out[row] = val;
        }
      }
    }
    W4_MARK(15);
    return;
  }
  // Batched form (decode-sized launches: a block owns no more tiles than there are stages, all of them requested
  // before the input vector was even available).  One tile at a time (wait, spans, block-wide sync, cross-warp sum,
  // store, next tile) would be a chain of short dependent steps; here every warp runs its spans over ALL tiles of
  // the block back to back, and one block-wide sync and one round of cross-warp sums serve them all.
  const int bsz = NS;
  for (int q0 = 0; q0 < my_steps; q0 += bsz) {
    const int nb = min(bsz, my_steps - q0);
    // residual rows are requested before the arithmetic so that their latency is not paid in the epilogue
    float resid = 0.0f;
    int e_s = 0, e_row0 = 0, e_rows = 0;
    const int e_tile = int(threadIdx.x) / S_ROWS, e_r = int(threadIdx.x) % S_ROWS;
    if (e_tile < nb) {
      locate(q0 + e_tile, e_s, e_row0, e_rows);
      if (MODE == W4_ADD && e_row0 + e_r < e_rows)
        resid = ll ? ll_get(reinterpret_cast<const ll_word*>(a.res) + e_row0 + e_r, tbase + a.id_res, a.status, 82)
                   : __ldcg(a.res + e_row0 + e_r);
    }
    bool ok = true;
#pragma unroll 1
    for (int j = 0; j < nb && ok; ++j) {
      {
        const int q = q0 + j;
        int s, row0, rows;
        locate(q, s, row0, rows);
        const int st = q % NS;
        if (!ptx::mbar_wait(ptx::smem_u32(&bars[st]), uint32_t(q / NS) & 1u, &abort_flag, a.status, 10)) ok = false;
        if (ok) {
          if (j == 0) W4_MARK(4);
          float acc[NM][2];
#pragma unroll
          for (int m = 0; m < NM; ++m) acc[m][0] = acc[m][1] = 0.0f;
          W4Tile tl;
          tl.base = stage_ptr(st, 0);
          tl.mat_bytes = mat_bytes;
          tl.mat_w = mat_w;
          tl.mat_s = mat_s;
          tl.row_bytes = row_bytes;
          tl.sc_row = sc_row;
          tl.has_z = has_z;
          // first span of this warp in tile j: the round-robin over the KP warps of a slab continues across tiles,
          // so e.g. 25 spans per tile over 16 warps still balance over the batch
          const int s0 = (kpart + KP - (j * nspans) % KP) % KP;
          if (row0 + slab * 16 < rows)
            w4_mma_spans<NM, HALF>(tl, slab * 16, S_ROWS, xs, nchunks, a.log2_cpg, s0, KP, lane, acc);
#pragma unroll
          for (int m = 0; m < NM; ++m)
#pragma unroll
            for (int h = 0; h < (HALF ? 1 : 2); ++h) {
              float v = acc[m][h];
              v += __shfl_xor_sync(0xffffffffu, v, 1);
              v += __shfl_xor_sync(0xffffffffu, v, 2);
              if ((lane & 3) == 0) red[j][m][kpart][slab * 16 + (lane >> 2) + 8 * h] = v;
            }
        }
      }
    }
    if (!ok) break;   // abort_flag is block-wide: every thread's wait has failed
    __syncthreads();  // partial sums published; every warp is done with the stages before they are refilled
    W4_MARK(5);
    // the stages of this batch are refilled (every thread makes the call: a ragged tile is copied by the whole block)
    issue_round(q0 + NS, nb);
    if (e_tile < nb) {
      const int row = e_row0 + e_r;
      float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
      for (int k = 0; k < KP; ++k) {
        v0 += red[e_tile][0][k][e_r];
        if (NM == 2) v1 += red[e_tile][NM - 1][k][e_r];
      }
      v0 *= inv_r;
      v1 *= inv_r;
      if (row < e_rows) {
        const float val = MODE == W4_STORE ? v0 : (MODE == W4_ADD ? resid + v0 : (v0 / (1.0f + expf(-v0))) * v1);
        if (ll && a.id_out != 0 && (MODE == W4_GATE_UP || e_s == 0)) ll_store_all(a.tp, a.out_off + uint32_t(row) * 8u, val, tbase + a.id_out);
        else a.seg[MODE == W4_GATE_UP ? 0 : e_s].out[row] = val;
      }
    }
    if (q0 + bsz < my_steps) __syncthreads();   // `red` is rewritten by the next batch
  }
  W4_MARK(15);
}

// Fills the tile bookkeeping, sizes the stages and launches.  All pointers are device pointers.
template <int MODE>
// grid_out: receives the number of blocks; dry_run: only plan (nothing is launched).
inline int w4_launch(W4Args a, cudaStream_t st, int sm_count, bool pdl = false, int* grid_out = nullptr, bool dry_run = false) {
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
  if ((reinterpret_cast<uintptr_t>(a.x) & 15u) || (reinterpret_cast<uintptr_t>(a.mul) & 15u))
    return set_error(SIMP_ERR_SHAPE, "w4_gemv: the input vector and the norm weights must be 16-byte aligned");
  // Rows per tile.  Larger tiles mean fewer barriers per weight; smaller ones keep every SM busy on the short
  // matrices of batch-1 decode.  Two tiles must fit in shared memory next to the packed input, with room for
  // 2-3 blocks per SM.
  const size_t xs_bytes = w4_packed_bytes(a.cols);
  auto need = [&](int tr, int ns = 2) { return xs_bytes + ns * w4_stage_bytes(a.cols, a.groups_per_row, NM, zeros, tr); };
  int tr = 32;
  while (tr > 8 && need(tr) > 74 * 1024) tr >>= 1;
  if (tr == 8 && need(16) <= 112 * 1024) tr = 16;
  while (tr > 8 && total_rows / tr < int64_t(sm_count)) tr >>= 1;
  // Wide form: 16 warps on 16-row tiles, one block per SM, as many stages as fit (up to 4).  Chosen when rows are so
  // long that three 8-warp blocks per SM would be left with 8-row tiles (half of every MMA unused, and every
  // block packs the input vector for itself), and for launches of a few tiles per SM (batch-1 decode), where the
  // fixed costs of a launch dominate: one pack per SM instead of three, half the dependent rounds per tile.
  const bool wide_fit = need(16) <= 220 * 1024 && total_rows / 16 >= int64_t(sm_count);
  bool wide = wide_fit && ((tr == 8 && need(16) > 112 * 1024) || total_rows / 16 <= 8 * int64_t(sm_count));
  int ns = 2;
  if (wide) {
    tr = 16;
    // as many stages as fit, up to 4 -- or up to 6 when that lets every block hold its whole share of a decode-sized
    // launch at once (9600 rows are 600 tiles on 148 SMs: eight blocks own five)
    const int64_t tiles16 = (total_rows + 15) / 16;
    const int share = int((tiles16 + sm_count - 1) / sm_count);
    const int want = share > 4 && share <= 6 ? share : 4;
    while (ns < want && need(16, ns + 1) <= 200 * 1024) ++ns;
  }
  const size_t smem = need(tr, ns);
  if (smem > W4_SMEM_LIMIT) return set_error(SIMP_ERR_SHAPE, "w4_gemv: row too long for the shared-memory pipeline");
  int g = 0;
  for (int s = 0; s < nseg_tiles; ++s) {
    a.seg_tile_start[s] = g;
    g += (a.seg[s].rows + tr - 1) / tr;
  }
  a.seg_tile_start[nseg_tiles] = g;
  a.total_tiles = g;
  a.any_ragged = 0;
  for (int s = 0; s < nseg_tiles; ++s)
    if (a.seg[s].rows % tr != 0) a.any_ragged = 1;
  int per_sm = int((227 * 1024) / (smem + 4096));
  per_sm = wide || per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
  const int cap = sm_count * per_sm;
  const int grid = g < cap ? g : cap;
  if (grid_out) *grid_out = grid;
  if (dry_run) return SIMP_OK;
  cudaError_t e;
  // decode-sized launches (a block owns at most two rounds of stages) take the batched form of the kernel
  const bool batch = int64_t(g) <= int64_t(grid) * ns * 2;
  const bool tagged = a.tp.n > 1;   // tensor parallel: the tagged-word form of the kernel
#define W4_LAUNCH_B(TRV, NWV, NSV, BV, LV)                                                                  \
  do {                                                                                                      \
    static bool attr_set = false;                                                                           \
    if (!attr_set) {                                                                                        \
      cudaFuncSetAttribute(w4_gemv_kernel<MODE, TRV, NWV, NSV, BV, LV>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024); \
      attr_set = true;                                                                                      \
    }                                                                                                       \
    e = launch_kernel(w4_gemv_kernel<MODE, TRV, NWV, NSV, BV, LV>, dim3(grid), dim3(NWV * 32), smem, st, pdl, a); \
  } while (0)
#define W4_LAUNCH_TR(TRV, NWV, NSV)                                                                         \
  do {                                                                                                      \
    if (batch && tagged) W4_LAUNCH_B(TRV, NWV, NSV, true, true);                                            \
    else if (batch) W4_LAUNCH_B(TRV, NWV, NSV, true, false);                                                \
    else if (tagged) W4_LAUNCH_B(TRV, NWV, NSV, false, true);                                               \
    else W4_LAUNCH_B(TRV, NWV, NSV, false, false);                                                          \
  } while (0)
  if (wide && ns == 6) W4_LAUNCH_TR(16, 16, 6);
  else if (wide && ns == 5) W4_LAUNCH_TR(16, 16, 5);
  else if (wide && ns == 4) W4_LAUNCH_TR(16, 16, 4);
  else if (wide && ns == 3) W4_LAUNCH_TR(16, 16, 3);
  else if (wide) W4_LAUNCH_TR(16, 16, 2);
  else if (tr == 32) W4_LAUNCH_TR(32, 8, 2);
  else if (tr == 16) W4_LAUNCH_TR(16, 8, 2);
  else W4_LAUNCH_TR(8, 8, 2);
#undef W4_LAUNCH_TR
#undef W4_LAUNCH_B
  if (e != cudaSuccess) return set_error(SIMP_ERR_CUDA, "w4_gemv launch failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

}  // namespace simp
