// gemm_f32_tc.cu -- tensor_matmul on f32 for GEMM-sized shapes on the tensor cores, at f32 accuracy (3 x TF32).
//
// Semantics: TensorMatMulOpLowering f32 branch (src/mlir/lowering/ConvertSimpToMemRef.cpp:2884-3291): C[M,N] = A[M,K] . B,
// f32 multiply-add; B as [K,N] or, for tensor_matmul_nt, [N,K]; `accumulate` adds into C (simp.matmul, :1794-1920).
//
// A plain TF32 product keeps 10 mantissa bits of each operand and would miss the 1e-4 relative tolerance of this
// path; every operand is therefore split into two TF32 numbers, x = hi + lo exactly up to 2^-22 |x|
// (hi = x rounded to TF32, lo = (x - hi) rounded to TF32), and the product is formed as
//     A . B  ~=  A_lo . B_hi + A_hi . B_lo + A_hi . B_hi          (the dropped A_lo . B_lo term is ~2^-22 relative)
// by three tcgen05.mma.kind::tf32 instructions per K step into the same f32 accumulator in TMEM.
//
// Two passes:
//  1. split: A -> A_hi, A_lo [M, Kp] and B -> B_hi, B_lo [N, Kp] (K-major planes, Kp = K rounded up to 32 and zero
//     filled; B given as [K,N] is transposed on the way) in library scratch.  3 x the operand bytes of HBM traffic,
//     a few percent of the GEMM's time at the sizes this path takes.
//  2. GEMM: the 2-CTA structure of the int8 kernel (gemm_i8.cu): a pair of CTAs owns a 256 x 256 tile, each CTA
//     TMA-loads its own 128 rows of the four planes (128-byte swizzle, 3 stages of 64 KB), the even CTA issues
//     tcgen05.mma.cta_group::2.kind::tf32 (M 256, N 256, K 8), accumulators double-buffered in TMEM, four epilogue
//     warps per CTA move TMEM -> registers -> swizzled shared tile -> TMA store (TMA f32 reduce-add for `accumulate`).
//     K is accumulated in TMEM in chunks of 2048 (F_CHUNK_KB) that are added into C one after the other; shapes with
//     few tiles deal (tile, chunk) units to the CTA pairs instead (split K, see F32Params::splitk).
// All waits are bounded (mbar_wait): on expiry the library status word is set and the kernel drains.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace simp {

using namespace ptx;

int make_map_f32(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int box_outer, bool operand);

namespace {

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
__device__ __forceinline__ void split2(float x, float& hi, float& lo) {
  hi = to_tf32(x);
  lo = to_tf32(x - hi);
}

// src [rows, k] row-major (row pitch ld) -> hi, lo [rows, kp]; columns k..kp-1 are zero.  One thread per four
// elements (kp is a multiple of 32; `vec`: k % 4 == 0 and src 16-byte aligned, so the loads are 16-byte loads too).
__global__ void __launch_bounds__(256) split_rows_kernel(const float* __restrict__ src, int64_t rows, int64_t k, int64_t ld,
                                                         float* __restrict__ hi, float* __restrict__ lo, int64_t kp, int vec) {
  const int64_t col = (int64_t(blockIdx.y) * 256 + threadIdx.x) * 4;
  const int64_t row = blockIdx.x;
  if (col >= kp) return;
  float x[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (vec && col + 4 <= k) {
    const float4 v = __ldg(reinterpret_cast<const float4*>(src + row * ld + col));
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (col + i < k) x[i] = __ldg(src + row * ld + col + i);
  }
  float h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) split2(x[i], h[i], l[i]);
  *reinterpret_cast<float4*>(hi + row * kp + col) = make_float4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<float4*>(lo + row * kp + col) = make_float4(l[0], l[1], l[2], l[3]);
}

// src [k, n] row-major -> hi, lo [n, kp] (transposed), zero fill for k..kp-1.  32 x 32 tiles through shared memory.
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ src, int64_t k, int64_t n,
                                                              float* __restrict__ hi, float* __restrict__ lo, int64_t kp) {
  __shared__ float t[32][33];
  const int64_t n0 = int64_t(blockIdx.x) * 32, k0 = int64_t(blockIdx.y) * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int64_t kk = k0 + r, nn = n0 + tx;
    t[r][tx] = (kk < k && nn < n) ? __ldg(src + kk * n + nn) : 0.0f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int64_t nn = n0 + r, kk = k0 + tx;
    if (nn < n && kk < kp) {
      float h, l;
      split2(t[tx][r], h, l);
      hi[nn * kp + kk] = h;
      lo[nn * kp + kk] = l;
    }
  }
}

constexpr int F_BK = 32;                       // floats per K block: 128-byte rows
constexpr int F_STAGES = 3;
constexpr int F_PLANE = 128 * 128;             // one CTA's 128 rows x 128 bytes of one plane
constexpr int F_STAGE_BYTES = 4 * F_PLANE;     // A_hi, A_lo, B_hi, B_lo
constexpr int F_BN = 256;
constexpr int F_THREADS = 192;
constexpr int F_TMEM_COLS = 512;
constexpr int F_EPI_BYTES = 4 * 2 * 4096;      // per epilogue warp: two 32 x 32 f32 staging tiles
// The tensor cores add into the f32 accumulator with truncation, so the error of a long accumulation grows with K
// (measured 3.4e-5 of max|C| at K = 4096, three instructions per 8 floats of K).  The accumulation is therefore cut
// into chunks of 2048 floats of K: the first chunk of a tile is stored (or added, for `accumulate`), every later one
// is added into C by a TMA reduce-add (a round-to-nearest f32 add in L2), in chunk order.
constexpr int F_CHUNK_KB = 64;
constexpr size_t F_SMEM = size_t(F_STAGES) * F_STAGE_BYTES + F_EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct F32Params {
  int M, N;
  int tiles_m, tiles_n, num_kb;
  int chunk_kb;     // K blocks accumulated in TMEM before the partial sum is added into C (see F_CHUNK_KB)
  int splitk;       // 1: the (tile, chunk) units are dealt round-robin to the CTA pairs and every unit is added into a
                    //    zeroed (or, for `accumulate`, the caller's) C -- for shapes with fewer tiles than CTA pairs
  uint32_t idesc;
  int accumulate;
  int* status;
};

// Instruction descriptor for kind::tf32: f32 accumulator, TF32 operands, both K-major.
constexpr uint32_t make_idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                 uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tile_coords_f(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // groups of 16 row-tiles, column-major inside a group: one wave of CTA pairs touches a compact block
  constexpr int G = 16;
  const int per_group = G * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int gsz = min(G, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % gsz;
  tn = in_group / gsz;
}

// Work of one CTA pair: units of (tile, chunk of K blocks).  Whole tiles: tile = pair + t * num_pairs, its chunks in
// order (`first` marks the chunk that may store instead of add).  Split K: unit u = pair + i * num_pairs.
struct UnitIter {
  int i = 0;
};
__device__ __forceinline__ bool next_unit(const F32Params& p, int pair, int num_pairs, UnitIter& it, int& tile, int& kc,
                                          bool& first) {
  const int nch = (p.num_kb + p.chunk_kb - 1) / p.chunk_kb;
  const int num_tiles = p.tiles_m * p.tiles_n;
  if (p.splitk) {
    const int u = pair + it.i * num_pairs;
    if (u >= num_tiles * nch) return false;
    tile = u / nch;
    kc = (u - tile * nch) * p.chunk_kb;
    first = false;
  } else {
    const int t = it.i / nch;
    tile = pair + t * num_pairs;
    if (tile >= num_tiles) return false;
    kc = (it.i - t * nch) * p.chunk_kb;
    first = kc == 0;
  }
  ++it.i;
  return true;
}

// Epilogue of one 128 x 256 f32 accumulator half for the 32 rows owned by this warp: TMEM -> registers -> 128-byte
// swizzled shared tile -> TMA store (or TMA reduce-add) of 32 x 32 boxes, two boxes in flight.
__device__ __forceinline__ void epilogue_rows_f32(const CUtensorMap* tmap_c, const F32Params& p, uint32_t tmem_acc, int q,
                                                  int lane, int row0, int n0, uint32_t stage_smem, uint32_t& nstore,
                                                  bool add) {
#pragma unroll 1
  for (int ch = 0; ch < F_BN / 32; ++ch) {
    uint32_t r[32];
    const int c0 = n0 + ch * 32;
    if (lane == 0) tma_store_wait_read<1>();   // at most the previous store (other buffer) is still reading
    __syncwarp();
    tmem_ld_32x32(tmem_acc + (uint32_t(q * 32) << 16) + uint32_t(ch * 32), r);
    tmem_ld_wait();
    if (row0 < p.M && c0 < p.N) {
      const uint32_t buf = stage_smem + (nstore & 1u) * 4096u;
      ++nstore;
      const uint32_t rowaddr = buf + uint32_t(lane) * 128u;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t addr = rowaddr + (uint32_t(j ^ (lane & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(r[4 * j]), "r"(r[4 * j + 1]),
                     "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                     : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if (add) tma_reduce_add_2d(tmap_c, buf, c0, row0);
        else tma_store_2d(tmap_c, buf, c0, row0);
        tma_store_commit();
      }
    }
  }
}

__global__ void __launch_bounds__(F_THREADS, 1)
    gemm_tf32x3_2cta_kernel(const __grid_constant__ CUtensorMap map_ahi, const __grid_constant__ CUtensorMap map_alo,
                            const __grid_constant__ CUtensorMap map_bhi, const __grid_constant__ CUtensorMap map_blo,
                            const __grid_constant__ CUtensorMap map_c, const F32Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + F_STAGES * F_STAGE_BYTES;
  const uint32_t bar_base = epi_base + F_EPI_BYTES;
  // barriers (8 bytes each): full[F_STAGES], empty[F_STAGES], tfull[2], tempty[2]; then the TMEM slot and the abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (F_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * F_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * F_STAGES + 2 + a); };
  uint8_t* bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_generic + 8 * (2 * F_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * F_STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0: even CTA (issues the MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&map_ahi);
    prefetch_tensormap(&map_alo);
    prefetch_tensormap(&map_bhi);
    prefetch_tensormap(&map_blo);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), F_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      UnitIter it;
      int tile, kc;
      bool first;
      while (ok && next_unit(p, pair, num_pairs, it, tile, kc, first)) {
        int tm, tn;
        tile_coords_f(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * 256 + int(cta_rank) * 128, n0 = tn * F_BN + int(cta_rank) * 128;
        const int kend = min(p.num_kb, kc + p.chunk_kb);
        for (int kb = kc; kb < kend; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 21)) { ok = false; break; }
          const uint32_t s0 = smem_base + stage * F_STAGE_BYTES;
          if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * F_STAGE_BYTES);
          tma_load_2d_pair(s0, &map_ahi, full_bar(stage), kb * F_BK, m0);
          tma_load_2d_pair(s0 + F_PLANE, &map_alo, full_bar(stage), kb * F_BK, m0);
          tma_load_2d_pair(s0 + 2 * F_PLANE, &map_bhi, full_bar(stage), kb * F_BK, n0);
          tma_load_2d_pair(s0 + 3 * F_PLANE, &map_blo, full_bar(stage), kb * F_BK, n0);
          if (++stage == F_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);   // let copies in flight land before the CTA retires
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      UnitIter it;
      int tile, kc;
      bool first;
      while (ok && next_unit(p, pair, num_pairs, it, tile, kc, first)) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 22)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * F_BN);
        const int kend = min(p.num_kb, kc + p.chunk_kb);
        for (int kb = kc; kb < kend; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 23)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t s0 = smem_base + stage * F_STAGE_BYTES;
          const uint64_t ahi = make_smem_desc_sw128(s0, 16u, 1024u);
          const uint64_t alo = make_smem_desc_sw128(s0 + F_PLANE, 16u, 1024u);
          const uint64_t bhi = make_smem_desc_sw128(s0 + 2 * F_PLANE, 16u, 1024u);
          const uint64_t blo = make_smem_desc_sw128(s0 + 3 * F_PLANE, 16u, 1024u);
#pragma unroll
          for (int j = 0; j < F_BK / 8; ++j) {   // one instruction consumes 8 floats = 32 bytes of K
            const uint64_t o = uint64_t(j * 2);  // descriptor start addresses count 16-byte units
            mma_tf32_ss_pair(d_tmem, alo + o, bhi + o, p.idesc, (kb != kc || j != 0) ? 1u : 0u);   // small terms first
            mma_tf32_ss_pair(d_tmem, ahi + o, blo + o, p.idesc, 1u);
            mma_tf32_ss_pair(d_tmem, ahi + o, bhi + o, p.idesc, 1u);
          }
          mma_commit_pair(empty_bar(stage));
          if (++stage == F_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit_pair(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;   // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t my_stage = epi_base + uint32_t(warp - 2) * 8192u;
    uint32_t nstore = 0;
    UnitIter it;
    int tile, kc;
    bool first;
    while (next_unit(p, pair, num_pairs, it, tile, kc, first)) {
      int tm, tn;
      tile_coords_f(tile, p.tiles_m, p.tiles_n, tm, tn);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 24)) break;
      tc_fence_after_sync();
      if (!p.splitk && !first) {
        // this warp's stores of the tile's previous chunk have been performed before the same elements are added to
        if (lane == 0) tma_store_wait_all<0>();
        __syncwarp();
      }
      epilogue_rows_f32(&map_c, p, tmem_base + uint32_t(acc * F_BN), q, lane, tm * 256 + int(cta_rank) * 128 + q * 32,
                        tn * F_BN, my_stage, nstore, p.splitk != 0 || p.accumulate != 0 || !first);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // no CTA of the pair retires while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, F_TMEM_COLS);
  }
}

}  // namespace

// Runs C (+)= A . B on the tensor cores when the shape qualifies.  Returns SIMP_OK when it ran, a negative error when
// a launch failed, and 1 when the shape does not qualify or scratch could not be had (the caller then takes the FFMA
// kernel).  a: [m, k]; b: [k, n] or, with b_transposed, [n, k]; c: [m, n]; all row-major and dense.
int gemm_f32_tc_run(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int accumulate,
                    int b_transposed) {
  if (m < 128 || n < 128 || k < 32 || n % 4 != 0 || (reinterpret_cast<uintptr_t>(c) & 15u) != 0) return 1;
  if (double(m) * double(n) * double(k) < double(int64_t(1) << 26)) return 1;   // too small to pay for the split pass
  if (m > 0x3fffffff || n > 0x3fffffff || k > 0x3fffffff) return 1;
  const int64_t kp = cdiv(k, F_BK) * F_BK;
  if (kp / 32 > 65535) return 1;   // grid limit of the transposing split
  const size_t a_plane = size_t(m) * size_t(kp) * 4, b_plane = size_t(n) * size_t(kp) * 4;
  if (2 * (a_plane + b_plane) > (size_t(8) << 30)) return 1;
  float* pa = static_cast<float*>(scratch(2 * a_plane, 13));
  float* pb = pa ? static_cast<float*>(scratch(2 * b_plane, 14)) : nullptr;
  if (!pa || !pb) return 1;
  float *a_hi = pa, *a_lo = pa + size_t(m) * kp, *b_hi = pb, *b_lo = pb + size_t(n) * kp;
  cudaStream_t st = ctx().stream;
  const int va = (k % 4 == 0 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0) ? 1 : 0;
  const int vb = (k % 4 == 0 && (reinterpret_cast<uintptr_t>(b) & 15u) == 0) ? 1 : 0;
  split_rows_kernel<<<dim3(unsigned(m), unsigned(cdiv(kp, 1024))), 256, 0, st>>>(a, m, k, k, a_hi, a_lo, kp, va);
  if (b_transposed)
    split_rows_kernel<<<dim3(unsigned(n), unsigned(cdiv(kp, 1024))), 256, 0, st>>>(b, n, k, k, b_hi, b_lo, kp, vb);
  else
    split_transpose_kernel<<<dim3(unsigned(cdiv(n, 32)), unsigned(kp / 32)), 256, 0, st>>>(b, k, n, b_hi, b_lo, kp);
  SIMP_LAUNCH_CHECK();

  CUtensorMap mahi, malo, mbhi, mblo, mc;
  if (int rc = make_map_f32(&mahi, a_hi, kp, m, 128, true)) return rc;
  if (int rc = make_map_f32(&malo, a_lo, kp, m, 128, true)) return rc;
  if (int rc = make_map_f32(&mbhi, b_hi, kp, n, 128, true)) return rc;
  if (int rc = make_map_f32(&mblo, b_lo, kp, n, 128, true)) return rc;
  if (int rc = make_map_f32(&mc, c, n, m, 32, false)) return rc;
  F32Params p{};
  p.M = int(m);
  p.N = int(n);
  p.tiles_m = int(cdiv(m, 256));
  p.tiles_n = int(cdiv(n, F_BN));
  p.num_kb = int(kp / F_BK);
  p.chunk_kb = F_CHUNK_KB;
  {
    // fewer tiles than CTA pairs (a few hundred rows times a long K): the chunks of a tile go to different pairs and
    // are all added into C; the order of those f32 adds is not fixed, so results may differ in the last bits from
    // run to run (within the tolerance of this path by orders of magnitude)
    const int64_t tiles0 = int64_t(p.tiles_m) * p.tiles_n;
    const int max_pairs0 = ctx().sm_count / 2;
    if (tiles0 * 2 <= max_pairs0 && p.num_kb >= 32) {
      const int want_chunks = int(cdiv(max_pairs0, tiles0));
      int ck = int(cdiv(p.num_kb, want_chunks));
      if (ck < 16) ck = 16;
      if (ck < p.num_kb) {
        p.chunk_kb = ck < F_CHUNK_KB ? ck : F_CHUNK_KB;
        p.splitk = 1;
        if (!accumulate) SIMP_CUDA(cudaMemsetAsync(c, 0, size_t(m) * size_t(n) * 4, st));
      }
    }
  }
  p.idesc = make_idesc_tf32(256, F_BN);
  p.accumulate = accumulate ? 1 : 0;
  p.status = ctx().dev_status;
  static bool attr_set = false;
  if (!attr_set) {
    SIMP_CUDA(cudaFuncSetAttribute(gemm_tf32x3_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(F_SMEM)));
    attr_set = true;
  }
  const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n * (p.splitk ? cdiv(p.num_kb, p.chunk_kb) : 1);
  const int max_pairs = ctx().sm_count / 2;
  const int pairs = int(tiles < max_pairs ? tiles : max_pairs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(2 * pairs));
  cfg.blockDim = dim3(F_THREADS);
  cfg.dynamicSmemBytes = F_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  SIMP_CUDA(cudaLaunchKernelEx(&cfg, gemm_tf32x3_2cta_kernel, mahi, malo, mbhi, mblo, mc, p));
  return SIMP_OK;
}

}  // namespace simp
