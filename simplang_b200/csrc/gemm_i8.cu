// gemm_i8.cu -- tensor_matmul on i8: C[M,N] (s32, wrap-around) = A[M,K] . B, bit-exact.
//
// Semantics: TensorMatMulOpLowering i8 branch (src/mlir/lowering/ConvertSimpToMemRef.cpp:3220-3247,
// sign-extend both, multiply, add in i32) and its VNNI rewrite (src/mlir/passes/VNNIPass.cpp:731-906);
// the unsigned-A form is raw vpdpbusd (simptensor/tests/test_vnni_correctness.cpp:28-42);
// B as [N,K] is tensor_matmul_nt (ConvertSimpToMemRef.cpp:3417-3443).
//
// Tensor-core kernel (persistent, warp-specialised, one CTA per SM):
//   warp 0      TMA producer: 128x128-byte A tile + 256x128-byte B tile per stage, 128-byte swizzle,
//               4-stage ring, mbarrier complete_tx
//   warp 1      issues tcgen05.mma.cta_group::1.kind::i8 (M128 x N256 x K32, s32 accumulators in
//               TMEM), 4 per stage; tcgen05.commit releases the stage / publishes the accumulator
//   warps 2..5  epilogue: tcgen05.ld 32x32b -> registers -> global, overlapped with the next
//               tile's main loop through two 256-column TMEM accumulators
// The unsigned/signed choice per operand is a bit of the instruction descriptor, so the u8 x s8
// and s8 x s8 products need neither the sign flip nor the 128*sum(B) correction of the CPU code.
// B given as [K,N] is consumed in place through an MN-major shared-memory descriptor: the
// transpose the CPU lowering performs (ConvertSimpToMemRef.cpp:3168-3216) does not exist here.
// Out-of-range parts of edge tiles are zero-filled by TMA and masked at the store.
// Shapes whose operand rows are not 16-byte multiples (a TMA requirement) run the dp4a kernel.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace simp {

using namespace ptx;

constexpr int BM = 128, BN = 256, BK = 128;  // BK in bytes == elements
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;            // 16 KB
constexpr int B_BYTES = BN * BK;            // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int EPI_BYTES = 4 * 2 * 4096;      // per epilogue warp: two 32x32 i32 staging tiles for TMA stores
constexpr size_t GEMM_SMEM = size_t(STAGES) * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

// The C buffers a tile is stored to when the all-gather is fused into the epilogue: m[self] is the tensor map of
// this rank's own copy (TMA store), c[r] the row-major [M, ldc] copies of the peers (plain stores over NVLink).
struct PeerMaps {
  CUtensorMap m[8];
  int32_t* c[8];
  int self, ldc;
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, num_kb;
  int b_mn_major;   // 1: B is [K,N] (N contiguous), 0: B is [N,K]
  uint32_t idesc;
  int32_t* C;
  int* status;
  int tma_store;    // 1: epilogue goes through shared memory + TMA stores (needs N % 4 == 0)
  uint32_t link_ns; // fused all-gather, 2-CTA kernel: time the link needs for everything this rank sends (0: no pacing)
  int n_peers;      // > 0: every C tile is written into n_peers buffers (own copy by TMA store, the peer GPUs' by plain
                    //      stores) at column col_offset
  int col_offset;
  int streamk;      // 1: the tiles x K-blocks work units are split evenly over the CTAs; partial tiles are
                    //    added into a zeroed C with TMA reduce-add (integer adds: exact in any order)
                    // 2: hybrid -- full waves as whole tiles, only the tiles of the last partial wave are split
  int bn;           // tile width in columns (multiple of 32, <= 256); the 2-CTA kernel always uses 256
  uint32_t stage_tx;  // bytes one stage's TMA loads deliver (1-CTA kernel)
  int mma_only;     // measurement aid (2-CTA kernel): no TMA loads, no epilogue traffic -- the MMA issuer runs
                    // over whatever the stages hold, which times the tensor pipe's issue ceiling for this tiling
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // groups of 16 row-tiles, column-major inside a group: one wave of CTAs touches a compact block
  constexpr int G = 16;
  const int per_group = G * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * G;
  const int gsz = min(G, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  tm = first_m + in_group % gsz;
  tn = in_group / gsz;
}


// Work of one CTA of the 1-CTA kernel.  Classic mode: whole tiles, tile = blockIdx.x + i*gridDim.x.
// Stream-K mode (streamk = 1): the num_tiles*num_kb (tile, K-block) units are cut into gridDim.x equal contiguous
// ranges, so every SM gets the same amount of math even when the tile count is not a multiple of the SM count.
// Hybrid mode (streamk = 2, more than one wave): the full waves run as whole tiles with plain stores, and only
// the tiles of the last, partial wave are cut into equal K ranges -- so only those few tiles pay for zeroing
// and reduce-adds.
struct WorkIter {
  int i = 0;          // whole tiles: iteration count
  int u = 0, u1 = 0;  // split part: next unit, end of this CTA's range
};
__device__ __forceinline__ int work_full_tiles(const GemmParams& p, int num_tiles) {
  return p.streamk == 2 ? (num_tiles / int(gridDim.x)) * int(gridDim.x) : (p.streamk == 1 ? 0 : num_tiles);
}
__device__ __forceinline__ void work_init(const GemmParams& p, int num_tiles, WorkIter& w) {
  if (p.streamk) {
    const long long total = (long long)(num_tiles - work_full_tiles(p, num_tiles)) * p.num_kb;
    w.u = int(total * blockIdx.x / gridDim.x);
    w.u1 = int(total * (blockIdx.x + 1) / gridDim.x);
  }
}
// Next work item: tile, K-block range, and whether the result is a partial sum to be reduce-added.
__device__ __forceinline__ bool work_next(const GemmParams& p, int num_tiles, WorkIter& w, int& tile, int& kb0, int& kb1,
                                          bool& partial) {
  const int full = work_full_tiles(p, num_tiles);
  tile = blockIdx.x + w.i * gridDim.x;
  if (tile < full) {
    ++w.i;
    kb0 = 0;
    kb1 = p.num_kb;
    partial = false;
    return true;
  }
  if (w.u >= w.u1) return false;
  const int t = w.u / p.num_kb;
  tile = full + t;
  kb0 = w.u - t * p.num_kb;
  kb1 = min(p.num_kb, kb0 + (w.u1 - w.u));
  w.u += kb1 - kb0;
  partial = true;
  return true;
}

// Zeroes the C region of the tiles [first, num_tiles) (the split tiles of the hybrid mode): one block per tile.
__global__ void zero_tiles_kernel(int32_t* __restrict__ C, int M, int N, int tiles_m, int tiles_n, int bn, int first) {
  int tm, tn;
  tile_coords(first + blockIdx.x, tiles_m, tiles_n, tm, tn);
  const int m0 = tm * 128, n0 = tn * bn;
  for (int r = threadIdx.x >> 5; r < 128; r += blockDim.x >> 5) {
    const int row = m0 + r;
    if (row >= M) break;
    for (int cidx = n0 + (threadIdx.x & 31); cidx < min(N, n0 + bn); cidx += 32) C[size_t(row) * N + cidx] = 0;
  }
}

// Epilogue of one 128 x 256 accumulator for the 32 rows owned by this warp: TMEM -> registers ->
// (a) 128-byte-swizzled shared-memory tile -> TMA store of full 128-byte lines, two tiles in flight, or
// (b) direct global stores when C's row pitch is not a 16-byte multiple.
// Returns after the last tcgen05.ld has completed (the accumulator may then be reused).
__device__ __forceinline__ void epilogue_rows(const CUtensorMap* tmap_c, const PeerMaps* peers, const GemmParams& p,
                                              uint32_t tmem_acc,
                                              int q, int lane, int row0, int n0, uint32_t stage_smem,
                                              uint32_t& nstore, bool partial = false, uint64_t* pace_next = nullptr,
                                              uint32_t pace_ns = 0) {
  const int row = row0 + lane;
  int32_t* crow = p.C + int64_t(row) * p.N + n0;
  const bool vec_ok = (p.N % 4) == 0;
#pragma unroll 1
  for (int ch = 0; ch < p.bn / 32; ++ch) {
    uint32_t r[32];
    const int c0 = n0 + ch * 32;
    if (p.tma_store) {
      if (lane == 0) tma_store_wait_read<1>();  // at most the previous store (other buffer) is still reading
      __syncwarp();
    }
    tmem_ld_32x32(tmem_acc + (uint32_t(q * 32) << 16) + uint32_t(ch * 32), r);
    tmem_ld_wait();
    if (p.tma_store) {
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
          if (p.n_peers > 0) {
            // fused all-gather, own copy: TMA store of the staged tile
            tma_store_2d(&peers->m[peers->self], buf, c0 + p.col_offset, row0);
          } else if (partial) {
            tma_reduce_add_2d(tmap_c, buf, c0, row0);
          } else {
            tma_store_2d(tmap_c, buf, c0, row0);
          }
          tma_store_commit();
        }
        if (p.n_peers > 1) {
          // fused all-gather, peers' copies: the warp reads the staged tile back (eight lanes per 128-byte row, four
          // rows per instruction) and stores whole 128-byte lines into every peer's C over NVLink.  Plain stores on
          // the load/store path: when the link pushes back only this epilogue warp waits -- TMA stores to peers sat
          // in the same queue as the operand loads of the main loop and stalled it (0.282 ms per step on 2 GPUs
          // where math and link each need 0.19).  Peers are visited from rank + 1 on, so that at any moment the
          // ranks target different destinations.
          const int prow = lane >> 3, pj = lane & 7;
          int4 v[8];
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + prow;
            const uint32_t addr = buf + uint32_t(r) * 128u + (uint32_t(pj ^ (r & 7)) << 4);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[it].x), "=r"(v[it].y), "=r"(v[it].z), "=r"(v[it].w) : "r"(addr));
          }
          if (pace_ns != 0) {
            // the warp's share of the link: this chunk's stores leave no earlier than the previous chunk's slot ended
            uint64_t now = globaltimer_ns();
            while (now < *pace_next) now = globaltimer_ns();   // bounded: the slot is never more than pace_ns ahead
            *pace_next = now + pace_ns;
          }
          for (int k = 1; k < p.n_peers; ++k) {
            int dst = peers->self + k;
            if (dst >= p.n_peers) dst -= p.n_peers;
            int32_t* cp = peers->c[dst] + int64_t(row0) * peers->ldc + c0 + p.col_offset + pj * 4;
#pragma unroll
            for (int it = 0; it < 8; ++it) {
              const int r = it * 4 + prow;
              if (row0 + r < p.M) *reinterpret_cast<int4*>(cp + int64_t(r) * peers->ldc) = v[it];
            }
          }
        }
      }
    } else if (row < p.M && c0 < p.N) {
      if (vec_ok && c0 + 32 <= p.N) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<int4*>(crow + ch * 32 + 4 * j) =
              make_int4(int(r[4 * j]), int(r[4 * j + 1]), int(r[4 * j + 2]), int(r[4 * j + 3]));
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < p.N) crow[ch * 32 + j] = int(r[j]);
      }
    }
  }
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_i8_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                           const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ PeerMaps peers,
                           const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + STAGES * STAGE_BYTES;
  const uint32_t bar_base = epi_base + EPI_BYTES;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tfull[2], tempty[2]; then tmem slot, abort flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  uint8_t* bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_generic + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * STAGES + 4) + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkIter wk;
      work_init(p, num_tiles, wk);
      int tile, kb0, kb1;
      bool partial;
      while (ok && work_next(p, num_tiles, wk, tile, kb0, kb1, partial)) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * p.bn;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          mbar_arrive_expect_tx(full_bar(stage), p.stage_tx);
          tma_load_2d(sa, &tmap_a, full_bar(stage), kb * BK, m0);
          if (p.b_mn_major) {
            tma_load_2d(sb, &tmap_b, full_bar(stage), n0, kb * BK);
            if (p.bn > 128) tma_load_2d(sb + B_BYTES / 2, &tmap_b, full_bar(stage), n0 + 128, kb * BK);
          } else {
            tma_load_2d(sb, &tmap_b, full_bar(stage), kb * BK, n0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // let copies already in flight land before the CTA retires (bounded)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t b_lbo = p.b_mn_major ? uint32_t(B_BYTES / 2) : 16u;
      const uint32_t b_kstep = p.b_mn_major ? (32u * 128u) >> 4 : 32u >> 4;  // descriptor units of 16 B
      WorkIter wk;
      work_init(p, num_tiles, wk);
      int tile, kb0, kb1;
      bool partial;
      while (ok && work_next(p, num_tiles, wk, tile, kb0, kb1, partial)) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 3)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint64_t a_desc = make_smem_desc_sw128(sa, 16u, 1024u);
          const uint64_t b_desc = make_smem_desc_sw128(sb, b_lbo, 1024u);
#pragma unroll
          for (int j = 0; j < BK / 32; ++j) {
            mma_i8_ss(d_tmem, a_desc + uint64_t(j * 2), b_desc + uint64_t(j) * b_kstep, p.idesc,
                      (kb != kb0 || j != 0) ? 1u : 0u);
          }
          mma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t my_stage = epi_base + uint32_t(warp - 2) * 8192u;
    uint32_t nstore = 0;
    WorkIter wk;
    work_init(p, num_tiles, wk);
    int tile, kb0, kb1;
    bool partial;
    while (work_next(p, num_tiles, wk, tile, kb0, kb1, partial)) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 4)) break;
      tc_fence_after_sync();
      epilogue_rows(&tmap_c, &peers, p, tmem_base + uint32_t(acc * BN), q, lane, tm * BM + q * 32, tn * p.bn, my_stage,
                    nstore, partial);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.tma_store && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// 2-CTA variant (cta_group::2): a pair of CTAs on neighbouring SMs owns one 256x256 tile.  Each CTA
// loads its own 128 rows of A and its own 128 columns of B (no multicast; the tensor cores read the
// peer's half of B over the cluster's shared-memory network), so a stage is 32 KB instead of 48 KB:
// one third less L2->SM traffic per MAC and six stages of look-ahead instead of four.  The even CTA
// issues tcgen05.mma.cta_group::2 (M = 256 across the pair); its commits are multicast to the
// barriers of both CTAs.  Both CTAs run a TMA producer and four epilogue warps.
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = 128 * BK, P_B_BYTES = 128 * BK;
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
// Rate at which plain stores issued by the SMs fill the peers' memory over NVLink on this machine, in bytes per
// nanosecond: between two GPUs a store kernel alone reaches 675-680 GB/s whatever the store shape (copy engines 740),
// and the fused GEMM is fastest paced at 700 (690: +1 %, 720: +4 %, 740 and more: as slow as unpaced, +12 %); with
// four GPUs the best pace is 650.
constexpr double PEER_STORE_GBS_PAIR = 700.0, PEER_STORE_GBS_SWITCHED = 650.0;
constexpr double KB_NS = 383.0;   // one 256 x 256 x 128 K-block of the 2-CTA main loop at full speed (24.5 us per 8192-deep tile)
constexpr size_t GEMM2_SMEM = size_t(P_STAGES) * P_STAGE_BYTES + EPI_BYTES + 1024 + 256;

#ifdef SIMP_W4_TRACE
// instrumented builds: [CTA pair][tile of the pair][accumulator free, last MMA issued, accumulator complete, tile stored]
__device__ unsigned long long g_gemm_trace[74 * 16 * 4];
#define GEMM_MARK(it, k) do { if (pair < 74 && (it) < 16) g_gemm_trace[(pair * 16 + (it)) * 4 + (k)] = globaltimer_ns(); } while (0)
#else
#define GEMM_MARK(it, k) do { } while (0)
#endif

__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_i8_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                                const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ PeerMaps peers,
                           const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + P_STAGES * P_STAGE_BYTES;
  const uint32_t bar_base = epi_base + EPI_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (P_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * P_STAGES + 2 + a); };
  uint8_t* bar_generic = smem_raw + (bar_base - smem_u32(smem_raw));
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_generic + 8 * (2 * P_STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_generic + 8 * (2 * P_STAGES + 4) + 8);

  if (p.n_peers > 0) pdl_launch_dependents();  // the rendezvous kernel may become resident; its wait covers this grid
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0: even CTA (issues MMAs), 1: odd CTA
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;  // 256 x 256 tiles

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // 4 epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Fused all-gather form: launched as a programmatic dependent of the rendezvous that closes the previous step, so
  // everything above ran while that step drained; nothing below touches global memory before the wait returns.
  if (p.n_peers > 0) pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && !p.mma_only) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * 256 + int(cta_rank) * 128, n0 = tn * 256 + int(cta_rank) * 128;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 11)) { ok = false; break; }
          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          const uint32_t sb = sa + P_A_BYTES;
          if (cta_rank == 0) mbar_arrive_expect_tx(full_bar(stage), 2 * P_STAGE_BYTES);
          tma_load_2d_pair(sa, &tmap_a, full_bar(stage), kb * BK, m0);
          if (p.b_mn_major) tma_load_2d_pair(sb, &tmap_b, full_bar(stage), n0, kb * BK);
          else tma_load_2d_pair(sb, &tmap_b, full_bar(stage), kb * BK, n0);
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok)
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t b_kstep = p.b_mn_major ? (32u * 128u) >> 4 : 32u >> 4;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 12)) { ok = false; break; }
        tc_fence_after_sync();
        GEMM_MARK((tile - pair) / num_pairs, 0);
        const uint32_t d_tmem = tmem_base + uint32_t(acc * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!p.mma_only && !mbar_wait(full_bar(stage), phase, abort_flag, p.status, 13)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_base + stage * P_STAGE_BYTES;
          const uint32_t sb = sa + P_A_BYTES;
          const uint64_t a_desc = make_smem_desc_sw128(sa, 16u, 1024u);
          const uint64_t b_desc = make_smem_desc_sw128(sb, 16u, 1024u);
#pragma unroll
          for (int j = 0; j < BK / 32; ++j)
            mma_i8_ss_pair(d_tmem, a_desc + uint64_t(j * 2), b_desc + uint64_t(j) * b_kstep, p.idesc,
                           (kb | j) != 0 ? 1u : 0u);
          mma_commit_pair(empty_bar(stage));
          if (++stage == P_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        mma_commit_pair(tfull_bar(acc));
        GEMM_MARK((tile - pair) / num_pairs, 1);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t my_stage = epi_base + uint32_t(warp - 2) * 8192u;
    uint32_t nstore = 0;
    uint64_t pace_next = 0;
    uint32_t pace_ns = 0;
    {
      // Pacing of the stores to the peers: the link carries everything this rank sends in link_ns; a pair that owns
      // n tiles spreads its 8 * n chunks per warp evenly over that time, so that all pairs finish together and the
      // stores never queue up in front of the operand loads (unpaced, a wave of finished tiles floods the path to
      // the link and the main loops behind it run up to 1.8x longer).
      const int my_tiles = (num_tiles - pair + num_pairs - 1) / num_pairs;
      if (p.link_ns != 0 && my_tiles > 0) pace_ns = p.link_ns / uint32_t(my_tiles * (BN / 32));
    }
    for (int tile = pair; tile < num_tiles; tile += num_pairs) {
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 14)) break;
      tc_fence_after_sync();
#ifdef SIMP_W4_TRACE
      const bool marker = warp == 2 && lane == 0 && cta_rank == 0;
      if (marker) GEMM_MARK((tile - pair) / num_pairs, 2);
#endif
      if (!p.mma_only)
        epilogue_rows(&tmap_c, &peers, p, tmem_base + uint32_t(acc * BN), q, lane,
                      tm * 256 + int(cta_rank) * 128 + q * 32, tn * BN, my_stage, nstore, false, &pace_next, pace_ns);
      tc_fence_before_sync();
      __syncwarp();
#ifdef SIMP_W4_TRACE
      if (marker) GEMM_MARK((tile - pair) / num_pairs, 3);
#endif
      if (lane == 0) mbar_arrive_even_cta(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (p.tma_store && lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // no CTA of the pair retires while the other may still signal or read it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// Integer dot-product kernel for shapes TMA cannot address (operand rows not 16-byte multiples)
// and for tiny problems.  64x64 tile, K step 32, dp4a with per-operand signedness.
template <bool A_UNSIGNED>
__global__ void __launch_bounds__(256) gemm_i8_dp4a_kernel(const uint8_t* __restrict__ A, const int8_t* __restrict__ B,
                                                           int32_t* __restrict__ C, int64_t M, int64_t K, int64_t N,
                                                           int b_t) {
  __shared__ uint32_t As[64][9];
  __shared__ uint32_t Bs[64][9];
  uint8_t* As8 = reinterpret_cast<uint8_t*>(&As[0][0]);
  uint8_t* Bs8 = reinterpret_cast<uint8_t*>(&Bs[0][0]);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int64_t m0 = int64_t(blockIdx.y) * 64, n0 = int64_t(blockIdx.x) * 64;
  int32_t acc[4][4] = {};
  for (int64_t p0 = 0; p0 < K; p0 += 32) {
    for (int e = threadIdx.x; e < 64 * 32; e += 256) {
      {
        const int r = e >> 5, c = e & 31;
        const int64_t gi = m0 + r, gp = p0 + c;
        As8[r * 36 + c] = (gi < M && gp < K) ? A[gi * K + gp] : uint8_t(0);
      }
      if (b_t) {
        const int r = e >> 5, c = e & 31;
        const int64_t gj = n0 + r, gp = p0 + c;
        Bs8[r * 36 + c] = (gj < N && gp < K) ? uint8_t(B[gj * K + gp]) : uint8_t(0);
      } else {
        const int c = e >> 6, r = e & 63;
        const int64_t gj = n0 + r, gp = p0 + c;
        Bs8[r * 36 + c] = (gj < N && gp < K) ? uint8_t(B[gp * N + gj]) : uint8_t(0);
      }
    }
    __syncthreads();
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      uint32_t a[4], b[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        a[u] = As[ty * 4 + u][w];
        b[u] = Bs[tx * 4 + u][w];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          if (A_UNSIGNED)
            asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(acc[u][v]) : "r"(a[u]), "r"(b[v]));
          else
            asm("dp4a.s32.s32 %0, %1, %2, %0;" : "+r"(acc[u][v]) : "r"(a[u]), "r"(b[v]));
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int u = 0; u < 4; ++u)
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int64_t gi = m0 + ty * 4 + u, gj = n0 + tx * 4 + v;
      if (gi < M && gj < N) C[gi * N + gj] = acc[u][v];
    }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// Encoded tensor maps are kept per (kind, address, extents, box): a map depends on nothing else, an encode costs
// about a microsecond, and a small GEMM (1024^3 is 6 us of device time) makes three per call.
struct MapKey {
  int kind;
  const void* base;
  int64_t inner, outer;
  int box_inner, box_outer;
  bool operator==(const MapKey& o) const {
    return kind == o.kind && base == o.base && inner == o.inner && outer == o.outer && box_inner == o.box_inner && box_outer == o.box_outer;
  }
};
struct MapCache {
  static constexpr int N = 32;
  MapKey key[N];
  CUtensorMap map[N];
  int used = 0, next = 0;
  std::mutex mu;
};
static MapCache g_maps;
static bool map_lookup(const MapKey& k, CUtensorMap* out) {
  std::lock_guard<std::mutex> lk(g_maps.mu);
  for (int i = 0; i < g_maps.used; ++i)
    if (g_maps.key[i] == k) {
      *out = g_maps.map[i];
      return true;
    }
  return false;
}
static void map_insert(const MapKey& k, const CUtensorMap& m) {
  std::lock_guard<std::mutex> lk(g_maps.mu);
  const int slot = g_maps.used < MapCache::N ? g_maps.used++ : (g_maps.next++ % MapCache::N);
  g_maps.key[slot] = k;
  g_maps.map[slot] = m;
}

// 2-D u8 tensor map: `inner` contiguous bytes per row, `outer` rows, 128-byte swizzle.
// 2-D i32 tensor map for C stores: 32 x 32 boxes (128-byte rows), 128-byte swizzle.
static int make_map_c_i32(CUtensorMap* map, const void* base, int64_t n, int64_t m) {
  const MapKey key{1, base, n, m, 32, 32};
  if (map_lookup(key, map)) return SIMP_OK;
  EncodeTiledFn enc = get_encode_fn();
  SIMP_REQUIRE(enc != nullptr, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(n), cuuint64_t(m)};
  cuuint64_t strides[1] = {cuuint64_t(n) * 4};
  cuuint32_t box[2] = {32, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SIMP_REQUIRE(r == CUDA_SUCCESS, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled (C) failed with CUresult %d", int(r));
  map_insert(key, *map);
  return SIMP_OK;
}

static int make_map_u8(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int box_inner,
                       int box_outer) {
  const MapKey key{0, base, inner, outer, box_inner, box_outer};
  if (map_lookup(key, map)) return SIMP_OK;
  EncodeTiledFn enc = get_encode_fn();
  SIMP_REQUIRE(enc != nullptr, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(inner), cuuint64_t(outer)};
  cuuint64_t strides[1] = {cuuint64_t(inner)};
  cuuint32_t box[2] = {cuuint32_t(box_inner), cuuint32_t(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SIMP_REQUIRE(r == CUDA_SUCCESS, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  map_insert(key, *map);
  return SIMP_OK;
}

// 2-D f32 tensor maps for the tensor-core f32 GEMM (gemm_f32_tc.cu): operand planes [outer, inner] with boxes of
// 32 floats (128 bytes) x box_outer rows, and C with 32 x 32 boxes; 128-byte swizzle.
int make_map_f32(CUtensorMap* map, const void* base, int64_t inner, int64_t outer, int box_outer, bool operand) {
  const MapKey key{operand ? 2 : 3, base, inner, outer, 32, box_outer};
  if (map_lookup(key, map)) return SIMP_OK;
  EncodeTiledFn enc = get_encode_fn();
  SIMP_REQUIRE(enc != nullptr, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(inner), cuuint64_t(outer)};
  cuuint64_t strides[1] = {cuuint64_t(inner) * 4};
  cuuint32_t box[2] = {32, cuuint32_t(box_outer)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   operand ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SIMP_REQUIRE(r == CUDA_SUCCESS, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled (f32) failed with CUresult %d", int(r));
  map_insert(key, *map);
  return SIMP_OK;
}

}  // namespace simp

namespace simp {
// Shared by simp_gpu_matmul_i8 (n_peers == 0: C is [M,N] in this GPU's memory) and the fused N-sharded GEMM
// (n_peers > 0: peer_c[r] are the row-major [M, ldc] copies of the full result on every rank, peer_c[self_rank]
// this rank's own; this rank's column block starts at col_offset).
int gemm_i8_run(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N, int a_unsigned,
                int b_transposed, int32_t* const* peer_c, int n_peers, int64_t ldc, int64_t col_offset, int self_rank) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(M >= 0 && K >= 0 && N >= 0, SIMP_ERR_ARG, "matmul_i8: negative size");
  if (M == 0 || N == 0) return SIMP_OK;
  SIMP_REQUIRE(A && B && (C || n_peers > 0), SIMP_ERR_ARG, "matmul_i8: null pointer");
  SIMP_REQUIRE(n_peers >= 0 && n_peers <= 8, SIMP_ERR_ARG, "matmul_i8: at most 8 peers");
  SIMP_REQUIRE(M <= 0x7fffffff && N <= 0x7fffffff && K <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_i8: dimension too large");
  cudaStream_t st = ctx().stream;
  if (K == 0) {
    SIMP_REQUIRE(n_peers == 0, SIMP_ERR_SHAPE, "matmul_i8: K == 0 is not supported by the fused all-gather form");
    SIMP_CUDA(cudaMemsetAsync(C, 0, size_t(M) * size_t(N) * sizeof(int32_t), st));
    return SIMP_OK;
  }
  const bool a16 = (reinterpret_cast<uintptr_t>(A) & 15u) == 0, b16 = (reinterpret_cast<uintptr_t>(B) & 15u) == 0;
  const bool tma_ok = a16 && b16 && (K % 16 == 0) && (b_transposed ? true : (N % 16 == 0)) &&
                      ((reinterpret_cast<uintptr_t>(C) & 15u) == 0);
  if (n_peers > 0)
    // The epilogue stores whole 32-column boxes at col_offset + c0 into the [M, ldc] maps of every rank, which are
    // clipped at ldc only: a column block that is not a multiple of 32 would spill zero columns into the next
    // rank's block.
    SIMP_REQUIRE(tma_ok && N % 32 == 0 && ldc % 4 == 0 && col_offset % 4 == 0 && col_offset + N <= ldc, SIMP_ERR_SHAPE,
                 "matmul_i8: the fused all-gather form needs 16-byte aligned operands, K %% 16 == 0 and column "
                 "blocks that are multiples of 32 columns");
  // The tensor-core kernel pays a fixed pipeline fill per tile; tiny problems stay on dp4a.
  const bool tiny = n_peers == 0 && M * N * K < int64_t(64) * 64 * 64;
  if (tma_ok && !tiny) {
    // Kernel choice (SIMP_GEMM_I8_KERNEL=1cta|2cta overrides it, for the tests): the 2-CTA kernel when 256x256 tiles fill its waves well (at least one wave on the 74 CTA
    // pairs and a last wave that is not nearly empty: 76 tiles would take two waves for 1.03 waves of work);
    // otherwise the 1-CTA kernel, whose hybrid stream-K mode spreads a partial last wave over all SMs.
    const int64_t tiles2 = cdiv(M, 256) * cdiv(N, 256);
    const int64_t pairs_all = ctx().sm_count / 2;
    const double eff2 = pairs_all > 0 ? double(tiles2) / double(cdiv(tiles2, pairs_all) * pairs_all) : 0.0;
    bool use_pair = tiles2 >= pairs_all && ctx().sm_count >= 2 && eff2 >= 0.8;
    if (const char* env = getenv("SIMP_GEMM_I8_KERNEL")) {
      if (!strcmp(env, "1cta")) use_pair = false;
      if (!strcmp(env, "2cta")) use_pair = true;
    }
    CUtensorMap ma, mb;
    if (int rc = make_map_u8(&ma, A, K, M, BK, 128)) return rc;
    if (b_transposed) {
      if (int rc = make_map_u8(&mb, B, K, N, BK, use_pair ? 128 : BN)) return rc;
    } else {
      if (int rc = make_map_u8(&mb, B, N, K, 128, BK)) return rc;
    }
    GemmParams p{};
    p.M = int(M); p.N = int(N); p.K = int(K);
    p.num_kb = int(cdiv(K, BK));
    p.b_mn_major = b_transposed ? 0 : 1;
    p.C = C;
    p.status = ctx().dev_status;
    p.tma_store = (N % 4 == 0) ? 1 : 0;
    CUtensorMap mc = ma;  // placeholder when unused
    PeerMaps peers;
    for (auto& pm : peers.m) pm = ma;
    p.n_peers = n_peers;
    p.col_offset = int(col_offset);
    // SIMP_GEMM_I8_ABLATE=mma: timing aid, the result is NOT computed (see GemmParams::mma_only).
    p.mma_only = 0;
    if (const char* env = getenv("SIMP_GEMM_I8_ABLATE"))
      if (!strcmp(env, "mma") && n_peers == 0) p.mma_only = 1;
    for (auto& pc : peers.c) pc = nullptr;
    peers.self = 0;
    peers.ldc = int(ldc);
    if (n_peers > 0) {
      p.tma_store = 1;
      SIMP_REQUIRE(self_rank >= 0 && self_rank < n_peers, SIMP_ERR_ARG, "matmul_i8: bad rank %d of %d", self_rank, n_peers);
      peers.self = self_rank;
      for (int r = 0; r < n_peers; ++r) {
        SIMP_REQUIRE(peer_c[r] != nullptr && (reinterpret_cast<uintptr_t>(peer_c[r]) & 15u) == 0, SIMP_ERR_ARG,
                     "matmul_i8: peer C pointer %d is null or misaligned", r);
        peers.c[r] = peer_c[r];
      }
      if (int rc = make_map_c_i32(&peers.m[self_rank], peer_c[self_rank], ldc, M)) return rc;
    } else if (p.tma_store) {
      if (int rc = make_map_c_i32(&mc, C, N, M)) return rc;
    }
    if (use_pair) {
      p.bn = BN;
      p.stage_tx = 0;
      p.streamk = 0;
      p.tiles_m = int(cdiv(M, 256)); p.tiles_n = int(cdiv(N, BN));
      p.idesc = make_idesc_i8(256, BN, /*a_signed=*/!a_unsigned, /*b_signed=*/true, false, !b_transposed);
      static bool attr2_set = false;
      if (!attr2_set) {
        SIMP_CUDA(cudaFuncSetAttribute(gemm_i8_tcgen05_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(GEMM2_SMEM)));
        attr2_set = true;
      }
      const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
      SIMP_REQUIRE(tiles <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_i8: too many tiles");
      const int max_pairs = ctx().sm_count / 2;
      const int pairs = int(tiles < max_pairs ? tiles : max_pairs);
      p.link_ns = 0;
      if (n_peers > 1) {
        // SIMP_PEER_STORE_GBS overrides the measured rate of this machine (0 switches pacing off)
        double gbs = n_peers == 2 ? PEER_STORE_GBS_PAIR : PEER_STORE_GBS_SWITCHED;
        if (const char* env = getenv("SIMP_PEER_STORE_GBS")) gbs = atof(env);
        const double ns = gbs > 0 ? double(M) * double(N) * 4.0 * (n_peers - 1) / gbs : 0.0;
        // Pacing protects the main loops from the flood of stores.  Where the link needs much longer than the math
        // (8192^3 on 4 ranks: 3x) the main loops have slack and the unpaced epilogue keeps the link as busy (354 us
        // either way), so pacing is used only up to a ratio of 2.5 (16384^3 on 4 ranks, 1.8x: 1402 -> 1316 us).
        const double math_ns = double(cdiv(tiles, pairs)) * double(p.num_kb) * KB_NS;
        p.link_ns = (ns > 0 && ns < 4.0e9 && ns < 2.5 * math_ns) ? uint32_t(ns) : 0u;
      }
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(unsigned(2 * pairs));
      cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = GEMM2_SMEM;
      cfg.stream = st;
      cudaLaunchAttribute at[2];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2;
      at[0].val.clusterDim.y = 1;
      at[0].val.clusterDim.z = 1;
      // fused all-gather form: the prologue (barriers, TMEM, tensor-map fetch) runs while the previous kernel on the
      // stream -- the rendezvous of the previous step -- is still waiting for the peers
      at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      at[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = at;
      cfg.numAttrs = n_peers > 0 ? 2 : 1;
      SIMP_CUDA(cudaLaunchKernelEx(&cfg, gemm_i8_tcgen05_2cta_kernel, ma, mb, mc, peers, p));
      return SIMP_OK;
    }
    // Tile width.  Measured on B200: a kind::i8 MMA of M = 128 takes the same ~128 clocks for every N <= 256
    // (the array is 256 columns wide and narrower tiles leave it idle), so narrower tiles never pay back in
    // math time; the width only shrinks for matrices narrower than one tile, to avoid loading padding.
    int bn = BN;
    {
      if (N < BN) bn = int(cdiv(N, 32) * 32);
      // Small problems (too little work for the K split to pay: measured 11.4 us split vs 8.2 whole at 1024^3) that
      // fill less than half of the SMs with 256-wide tiles: narrower tiles put more SMs to work and halve the
      // epilogue per CTA (1024^3: 8.2 us at 256, 6.9 at 128, 6.4 at 64).
      const int64_t tm1 = cdiv(M, BM);
      if (n_peers == 0 && M > 256 && tm1 * cdiv(N, BN) * cdiv(K, BK) < int64_t(ctx().sm_count) * 4)
        while (bn > 64 && tm1 * cdiv(N, bn) * 2 <= ctx().sm_count) bn >>= 1;
    }
    if (b_transposed) {  // the K-major B box height follows the tile width
      if (int rc = make_map_u8(&mb, B, K, N, BK, bn)) return rc;
    }
    p.bn = bn;
    p.stage_tx = uint32_t(A_BYTES + (b_transposed ? bn * BK : (bn > 128 ? 2 : 1) * 128 * BK));
    p.tiles_m = int(cdiv(M, BM)); p.tiles_n = int(cdiv(N, bn));
    p.idesc = make_idesc_i8(BM, bn, /*a_signed=*/!a_unsigned, /*b_signed=*/true, false, !b_transposed);
    static bool attr_set = false;
    if (!attr_set) {
      SIMP_CUDA(cudaFuncSetAttribute(gemm_i8_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     int(GEMM_SMEM)));
      attr_set = true;
    }
    const int64_t tiles = int64_t(p.tiles_m) * p.tiles_n;
    SIMP_REQUIRE(tiles <= 0x7fffffff, SIMP_ERR_SHAPE, "matmul_i8: too many tiles");
    int grid = int(tiles < ctx().sm_count ? tiles : ctx().sm_count);
    // Stream-K when whole tiles would leave a large part of the last wave idle (e.g. 152 or 52 tiles on 148
    // SMs): every CTA then gets the same number of K-blocks; C is zeroed and partial tiles are reduce-added.
    p.streamk = 0;
    {
      const int sms = ctx().sm_count;
      const int64_t waves = cdiv(tiles, sms);
      const double eff = double(tiles) / double(waves * sms);
      // Skinny problems (M <= 256: one or two row tiles, prefill of a few tokens) are weight-bandwidth bound and
      // have few tiles; splitting K over all SMs is what lets every SM stream a share of B, and the partial
      // tiles that are reduce-added hold only M rows.
      const bool enough = tiles * p.num_kb >= int64_t(sms) * 4 || (M <= 256 && tiles * p.num_kb >= sms / 2);
      bool want = p.tma_store && n_peers == 0 && eff < 0.85 && enough && waves <= 8;
      if (const char* env = getenv("SIMP_GEMM_I8_STREAMK")) want = p.tma_store && n_peers == 0 && atoi(env) != 0;
      // (waves <= 8 above: with many waves the last one matters little; SIMP_GEMM_I8_STREAMK=1 forces the split anyway)
      if (want) {
        grid = sms;
        if (tiles > sms) {   // more than one wave: only the last, partial wave is split and needs zeroing
          p.streamk = 2;
          const int full = int(tiles / sms) * sms;
          zero_tiles_kernel<<<int(tiles) - full, 256, 0, st>>>(C, int(M), int(N), p.tiles_m, p.tiles_n, bn, full);
        } else {
          p.streamk = 1;
          SIMP_CUDA(cudaMemsetAsync(C, 0, size_t(M) * size_t(N) * sizeof(int32_t), st));
        }
      }
    }
    gemm_i8_tcgen05_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, st>>>(ma, mb, mc, peers, p);
  } else {
    const int64_t gx = cdiv(N, 64), gy = cdiv(M, 64);
    SIMP_REQUIRE(gy <= 65535, SIMP_ERR_SHAPE, "matmul_i8: M too large for the dp4a kernel");
    dim3 grid{unsigned(gx), unsigned(gy)};
    if (a_unsigned)
      gemm_i8_dp4a_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(A), B, C, M, K, N, b_transposed);
    else
      gemm_i8_dp4a_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(A), B, C, M, K, N, b_transposed);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
}  // namespace simp

SIMP_API int simp_gpu_matmul_i8(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N,
                                int a_unsigned, int b_transposed) {
  return simp::gemm_i8_run(A, B, C, M, K, N, a_unsigned, b_transposed, nullptr, 0, N, 0, 0);
}

#ifdef SIMP_W4_TRACE
// Instrumented builds: the per-tile time marks of the last 2-CTA GEMM launch (74 pairs x 16 tiles x 4 marks).
SIMP_API int simp_debug_gemm_trace(unsigned long long* host_out) {
  SIMP_CUDA(cudaMemcpyFromSymbol(host_out, simp::g_gemm_trace, sizeof(unsigned long long) * 74 * 16 * 4));
  return SIMP_OK;
}
#endif
