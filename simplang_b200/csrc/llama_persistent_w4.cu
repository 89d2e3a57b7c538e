// llama_persistent_w4.cu -- one token of the W4 LLaMA model (examples/llama2 W4 decode; weights
// dequantised as MatMulQuantOpLowering does, src/mlir/lowering/ConvertSimpToMemRef.cpp:3906-4005) as ONE
// persistent cooperative kernel: one block per SM, 16 compute warps + 1 producer warp, the phases of the
// forward pass separated by bounded grid barriers.
//
// A layer's 4-bit weights (~0.4 MB per SM for the 3B model) do not fit in shared memory, so they stream
// through a ring of three tile slots.  Every block owns a fixed, contiguous slice of the rows of each
// projection; the producer warp walks the block's tiles in program order -- across phases and layers -- and
// requests each one (cp.async.bulk: weight rows, their group scales, optional zeros; completion on the
// slot's `full` mbarrier) as soon as the compute warps have released the slot (`empty` mbarrier).  The grid
// barriers only gate the compute, never the weight stream, so HBM keeps streaming while a phase waits for
// its input vector and the ring is full when the phase starts.
//
// Compute: the activation vector is packed to 16-bit block floating point in shared memory (w4_pack_quarter,
// four threads per chunk), a tile is cut into slabs of 16 rows and the 16 warps are arranged as
// slabs x matrices x interleaved sets of 128-weight spans; each warp runs the tensor-core integer dot products of
// w4_mma_spans (exact integer accumulation per 32-weight chunk, see w4_core.cuh), partial sums of the span sets
// are added in set order.  The next rmsnorm is deferred exactly as in the per-op path:
// the packed vector holds x*w_norm and every dot product is scaled by 1/sqrt(mean(x^2)+eps).
// Per layer: q/k/v | attention | wo + residual | gate/up + silu*mul | down + residual; then the f32
// classifier streamed from HBM + greedy argmax.  Reduction orders are fixed: results are run-to-run identical.
#include "llama_persistent.cuh"
#include "llama_model.hpp"
#include "w4_core.cuh"

namespace simp {

constexpr int PW_SLOTS = 3;
constexpr int PW_MAX_TR = 32;   // rows per tile (per matrix) never exceed this
constexpr int PW_MAX_KS = 16;   // span sets per row never exceed this
constexpr size_t PW_STATIC_SMEM = 3072;

// Tile geometry of one phase kind.
struct PwKind {
  int cols, nchunks, row_bytes, gpr, log2_cpg;
  int sl, ms, kp;   // warps = sl slabs of 16 rows x ms matrices x kp interleaved span sets
  int tr;           // rows per tile and matrix (at most 16 * sl)
  int unit;         // row slices and tiles are multiples of `unit` rows (keeps every scale row block 16-byte aligned)
};

struct PersistW4Args {
  PkCommon c;
  const uint8_t* qw;
  const float* sc;
  const float* zr;        // nullptr: symmetric (zero = -8 * scale)
  long long off[7];       // element offsets of wq wk wv wo w1 w2 w3 (layer 0) in the arrays above
  int gs;
  PwKind ka;              // cols = dim, one matrix per tile (q, k, v, wo)
  PwKind kg;              // cols = dim, two matrices per tile (gate + up)
  PwKind kd;              // cols = hidden_dim (down)
  uint32_t slot_off[PW_SLOTS], xp_off, vec_off, part_off;
};

// One projection of a layer as the tile walk sees it.
struct PwSeg {
  int fam0, fam1;   // weight families (fam1 = -1: single matrix)
  int rows;         // output rows of the whole matrix
  int u0, nu;       // this block's slice, in units of K.unit rows
};

__device__ __forceinline__ const PwKind& pw_kind(const PersistW4Args& a, int s) { return s == 4 ? a.kg : (s == 5 ? a.kd : a.ka); }

__device__ __forceinline__ PwSeg pw_seg(const PersistW4Args& a, int s) {
  const PkCommon& c = a.c;
  PwSeg g;
  g.fam0 = s == 4 ? 4 : (s == 5 ? 5 : s);   // s: 0 wq, 1 wk, 2 wv, 3 wo, 4 w1 (+ w3), 5 w2
  g.fam1 = s == 4 ? 6 : -1;
  g.rows = (s == 1 || s == 2) ? c.kv : (s == 4 ? c.hd : c.dim);
  const int units = g.rows / pw_kind(a, s).unit;
  g.nu = share_rows(units, gridDim.x, blockIdx.x);
  g.u0 = share_row0(units, gridDim.x, blockIdx.x);
  return g;
}
// Tile i of a slice of nu units split into nt near-equal tiles: first unit and unit count.
__device__ __forceinline__ void pw_tile_range(int nu, int nt, int i, int& first, int& count) {
  const int base = nu / nt, rem = nu % nt;
  first = i * base + min(i, rem);
  count = base + (i < rem ? 1 : 0);
}

// Partial dot products of one tile: this warp's slab (and matrix) x its set of spans.
template <int NM>
__device__ __forceinline__ void pw_tile_partials(const uint8_t* slot, int tr_i, const PwKind& K, bool has_z,
                                                 const uint4* __restrict__ xp, float* __restrict__ partial) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slab = warp % K.sl, rest = warp / K.sl;
  const int msel = rest % K.ms, kpart = rest / K.ms;
  if (slab * 16 >= tr_i) return;
  W4Tile tl;
  tl.mat_w = size_t(tr_i) * K.row_bytes;
  tl.mat_s = size_t(tr_i) * K.gpr * 4;
  tl.mat_bytes = tl.mat_w + tl.mat_s * (has_z ? 2 : 1);
  tl.row_bytes = K.row_bytes;
  tl.sc_row = K.gpr;
  tl.has_z = has_z;
  tl.base = slot + (NM == 1 ? msel : 0) * tl.mat_bytes;
  float acc[NM][2];
#pragma unroll
  for (int m = 0; m < NM; ++m) acc[m][0] = acc[m][1] = 0.0f;
  w4_mma_spans<NM, false>(tl, slab * 16, tr_i, xp, K.nchunks, K.log2_cpg, kpart, K.kp, lane, acc);
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float v = acc[m][h];
      v += __shfl_xor_sync(0xffffffffu, v, 1);
      v += __shfl_xor_sync(0xffffffffu, v, 2);
      const int mm = NM == 1 ? msel : m;
      if ((lane & 3) == 0) partial[(mm * PW_MAX_TR + slab * 16 + (lane >> 2) + 8 * h) * PW_MAX_KS + kpart] = v;
    }
}

// Packs n32 chunks of a global vector (optionally times mul) into xp, four threads per chunk: two 16-byte loads
// through L2 per thread and operand.  Returns this thread's share of sum(x^2) of the unscaled input.
__device__ __forceinline__ float pw_pack_global(const float* __restrict__ x, const float* __restrict__ mul, uint8_t* xp,
                                                int n32) {
  float ss = 0.0f;
  for (int base = 0; base < n32 * 4; base += PK_THREADS) {
    const int q = base + int(threadIdx.x);
    const bool active = q < n32 * 4;
    float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (active) {
      const float4* src = reinterpret_cast<const float4*>(x + size_t(q) * 8);
      const float4 t0 = __ldcg(src), t1 = __ldcg(src + 1);
      v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
      if (mul) {
        const float4* ms = reinterpret_cast<const float4*>(mul + size_t(q) * 8);
        const float4 m0 = __ldg(ms), m1 = __ldg(ms + 1);
        v[0] *= m0.x; v[1] *= m0.y; v[2] *= m0.z; v[3] *= m0.w; v[4] *= m1.x; v[5] *= m1.y; v[6] *= m1.z; v[7] *= m1.w;
      }
    }
    w4_pack_quarter(v, active, q & 3, xp + size_t(q >> 2) * (W4_CHUNK_U4 * 16));
  }
  return ss;
}
__device__ __forceinline__ void pw_pack_shared(const float* vec, uint8_t* xp, int n32) {
  for (int base = 0; base < n32 * 4; base += PK_THREADS) {
    const int q = base + int(threadIdx.x);
    const bool active = q < n32 * 4;
    float v[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
    if (active) {
      const float4* src = reinterpret_cast<const float4*>(vec + size_t(q) * 8);
      const float4 t0 = src[0], t1 = src[1];
      v[0] = t0.x; v[1] = t0.y; v[2] = t0.z; v[3] = t0.w; v[4] = t1.x; v[5] = t1.y; v[6] = t1.z; v[7] = t1.w;
    }
    w4_pack_quarter(v, active, q & 3, xp + size_t(q >> 2) * (W4_CHUNK_U4 * 16));
  }
}

__global__ void __launch_bounds__(PK_BLOCK, 1) llama_w4_token_kernel(const PersistW4Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ PkStatic S;
  __shared__ __align__(8) uint64_t full[PW_SLOTS];    // the slot's tile has landed
  __shared__ __align__(8) uint64_t empty[PW_SLOTS];   // the compute warps are done with the slot
  const PkCommon& c = a.c;
  uint8_t* xp = smem + a.xp_off;                                   // packed activation vector
  float* vec = reinterpret_cast<float*>(smem + a.vec_off);         // f32 vector (attention output, classifier input)
  float* sm_acc = reinterpret_cast<float*>(xp);                    // attention scratch (xp is idle then)
  float* part = reinterpret_cast<float*>(smem + a.part_off);       // [2][NM][PW_MAX_TR][PW_MAX_KS] slice partials
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dim = c.dim, hd = c.hd;
  const bool has_z = a.zr != nullptr;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < PW_SLOTS; ++k) {
      ptx::mbar_init(ptx::smem_u32(&full[k]), 1);
      ptx::mbar_init(ptx::smem_u32(&empty[k]), 1);
    }
    S.sh_abort = 0;
    S.prod_done = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();

  // ================================================================== producer warp
  if (warp == PK_WARPS) {
    // A bulk-copy instruction holds its issuing thread for a few hundred nanoseconds whatever its size, so
    // a tile is requested by all 32 lanes at once: the weight rows of each matrix are cut into up to 24
    // pieces (lanes 0-23), scales and zeros go to lanes 24-27.  Lane 0 owns the barriers.
    uint32_t slot = 0, use = 0;
    uint32_t last_use[PW_SLOTS] = {0, 0, 0};
    uint32_t used = 0;                   // bit s: slot s has been requested at least once
    bool ok = true;
    for (int l = 0; l < c.n_layers && ok; ++l)
      for (int s = 0; s < 6 && ok; ++s) {
        const PwKind& K = pw_kind(a, s);
        const PwSeg g = pw_seg(a, s);
        if (g.nu == 0) continue;
        const int cap = K.tr / K.unit;
        const int nt = (g.nu + cap - 1) / cap;
        const int nm = g.fam1 >= 0 ? 2 : 1;
        for (int i = 0; i < nt && ok; ++i) {
          int first, count;
          pw_tile_range(g.nu, nt, i, first, count);
          const int tr_i = count * K.unit;
          const long long row = (long long)(g.u0 + first) * K.unit;
          const uint32_t bar = ptx::smem_u32(&full[slot]);
          const uint32_t mat_w = uint32_t(tr_i) * uint32_t(K.row_bytes), mat_s = uint32_t(tr_i) * uint32_t(K.gpr) * 4u;
          const uint32_t mat_bytes = mat_w + mat_s * (has_z ? 2u : 1u);
          if (lane == 0) {
            if (use > 0) ok = ptx::mbar_wait(ptx::smem_u32(&empty[slot]), (use - 1) & 1u, &S.sh_abort, c.status, 40 + int(slot));
            if (ok) ptx::mbar_arrive_expect_tx(bar, mat_bytes * uint32_t(nm));
          }
          ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
          if (!ok) break;
          if (lane < 24) {
            const int wl = 24 / nm;                 // lanes per matrix
            const int m = lane / wl, piece = lane - m * wl;
            const uint32_t psz = ((mat_w / 16 + wl - 1) / wl) * 16;
            const uint32_t off = uint32_t(piece) * psz;
            if (off < mat_w) {
              const long long o = a.off[m == 0 ? g.fam0 : g.fam1] + ((long long)l * g.rows + row) * K.cols;
              ptx::bulk_load(ptx::smem_u32(smem + a.slot_off[slot] + m * mat_bytes + off), a.qw + o / 2 + off,
                             min(psz, mat_w - off), bar);
            }
          } else if (lane < 28) {
            const int m = lane & 1, zsel = (lane - 24) >> 1;   // 24, 25: scales of matrix 0, 1; 26, 27: zeros
            if (m < nm && (zsel == 0 || has_z)) {
              const long long o = a.off[m == 0 ? g.fam0 : g.fam1] + ((long long)l * g.rows + row) * K.cols;
              const float* src = (zsel ? a.zr : a.sc) + o / a.gs;
              ptx::bulk_load(ptx::smem_u32(smem + a.slot_off[slot] + m * mat_bytes + mat_w + zsel * mat_s), src, mat_s, bar);
            }
          }
          last_use[slot] = use;
          used |= 1u << slot;
          if (++slot == PW_SLOTS) { slot = 0; ++use; }
        }
      }
    // Before this warp leaves, its last requests must have landed (they have, unless the kernel is being
    // abandoned; then the bounded wait keeps copies from arriving in shared memory that is no longer ours).
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < PW_SLOTS; ++k)
        if (used & (1u << k))
          for (int spin = 0; spin < 400000; ++spin)
            if (ptx::mbar_try_wait(ptx::smem_u32(&full[k]), last_use[k] & 1u)) break;
      *reinterpret_cast<volatile int*>(&S.prod_done) = 1;
    }
    return;
  }

  // ================================================================== compute warps
  unsigned epoch = 0;
  uint32_t slot = 0, use = 0, tcount = 0;
  // Error exit: raise the abort flag for the producer and give it a bounded time to see its copies land.
  auto drain = [&]() {
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(&S.sh_abort) = 1;
      for (int spin = 0; spin < 4000000 && *reinterpret_cast<volatile int*>(&S.prod_done) == 0; ++spin) {}
    }
    csync();
  };
  // All tiles of segment s of layer l: wait for the slot, slice partials, reduce the column slices in order,
  // epilogue, release the slot.  mode 0: out[row] = v*inv_r; 1: x[row] += v; 2: hb[row] = silu(g*inv_r) * (u*inv_r).
  auto run_segment = [&](int s, int mode, float* out, float inv_r) -> bool {
    const PwKind& K = pw_kind(a, s);
    const PwSeg g = pw_seg(a, s);
    if (g.nu == 0) return true;
    const int cap = K.tr / K.unit;
    const int nt = (g.nu + cap - 1) / cap;
    for (int i = 0; i < nt; ++i) {
      int first, count;
      pw_tile_range(g.nu, nt, i, first, count);
      const int tr_i = count * K.unit;
      const int row0 = (g.u0 + first) * K.unit;
      if (!ptx::mbar_wait(ptx::smem_u32(&full[slot]), use & 1u, &S.sh_abort, c.status, 50 + int(slot))) return false;
      const uint8_t* sl = smem + a.slot_off[slot];
      float* pbuf = part + (tcount & 1u) * (2 * PW_MAX_TR * PW_MAX_KS);
      const uint4* xq = reinterpret_cast<const uint4*>(xp);
      if (mode == 2 && K.ms == 1) pw_tile_partials<2>(sl, tr_i, K, has_z, xq, pbuf);
      else pw_tile_partials<1>(sl, tr_i, K, has_z, xq, pbuf);
      // residual rows are requested before the block-wide sync so their latency overlaps it
      const int r = threadIdx.x;
      const float resid = (mode == 1 && r < tr_i) ? __ldcg(c.x + row0 + r) : 0.0f;
      csync();
      if (threadIdx.x == 0) ptx::mbar_arrive(ptx::smem_u32(&empty[slot]));   // every warp has read the slot
      if (r < tr_i) {
        float v0 = 0.0f, v1 = 0.0f;
        for (int k = 0; k < K.kp; ++k) v0 += pbuf[r * PW_MAX_KS + k];
        if (mode == 2)
          for (int k = 0; k < K.kp; ++k) v1 += pbuf[(PW_MAX_TR + r) * PW_MAX_KS + k];
        if (mode == 0) out[row0 + r] = v0 * inv_r;
        if (mode == 1) c.x[row0 + r] = resid + v0;
        if (mode == 2) {
          const float gt = v0 * inv_r, up = v1 * inv_r;
          out[row0 + r] = (gt / (1.0f + expf(-gt))) * up;
        }
      }
      ++tcount;
      if (++slot == PW_SLOTS) { slot = 0; ++use; }
    }
    return true;
  };

  // ---- embedding: x = table[token] (each block copies a slice), then everyone may read x
  {
    const int64_t token = c.ctl[0];
    for (int i = blockIdx.x * PK_THREADS + threadIdx.x; i < dim; i += gridDim.x * PK_THREADS) c.x[i] = c.tok_emb[token * dim + i];
  }
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  const int pos = c.ctl[1];

  for (int l = 0; l < c.n_layers; ++l) {
    // ------------------------------------------------------------------ phase 0: q/k/v
    {
      const float ss = compute_sum(pw_pack_global(c.x, c.rms_att + size_t(l) * dim, xp, dim >> 5), S.red);
      const float inv_r = 1.0f / sqrtf(ss / float(dim) + 1e-5f);
      for (int s = 0; s < 3; ++s)
        if (!run_segment(s, 0, s == 0 ? c.q : (s == 1 ? c.k : c.v), inv_r)) { drain(); return; }
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 1: attention
    pk_attention(c, S, sm_acc, l, pos);
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    // ------------------------------------------------------------------ phase 2: wo + residual
    {
      pk_merge_heads(c, vec);
      csync();
      pw_pack_shared(vec, xp, dim >> 5);
      csync();
      if (!run_segment(3, 1, nullptr, 1.0f)) { drain(); return; }
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 3: gate / up, silu * mul
    {
      const float ss = compute_sum(pw_pack_global(c.x, c.rms_ffn + size_t(l) * dim, xp, dim >> 5), S.red);
      const float inv_r = 1.0f / sqrtf(ss / float(dim) + 1e-5f);
      if (!run_segment(4, 2, c.hb, inv_r)) { drain(); return; }
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 4: down + residual
    {
      pw_pack_global(c.hb, nullptr, xp, hd >> 5);
      csync();
      if (!run_segment(5, 1, nullptr, 1.0f)) { drain(); return; }
      if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    }
  }

  // ---------------------------------------------------------------------- classifier + argmax
  {
    const float r = stage_x_rms(c.x, vec, dim, S.red);
    finish_rmsnorm(vec, c.rms_final, r, dim);
  }
  pk_classifier(c, S, vec);
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  pk_advance(c, pos);
}

// ---------------------------------------------------------------------------------------------
struct PersistW4Plan {
  PwKind ka, kg, kd;
  uint32_t slot_off[PW_SLOTS], xp_off, vec_off, part_off;
  size_t total;
  bool ok;
};

static int gcd_i(int a, int b) { return b ? gcd_i(b, a % b) : a; }

// Tile size and warp arrangement for tiles of `nm` matrices with rows of `cols` weights: the largest tile of at
// most 32 rows (a multiple of the unit) that fits a slot; 16 warps = slabs x matrices x span sets.
static bool pw_pick(int cols, int gs, int nm, bool zeros, size_t slot_bytes, PwKind& K) {
  K = PwKind{};
  K.cols = cols;
  K.nchunks = cols / 32;
  K.row_bytes = cols / 2;
  K.gpr = cols / gs;
  K.log2_cpg = __builtin_ctz(unsigned(gs / 32));
  K.unit = 4 / gcd_i(4, K.gpr);
  const size_t row_b = size_t(K.row_bytes) + size_t(K.gpr) * 4 * (zeros ? 2 : 1);
  int tr = int(std::min<size_t>(PW_MAX_TR, slot_bytes / (size_t(nm) * row_b)));
  tr -= tr % K.unit;
  if (tr < K.unit || tr < 4) return false;
  K.tr = tr;
  K.sl = (tr + 15) / 16;
  K.ms = (nm == 2 && K.sl == 1) ? 2 : 1;
  K.kp = PK_WARPS / (K.sl * K.ms);
  return K.kp >= 1 && K.kp <= PW_MAX_KS;
}

static PersistW4Plan persist_w4_plan(const LlamaModel& m) {
  PersistW4Plan p{};
  const int dim = int(m.cfg.dim), hd = int(m.cfg.hidden_dim), kv = int(m.kv_dim), gs = int(m.cfg.group_size);
  auto al = [](size_t v) { return (v + 127) & ~size_t(127); };
  if (dim % 32 || hd % 32 || gs < 32 || (gs & (gs - 1)) || dim % gs || hd % gs) return p;
  const size_t xp_bytes = al(std::max<size_t>(w4_packed_bytes(std::max(dim, hd)), size_t(PK_WARPS) * 128 * 4));
  const size_t vec_bytes = al(size_t(dim) * 4);
  const size_t part_bytes = al(size_t(2) * 2 * PW_MAX_TR * PW_MAX_KS * 4);
  const size_t fixed = xp_bytes + vec_bytes + part_bytes + PW_STATIC_SMEM;
  if (fixed + PW_SLOTS * 4096 > PK_SMEM_LIMIT) return p;
  const size_t slot_bytes = ((PK_SMEM_LIMIT - fixed) / PW_SLOTS) & ~size_t(127);
  const bool zeros = m.zeros != nullptr;
  if (!pw_pick(dim, gs, 1, zeros, slot_bytes, p.ka) || !pw_pick(dim, gs, 2, zeros, slot_bytes, p.kg) ||
      !pw_pick(hd, gs, 1, zeros, slot_bytes, p.kd))
    return p;
  // every projection's row count must split into whole units
  if (dim % p.ka.unit || kv % p.ka.unit || hd % p.kg.unit || dim % p.kd.unit) return p;
  size_t off = 0;
  for (int s = 0; s < PW_SLOTS; ++s) { p.slot_off[s] = uint32_t(off); off += slot_bytes; }
  p.xp_off = uint32_t(off); off += xp_bytes;
  p.vec_off = uint32_t(off); off += vec_bytes;
  p.part_off = uint32_t(off); off += part_bytes;
  p.total = off;
  p.ok = true;
  return p;
}

bool persistent_w4_supported(const LlamaModel& m) {
  if (!m.cfg.w4 || !pk_device_ok(m) || !m.offsets_set) return false;
  // bulk copies need 16-byte aligned sources: array bases and every family offset
  if ((reinterpret_cast<uintptr_t>(m.qweights) & 15u) || (reinterpret_cast<uintptr_t>(m.scales) & 15u) ||
      (m.zeros && (reinterpret_cast<uintptr_t>(m.zeros) & 15u)))
    return false;
  for (int f = 0; f < 7; ++f)
    if (m.loff[f] % 32 || (m.loff[f] / m.cfg.group_size) % 4) return false;
  return persist_w4_plan(m).ok;
}

int enqueue_token_persistent_w4(LlamaModel& m, cudaStream_t st) {
  PersistW4Args a{};
  if (int rc = pk_fill_common(m, a.c)) return rc;
  const PersistW4Plan p = persist_w4_plan(m);
  SIMP_REQUIRE(p.ok, SIMP_ERR_UNSUPPORTED, "persistent W4 decode: model does not fit the shared-memory plan");
  a.qw = m.qweights; a.sc = m.scales; a.zr = m.zeros;
  for (int f = 0; f < 7; ++f) a.off[f] = m.loff[f];
  a.gs = int(m.cfg.group_size);
  a.ka = p.ka; a.kg = p.kg; a.kd = p.kd;
  for (int s = 0; s < PW_SLOTS; ++s) a.slot_off[s] = p.slot_off[s];
  a.xp_off = p.xp_off; a.vec_off = p.vec_off; a.part_off = p.part_off;
  if (!m.pk_attr_done) {   // first (eager) pass of this model, outside any stream capture
    SIMP_CUDA(cudaFuncSetAttribute(llama_w4_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PK_SMEM_LIMIT - PW_STATIC_SMEM)));
    m.pk_attr_done = true;
  }
  return pk_launch(reinterpret_cast<const void*>(llama_w4_token_kernel), &a, a.c.bar, p.total, st);
}

}  // namespace simp
