// llama_i8_persistent.cu -- one token of the int8 LLaMA-3.2-1B-style model
// (examples/llama2/llama32_1b_int8_tensor.sl:16-305) as ONE persistent cooperative kernel: one block per SM,
// 16 compute warps + 1 producer warp, the phases of the forward pass separated by bounded grid barriers.
//
// Every block owns a fixed, contiguous slice of the rows of each projection.  The int8 weights of a layer
// (0.41 MB per SM for the 1B model) stream through a ring of three tile slots in shared memory: the producer
// warp walks the block's tiles in program order, across phases and layers, and requests each one
// (cp.async.bulk, all 32 lanes issue pieces, completion on the slot's `full` mbarrier) as soon as the compute
// warps have released the slot (`empty` mbarrier).  Grid barriers gate the compute only, never the weight
// stream.  Compute per tile: a warp per row, 16-byte pieces of the row against the int8 input vector in shared
// memory with dp4a.s32.s32 (exact i32), one shuffle reduction, and the epilogue of the phase on lane 0:
// store (q | k | v), x += acc / 65536 (wo, down), (i8)(silu(g / 65536) * (u / 65536) * 127) (gate | up).
// Per layer: rmsnorm + quantise + q/k/v | attention over the int8 cache ((head, split) items) | merge +
// requantise + wo | rmsnorm + quantise + gate/up | down; then rmsnorm + f32 classifier streamed from HBM.
// The arithmetic of every step is that of the per-op kernels in llama_i8.cu.
#include <algorithm>

#include "llama_i8_model.hpp"
#include "llama_persistent.cuh"

namespace simp {

constexpr int PI_SLOTS = 3;
constexpr size_t PI_STATIC_SMEM = 3072;
constexpr int PI_NW_REG = 8;   // norm weights a thread holds ahead of the barrier (dim <= 8 * 512)

struct PersistI8Args {
  PkCommon c;
  const int8_t *wq, *wk, *wv, *wo, *w1, *w2, *w3;
  const int8_t* x_in;    // int8 input vector [dim]
  int8_t *kc, *vc, *hb;  // caches [n_layers, max_seq, kv_dim]; FFN activation [hidden]
  int32_t *q, *k, *v;
  uint32_t slot_off[PI_SLOTS], xs_off, vec_off;
  int tr_a, tr_g, tr_d;  // rows per tile: single matrix with K = dim | gate + up pairs | K = hidden
};

struct PiSeg {
  const int8_t *w0, *w1;   // w1 != nullptr: gate + up pair
  int rows, K, cap;        // output rows of the matrix, row length in bytes, rows per tile
  int r0, n;               // this block's slice
};
__device__ __forceinline__ PiSeg pi_seg(const PersistI8Args& a, int l, int s) {
  const PkCommon& c = a.c;
  PiSeg g;
  g.w1 = nullptr;
  g.K = c.dim;
  g.cap = a.tr_a;
  const size_t L = size_t(l);
  if (s == 0) { g.rows = c.dim; g.w0 = a.wq + L * c.dim * c.dim; }
  else if (s == 1) { g.rows = c.kv; g.w0 = a.wk + L * c.kv * c.dim; }
  else if (s == 2) { g.rows = c.kv; g.w0 = a.wv + L * c.kv * c.dim; }
  else if (s == 3) { g.rows = c.dim; g.w0 = a.wo + L * c.dim * c.dim; }
  else if (s == 4) { g.rows = c.hd; g.w0 = a.w1 + L * c.hd * c.dim; g.w1 = a.w3 + L * c.hd * c.dim; g.cap = a.tr_g; }
  else { g.rows = c.dim; g.K = c.hd; g.w0 = a.w2 + L * c.dim * c.hd; g.cap = a.tr_d; }
  g.n = share_rows(g.rows, gridDim.x, blockIdx.x);
  g.r0 = share_row0(g.rows, gridDim.x, blockIdx.x);
  return g;
}
__device__ __forceinline__ void pi_tile_range(int n, int nt, int i, int& first, int& count) {
  const int base = n / nt, rem = n % nt;
  first = i * base + min(i, rem);
  count = base + (i < rem ? 1 : 0);
}
__device__ __forceinline__ int pi_dp4a(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int8_t pi_quant_clamped(float v) {   // clamp to [-128, 127], truncate toward zero
  v = fminf(v, 127.0f);
  v = fmaxf(v, -128.0f);
  return int8_t(__float2int_rz(v));
}
__device__ __forceinline__ float pi_compute_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  csync();
  if (lane == 0) red[warp] = v;
  csync();
  if (warp == 0) {
    float t = lane < PK_WARPS ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  csync();
  return red[32];
}

__global__ void __launch_bounds__(PK_BLOCK, 1) llama_i8_token_kernel(const PersistI8Args a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ PkStatic S;
  __shared__ __align__(8) uint64_t full[PI_SLOTS];
  __shared__ __align__(8) uint64_t empty[PI_SLOTS];
  const PkCommon& c = a.c;
  int8_t* xs = reinterpret_cast<int8_t*>(smem + a.xs_off);   // int8 input vector of the current projection
  float* scores = reinterpret_cast<float*>(smem + a.xs_off); // attention: scores of this block's split (xs is idle then)
  float* vec = reinterpret_cast<float*>(smem + a.vec_off);   // f32 vector (classifier input); attention scratch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dim = c.dim, hd = c.hd, hs = c.hs, kv_dim = c.kv;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < PI_SLOTS; ++k) {
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
    uint32_t slot = 0, use = 0;
    uint32_t last_use[PI_SLOTS] = {};
    uint32_t used = 0;
    bool ok = true;
    for (int l = 0; l < c.n_layers && ok; ++l)
      for (int s = 0; s < 6 && ok; ++s) {
        const PiSeg g = pi_seg(a, l, s);
        if (g.n == 0) continue;
        const int nt = (g.n + g.cap - 1) / g.cap;
        const int nm = g.w1 ? 2 : 1;
        for (int i = 0; i < nt && ok; ++i) {
          int first, count;
          pi_tile_range(g.n, nt, i, first, count);
          const uint32_t bar = ptx::smem_u32(&full[slot]);
          const uint32_t mat_bytes = uint32_t(count) * uint32_t(g.K);
          if (lane == 0) {
            if (use > 0) ok = ptx::mbar_wait(ptx::smem_u32(&empty[slot]), (use - 1) & 1u, &S.sh_abort, c.status, 60 + int(slot));
            if (ok) ptx::mbar_arrive_expect_tx(bar, mat_bytes * uint32_t(nm));
          }
          ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
          if (!ok) break;
          if (lane < 24) {   // 24 lanes issue the pieces of the tile together (12 per matrix for a pair)
            const int wl = 24 / nm, mi = lane / wl, piece = lane - mi * wl;
            const uint32_t psz = ((mat_bytes / 16 + wl - 1) / wl) * 16;
            const uint32_t off = uint32_t(piece) * psz;
            if (off < mat_bytes) {
              const int8_t* src = (mi == 0 ? g.w0 : g.w1) + size_t(g.r0 + first) * g.K + off;
              ptx::bulk_load(ptx::smem_u32(smem + a.slot_off[slot] + mi * mat_bytes + off), src, min(psz, mat_bytes - off), bar);
            }
          }
          last_use[slot] = use;
          used |= 1u << slot;
          if (++slot == PI_SLOTS) { slot = 0; ++use; }
        }
      }
    // Before this warp leaves, its last requests must have landed (bounded; see the W4 kernel).
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < PI_SLOTS; ++k)
        if (used & (1u << k))
          for (int spin = 0; spin < 400000; ++spin)
            if (ptx::mbar_try_wait(ptx::smem_u32(&full[k]), last_use[k] & 1u)) break;
      *reinterpret_cast<volatile int*>(&S.prod_done) = 1;
    }
    return;
  }

  // ================================================================== compute warps
  unsigned epoch = 0;
  uint32_t slot = 0, use = 0;
  int tile_parity = 0;
  auto drain = [&]() {
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(&S.sh_abort) = 1;
      for (int spin = 0; spin < 4000000 && *reinterpret_cast<volatile int*>(&S.prod_done) == 0; ++spin) {}
    }
    csync();
  };
  // All tiles of segment s of layer l.  mode 0: out[row] = acc; 1: x[row] += acc / 65536; 2: hb[row] = swiglu.
  auto run_segment = [&](int l, int s, int mode, int32_t* out) -> bool {
    const PiSeg g = pi_seg(a, l, s);
    if (g.n == 0) return true;
    const int nt = (g.n + g.cap - 1) / g.cap;
    const int k16 = g.K >> 4;
    const uint4* xv = reinterpret_cast<const uint4*>(xs);
    for (int i = 0; i < nt; ++i) {
      int first, count;
      pi_tile_range(g.n, nt, i, first, count);
      if (!ptx::mbar_wait(ptx::smem_u32(&full[slot]), use & 1u, &S.sh_abort, c.status, 70 + int(slot))) return false;
      const uint8_t* sl = smem + a.slot_off[slot];
      const size_t mat_bytes = size_t(count) * g.K;
      // Few rows in the tile: two warps share a row (halves of K), so all 16 warps work and a row's latency chain
      // is half as long; the halves meet in shared memory and one thread per row runs the epilogue.
      const bool split = count <= PK_WARPS / 2;
      int* pbuf = S.halves[tile_parity];
      auto epilogue = [&](int r, int acc0, int acc1, float resid) {
        const int row = g.r0 + first + r;
        if (mode == 0) out[row] = acc0;
        if (mode == 1) c.x[row] = resid + float(acc0) / 65536.0f;
        if (mode == 2) {
          const float gate_f = float(acc0) / 65536.0f;
          const float silu = gate_f / (1.0f + expf(0.0f - gate_f));
          const float up_f = float(acc1) / 65536.0f;
          float hbv = silu * up_f * 127.0f;
          hbv = fmaxf(fminf(hbv, 2147483520.0f), -2147483648.0f);
          a.hb[row] = int8_t(uint8_t(uint32_t(__float2int_rz(hbv)) & 0xffu));
        }
      };
      // A warp has one or two rows per tile, so a row is a latency chain: four pieces of every operand are
      // requested before the first dp4a, two accumulators per matrix, and the lane sums are combined with the
      // integer warp-reduce instruction instead of five shuffle steps.
      auto row_dot = [&](int r, int jbeg, int jend, int& acc0, int& acc1) {
        const uint4* w0 = reinterpret_cast<const uint4*>(sl + size_t(r) * g.K);
        const uint4* w1 = reinterpret_cast<const uint4*>(sl + mat_bytes + size_t(r) * g.K);
        int accA[2] = {0, 0}, accB[2] = {0, 0};
        for (int j0 = jbeg + lane; j0 < jend; j0 += 128) {
          uint4 x4[4], p[4], q[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int j = j0 + 32 * u;
            const bool on = j < jend;
            x4[u] = on ? xv[j] : make_uint4(0u, 0u, 0u, 0u);
            p[u] = on ? w0[j] : make_uint4(0u, 0u, 0u, 0u);
            q[u] = (on && mode == 2) ? w1[j] : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            int t = accA[u & 1];
            t = pi_dp4a(p[u].x, x4[u].x, t); t = pi_dp4a(p[u].y, x4[u].y, t);
            t = pi_dp4a(p[u].z, x4[u].z, t); t = pi_dp4a(p[u].w, x4[u].w, t);
            accA[u & 1] = t;
            if (mode == 2) {
              int v = accB[u & 1];
              v = pi_dp4a(q[u].x, x4[u].x, v); v = pi_dp4a(q[u].y, x4[u].y, v);
              v = pi_dp4a(q[u].z, x4[u].z, v); v = pi_dp4a(q[u].w, x4[u].w, v);
              accB[u & 1] = v;
            }
          }
        }
        acc0 = __reduce_add_sync(0xffffffffu, accA[0] + accA[1]);
        acc1 = mode == 2 ? __reduce_add_sync(0xffffffffu, accB[0] + accB[1]) : 0;
      };
      if (split) {
        const int r = warp >> 1, half = warp & 1;
        const int kh = ((k16 + 1) >> 1);
        float resid = 0.0f;
        if (mode == 1 && int(threadIdx.x) < count) resid = __ldcg(c.x + g.r0 + first + threadIdx.x);   // ahead of the sync
        if (r < count) {
          int acc0, acc1;
          row_dot(r, half * kh, min(k16, (half + 1) * kh), acc0, acc1);
          if (lane == 0) { pbuf[(half * 2 + 0) * PK_WARPS + r] = acc0; pbuf[(half * 2 + 1) * PK_WARPS + r] = acc1; }
        }
        csync();
        if (threadIdx.x == 0) ptx::mbar_arrive(ptx::smem_u32(&empty[slot]));   // every warp has read the slot
        if (int(threadIdx.x) < count) {
          const int t = threadIdx.x;
          epilogue(t, pbuf[0 * PK_WARPS + t] + pbuf[2 * PK_WARPS + t], pbuf[1 * PK_WARPS + t] + pbuf[3 * PK_WARPS + t], resid);
        }
      } else {
        // residual rows are requested before the dot products so their L2 round trip overlaps them
        float resid[2] = {0.0f, 0.0f};
        if (mode == 1) {
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int r = warp + u * PK_WARPS;
            if (r < count) resid[u] = __ldcg(c.x + g.r0 + first + r);
          }
        }
        for (int r = warp; r < count; r += PK_WARPS) {
          int acc0, acc1;
          row_dot(r, 0, k16, acc0, acc1);
          if (lane == 0) epilogue(r, acc0, acc1, r < 2 * PK_WARPS ? resid[r >= PK_WARPS ? 1 : 0] : __ldcg(c.x + g.r0 + first + r));
        }
        csync();
        if (threadIdx.x == 0) ptx::mbar_arrive(ptx::smem_u32(&empty[slot]));   // every warp has read the slot
      }
      tile_parity ^= 1;
      if (++slot == PI_SLOTS) { slot = 0; ++use; }
    }
    return true;
  };
  // xs = quantise(rmsnorm(x) * w): y = (x / r) * w, v = y * 127 clamped and truncated.  nw holds the first
  // PI_NW_REG norm weights of each thread, requested before the preceding grid barrier.
  auto stage_norm_quant = [&](const float* w, const float (&nw)[PI_NW_REG]) {
    float xr[PI_NW_REG];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < PI_NW_REG; ++u) {
      const int i = threadIdx.x + u * PK_THREADS;
      xr[u] = i < dim ? __ldcg(c.x + i) : 0.0f;
      ss += xr[u] * xr[u];
    }
    for (int i = threadIdx.x + PI_NW_REG * PK_THREADS; i < dim; i += PK_THREADS) {
      const float t = __ldcg(c.x + i);
      ss += t * t;
    }
    ss = compute_sum(ss, S.red);
    const float r = sqrtf(ss / float(dim) + 1e-5f);
#pragma unroll
    for (int u = 0; u < PI_NW_REG; ++u) {
      const int i = threadIdx.x + u * PK_THREADS;
      if (i < dim) xs[i] = pi_quant_clamped(((xr[u] / r) * nw[u]) * 127.0f);
    }
    for (int i = threadIdx.x + PI_NW_REG * PK_THREADS; i < dim; i += PK_THREADS)
      xs[i] = pi_quant_clamped(((__ldcg(c.x + i) / r) * w[i]) * 127.0f);
    csync();
  };
  auto load_norm_w = [&](const float* w, float (&nw)[PI_NW_REG]) {
#pragma unroll
    for (int u = 0; u < PI_NW_REG; ++u) {
      const int i = threadIdx.x + u * PK_THREADS;
      nw[u] = i < dim ? __ldg(w + i) : 0.0f;
    }
  };

  // ---- x = (f32) x_i8 (each block converts a slice), then everyone may read x
  for (int i = blockIdx.x * PK_THREADS + threadIdx.x; i < dim; i += gridDim.x * PK_THREADS) c.x[i] = float(a.x_in[i]) * 1.0f;
  float nw[PI_NW_REG];
  load_norm_w(c.rms_att, nw);
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  const int pos = c.ctl[0], seq = pos + 1;
  const int NS = c.nsplit;   // sequence splits per head (blocks of empty splits publish an empty partial)

  for (int l = 0; l < c.n_layers; ++l) {
    // ------------------------------------------------------------------ phase 0: q | k | v
    stage_norm_quant(c.rms_att + size_t(l) * dim, nw);
    if (!run_segment(l, 0, 0, a.q) || !run_segment(l, 1, 0, a.k) || !run_segment(l, 2, 0, a.v)) { drain(); return; }
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    // ------------------------------------------------------------------ phase 1: attention
    if (int(blockIdx.x) < c.n_heads * NS) {
      const int h = blockIdx.x / NS, sp = blockIdx.x % NS, kvh = h / c.kv_mul;
      float* qf = S.qs;
      float* knew = S.ks;
      float* vnew = S.vs;
      int8_t* kbase = a.kc + size_t(l) * c.seq_len * kv_dim + kvh * hs;
      int8_t* vbase = a.vc + size_t(l) * c.seq_len * kv_dim + kvh * hs;
      for (int d = threadIdx.x; d < hs; d += PK_THREADS) {
        qf[d] = float(__ldcg(a.q + h * hs + d));
        const int8_t k8 = int8_t(uint8_t(uint32_t(__ldcg(a.k + kvh * hs + d) / 256) & 0xffu));
        const int8_t v8 = int8_t(uint8_t(uint32_t(__ldcg(a.v + kvh * hs + d) / 256) & 0xffu));
        knew[d] = float(k8);
        vnew[d] = float(v8);
        if (sp == 0 && h % c.kv_mul == 0) {
          kbase[size_t(pos) * kv_dim + d] = k8;
          vbase[size_t(pos) * kv_dim + d] = v8;
        }
      }
      csync();
      const int per = (seq + NS - 1) / NS;
      const int t0 = sp * per, t1 = min(seq, t0 + per), len = max(0, t1 - t0);
      const int pieces = hs >> 4, tpw = 32 / pieces;
      const int piece = lane % pieces, tsub = lane / pieces;
      float q_r[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) q_r[i] = qf[piece * 16 + i];
      auto load_row = [&](const int8_t* base, const float* fresh, int t, float (&f)[16]) {
        if (t == pos) {
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = fresh[piece * 16 + i];
        } else {
          const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(base + size_t(t) * kv_dim + piece * 16));
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 16; ++i) f[i] = float(int8_t(uint8_t(w[i >> 2] >> (8 * (i & 3)))));
        }
      };
      for (int tb = t0 + warp * tpw; tb < t1; tb += PK_WARPS * tpw) {
        const int t = tb + tsub;
        float sc = 0.0f;
        if (t < t1) {
          float kf[16];
          load_row(kbase, knew, t, kf);
#pragma unroll
          for (int i = 0; i < 16; ++i) sc = fmaf(q_r[i], kf[i], sc);
        }
        for (int o = 1; o < pieces; o <<= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
        if (piece == 0 && t < t1) scores[t - t0] = sc / 8.0f;
      }
      csync();
      float mx = -INFINITY;
      for (int i = threadIdx.x; i < len; i += PK_THREADS) mx = fmaxf(mx, scores[i]);
      mx = pi_compute_max(mx, S.red);
      float sum = 0.0f;
      for (int i = threadIdx.x; i < len; i += PK_THREADS) {
        const float e = expf(scores[i] - mx);
        scores[i] = e;
        sum += e;
      }
      sum = compute_sum(sum, S.red);
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
      for (int tb = t0 + warp * tpw; tb < t1; tb += PK_WARPS * tpw) {
        const int t = tb + tsub;
        if (t < t1) {
          float vf[16];
          load_row(vbase, vnew, t, vf);
          const float p = scores[t - t0];
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[i] = fmaf(p, vf[i], acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float v = acc[i];
        for (int o = pieces; o < 32; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[i] = v;
      }
      if (tsub == 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) vec[warp * 128 + piece * 16 + i] = acc[i];
      }
      csync();
      float* mine = c.part + (size_t(h) * NS + sp) * (hs + 2);
      for (int d = threadIdx.x; d < hs; d += PK_THREADS) {
        float val = 0.0f;
#pragma unroll
        for (int w = 0; w < PK_WARPS; ++w) val += vec[w * 128 + d];
        mine[2 + d] = val;
      }
      if (threadIdx.x == 0) { mine[0] = len > 0 ? mx : -INFINITY; mine[1] = len > 0 ? sum : 0.0f; }
    }
    load_norm_w(c.rms_ffn + size_t(l) * dim, nw);
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    // ------------------------------------------------------------------ phase 2: merge + requantise, wo
    pk_merge_heads(c, vec);   // normalised attention output of every head, f32
    csync();
    for (int i = threadIdx.x; i < dim; i += PK_THREADS) {
      const int32_t outv = __float2int_rz(vec[i]);                // attn_out = val as i32
      xs[i] = pi_quant_clamped(float(outv) / 256.0f);             // next projection's input
    }
    csync();
    if (!run_segment(l, 3, 1, nullptr)) { drain(); return; }
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    // ------------------------------------------------------------------ phase 3: gate | up
    stage_norm_quant(c.rms_ffn + size_t(l) * dim, nw);
    if (!run_segment(l, 4, 2, nullptr)) { drain(); return; }
    if (l + 1 < c.n_layers) load_norm_w(c.rms_att + size_t(l + 1) * dim, nw);
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
    // ------------------------------------------------------------------ phase 4: down
    for (int i = threadIdx.x; i < (hd >> 4); i += PK_THREADS)
      reinterpret_cast<uint4*>(xs)[i] = __ldcg(reinterpret_cast<const uint4*>(a.hb) + i);
    csync();
    if (!run_segment(l, 5, 1, nullptr)) { drain(); return; }
    if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  }

  // ---------------------------------------------------------------------- final norm + f32 classifier
  {
    const float r = stage_x_rms(c.x, vec, dim, S.red);
    finish_rmsnorm(vec, c.rms_final, r, dim);
  }
  pk_classifier(c, S, vec);
  if (!grid_sync(c.bar, epoch, &S.sh_abort, c.status, 0)) { drain(); return; }
  if (blockIdx.x == 0 && threadIdx.x == 0) c.ctl[0] = pos + 1;
}

// ---------------------------------------------------------------------------------------------
struct PersistI8Plan {
  uint32_t slot_off[PI_SLOTS], xs_off, vec_off;
  int tr_a, tr_g, tr_d;
  size_t total;
  bool ok;
};
static PersistI8Plan persist_i8_plan(const LlamaI8Model& m, int G) {
  PersistI8Plan p{};
  const simp_llama_i8_config& c = m.cfg;
  auto al = [](size_t v) { return (v + 127) & ~size_t(127); };
  const int nsplit = 4;
  const size_t score_bytes = (size_t(c.max_seq_len + nsplit - 1) / nsplit + 1) * 4;
  const size_t xs_bytes = al(std::max<size_t>(size_t(std::max(c.dim, c.hidden_dim)), score_bytes));
  const size_t vec_bytes = al(std::max<size_t>(size_t(c.dim) * 4, size_t(PK_WARPS) * 128 * 4));
  const size_t fixed = xs_bytes + vec_bytes + PI_STATIC_SMEM;
  if (fixed + PI_SLOTS * 4096 > PK_SMEM_LIMIT) return p;
  const size_t slot_bytes = ((PK_SMEM_LIMIT - fixed) / PI_SLOTS) & ~size_t(127);
  p.tr_a = int(std::min<size_t>(2 * PK_WARPS, slot_bytes / size_t(c.dim)));
  p.tr_g = int(std::min<size_t>(PK_WARPS, slot_bytes / size_t(2 * c.dim)));
  p.tr_d = int(std::min<size_t>(2 * PK_WARPS, slot_bytes / size_t(c.hidden_dim)));
  if (p.tr_a < 1 || p.tr_g < 1 || p.tr_d < 1) return p;
  if (c.n_heads > G || c.dim > PI_NW_REG * PK_THREADS * 8) return p;
  size_t off = 0;
  for (int s = 0; s < PI_SLOTS; ++s) { p.slot_off[s] = uint32_t(off); off += slot_bytes; }
  p.xs_off = uint32_t(off); off += xs_bytes;
  p.vec_off = uint32_t(off); off += vec_bytes;
  p.total = off;
  p.ok = true;
  return p;
}

bool persistent_i8_supported(const LlamaI8Model& m) {
  if (!ctx().ready) return false;
  int coop = 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx().device) != cudaSuccess || !coop) return false;
  return persist_i8_plan(m, ctx().sm_count).ok;
}

int enqueue_token_persistent_i8(LlamaI8Model& m, cudaStream_t st) {
  const int G = ctx().sm_count;
  const PersistI8Plan p = persist_i8_plan(m, G);
  SIMP_REQUIRE(p.ok, SIMP_ERR_UNSUPPORTED, "persistent int8 decode: model does not fit the shared-memory plan");
  const simp_llama_i8_config& c = m.cfg;
  PersistI8Args a{};
  PkCommon& k = a.c;
  k.dim = int(c.dim); k.hd = int(c.hidden_dim); k.kv = int(m.kv_dim); k.hs = int(c.head_dim);
  k.n_heads = int(c.n_heads); k.kv_mul = int(c.n_heads / c.n_kv_heads); k.n_layers = int(c.n_layers);
  k.vocab = int(c.vocab_size); k.seq_len = int(c.max_seq_len);
  k.nsplit = 4;
  while (k.nsplit > 1 && k.n_heads * k.nsplit > G) k.nsplit >>= 1;
  k.rms_att = m.rms_att; k.rms_ffn = m.rms_ffn; k.rms_final = m.rms_final; k.wcls = m.wcls;
  k.x = m.x; k.logits = m.logits; k.part = m.pk_part; k.ctl = m.ctl;
  k.bar = m.pk_bar; k.best_val = m.pk_best_val; k.best_idx = m.pk_best_idx; k.status = ctx().dev_status;
  a.wq = m.wq; a.wk = m.wk; a.wv = m.wv; a.wo = m.wo; a.w1 = m.w1; a.w2 = m.w2; a.w3 = m.w3;
  a.x_in = m.x_i8; a.kc = m.kc; a.vc = m.vc; a.hb = m.ffn_hb; a.q = m.q; a.k = m.k; a.v = m.v;
  for (int s = 0; s < PI_SLOTS; ++s) a.slot_off[s] = p.slot_off[s];
  a.xs_off = p.xs_off; a.vec_off = p.vec_off;
  a.tr_a = p.tr_a; a.tr_g = p.tr_g; a.tr_d = p.tr_d;
  if (!m.pk_attr_done) {   // first (eager) pass of this model, outside any stream capture
    SIMP_CUDA(cudaFuncSetAttribute(llama_i8_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   int(PK_SMEM_LIMIT - PI_STATIC_SMEM)));
    m.pk_attr_done = true;
  }
  return pk_launch(reinterpret_cast<const void*>(llama_i8_token_kernel), &a, m.pk_bar, p.total, st);
}

}  // namespace simp
