// llama_persistent.cu -- one token of the f32 LLaMA model (examples/llama2/stories110M.sl:5-247) as ONE
// persistent cooperative kernel: one block per SM (16 compute warps + 1 producer warp), the phases of the
// forward pass separated by grid-wide barriers instead of kernel launches.
//
// Why: at batch 1 the per-op graph is a chain of ~64 dependent kernels whose launch floor (~1.2 us each)
// and cold first loads dominate, while a layer's weights are only ~190 KB per SM.  Here every block owns a
// fixed, contiguous slice of the rows of each projection, and shared memory holds one buffer per
// projection group (q/k/v + norm weights | wo | gate/up + norm weights | down).  The producer warp refills
// a buffer with the next layer's slice (cp.async.bulk + mbarrier) the moment the compute warps release it,
// so each slice has a whole layer's time to arrive, HBM streams continuously under the dependency chain,
// and a phase costs one grid barrier plus its short compute out of shared memory.
// Per layer: q/k/v (rmsnorm folded in) | attention (RoPE, KV store, split-sequence online softmax) |
// wo + residual (merging the attention partials) | gate/up + silu*mul (rmsnorm folded in) | down + residual;
// then rmsnorm + classifier streamed from HBM + greedy argmax.  Arithmetic and reduction orders are fixed,
// so results are run-to-run identical.
//
// Grid barrier: one global arrival counter, monotonic within a launch (zeroed by a memset node before the
// kernel).  The wait is bounded (1 s): on expiry an error word is set that every waiter polls, all blocks
// leave, and the host reports the timeout; cooperative launch guarantees all blocks are co-resident.
#include "common.cuh"
#include "llama_model.hpp"
#include "sm100_ptx.cuh"

namespace simp {

constexpr int PK_THREADS = 512;
constexpr int PK_WARPS = PK_THREADS / 32;
constexpr int PK_BLOCK = PK_THREADS + 32;   // 16 compute warps + 1 producer warp (weight requests)
constexpr uint32_t PK_COPY_CHUNK = 16384;
constexpr size_t PK_MAX_DYN_SMEM = 227 * 1024 - 2560;   // per-block limit less this kernel's static shared memory

struct PersistArgs {
  int dim, hd, kv, hs, n_heads, kv_mul, n_layers, vocab, seq_len, nsplit;
  const float *tok_emb, *rms_att, *rms_ffn, *rms_final, *wcls, *wq, *wk, *wv, *wo, *w1, *w2, *w3;
  float *x, *xb, *hb, *q, *k, *v, *logits, *kc, *vc, *part;
  int* ctl;
  const int32_t* prompt;
  int32_t* out_tokens;
  unsigned* bar;    // [0] arrivals, [1] error word
  float* best_val;  // per-block argmax partials
  int* best_idx;
  int* status;      // library-wide device status word
  uint32_t koff[5];     // shared-memory byte offset of the weight buffer of each phase kind (kind 1 has none)
  uint32_t xs_off;      // offset of the staged-vector buffer
};

__device__ __forceinline__ int share_rows(int R, int G, int b) { return R / G + (b < R % G ? 1 : 0); }
__device__ __forceinline__ int share_row0(int R, int G, int b) { return b * (R / G) + min(b, R % G); }

// Barrier over the compute warps only; the producer warp never joins it.
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(PK_THREADS) : "memory"); }

__device__ __forceinline__ float compute_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  csync();
  if (lane == 0) red[warp] = v;
  csync();
  if (warp == 0) {
    float t = lane < PK_WARPS ? red[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  csync();
  return red[32];
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded grid-wide barrier, entered by the compute warps.  Returns false when the barrier was abandoned
// (error word set).  `freed` (0 = none) is the shared-memory address of the mbarrier that tells the producer
// warp that this phase's weight buffer may be refilled: it is signalled right after the leading block-wide
// sync, off the barrier's critical path.
__device__ __forceinline__ bool grid_sync(unsigned* bar, unsigned& epoch, int* sh_abort, int* status, uint32_t freed) {
  csync();
  ++epoch;
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
    if (freed) ptx::mbar_arrive(freed);
    const unsigned target = epoch * gridDim.x;
    const uint64_t t0 = ptx::globaltimer_ns();
    for (unsigned spin = 1;; ++spin) {
      if (ld_acquire_u32(&bar[0]) >= target) break;
      if ((spin & 63u) == 0) {
        if (ld_acquire_u32(&bar[1]) != 0) { *sh_abort = 1; break; }
        if (ptx::globaltimer_ns() - t0 > 1000000000ull) {
          atomicExch(&bar[1], 1u);
          if (atomicCAS(status, 0, 1) == 0) status[1] = 30;
          *sh_abort = 1;
          break;
        }
      }
    }
  }
  csync();
  return *reinterpret_cast<volatile int*>(sh_abort) == 0;
}

// y (shared) = rmsnorm(x (global)) * w: the arithmetic of RMSNormOpLowering.
// Returns with xs holding the un-normalised x; finish_rmsnorm() applies (x / r) * w once w is at hand.
__device__ __forceinline__ float stage_x_rms(const float* __restrict__ x, float* xs, int n, float* red) {
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += PK_THREADS) {
    const float t = __ldcg(x + i);
    xs[i] = t;
    ss += t * t;
  }
  ss = compute_sum(ss, red);
  return sqrtf(ss / float(n) + 1e-5f);
}
__device__ __forceinline__ void finish_rmsnorm(float* xs, const float* w, float r, int n) {
  for (int i = threadIdx.x; i < n; i += PK_THREADS) xs[i] = (xs[i] / r) * w[i];
  csync();
}

// dot of one row held in shared memory (k4 float4) with the staged vector.
__device__ __forceinline__ float row_dot(const float4* __restrict__ row, const float4* __restrict__ xv, int k4, int lane) {
  float acc = 0.0f;
  for (int i = lane; i < k4; i += 32) {
    const float4 a = row[i], b = xv[i];
    acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc);
    acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
  }
  return warp_sum(acc);
}

// Two rows against the staged vector at once: the vector is read from shared memory once per pair, which
// matters because these dots run at the shared-memory bandwidth limit.
__device__ __forceinline__ void row_dot2(const float4* __restrict__ r0, const float4* __restrict__ r1,
                                         const float4* __restrict__ xv, int k4, int lane, float& o0, float& o1) {
  float a0 = 0.0f, a1 = 0.0f;
  for (int i = lane; i < k4; i += 32) {
    const float4 b = xv[i], p = r0[i], q = r1[i];
    a0 = fmaf(p.x, b.x, a0); a0 = fmaf(p.y, b.y, a0); a0 = fmaf(p.z, b.z, a0); a0 = fmaf(p.w, b.w, a0);
    a1 = fmaf(q.x, b.x, a1); a1 = fmaf(q.y, b.y, a1); a1 = fmaf(q.z, b.z, a1); a1 = fmaf(q.w, b.w, a1);
  }
  o0 = warp_sum(a0);
  o1 = warp_sum(a1);
}

__global__ void __launch_bounds__(PK_BLOCK, 1) llama_f32_token_kernel(const PersistArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ float red[33];
  __shared__ __align__(8) uint64_t full[5];   // weights of a phase kind have landed (phase parity = layer parity)
  __shared__ __align__(8) uint64_t freeb[5];  // the compute warps are done with that kind's buffer
  __shared__ int sh_abort, prod_done;
  __shared__ float sm_m[PK_WARPS], sm_s[PK_WARPS];
  __shared__ float qs[128], ks[128], vs[128];
  float* xs = reinterpret_cast<float*>(smem + a.xs_off);   // staged input vector
  float* sm_acc = xs;                                      // [PK_WARPS][128] attention scratch (xs is idle then)
  const int G = gridDim.x, b = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dim = a.dim, hd = a.hd, kv = a.kv, hs = a.hs;
  unsigned epoch = 0;
  // this block's row slices of the three output widths
  const int n_dim = share_rows(dim, G, b), r0_dim = share_row0(dim, G, b);
  const int n_kv = share_rows(kv, G, b), r0_kv = share_row0(kv, G, b);
  const int n_hd = share_rows(hd, G, b), r0_hd = share_row0(hd, G, b);

  if (threadIdx.x == 0) {
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      ptx::mbar_init(ptx::smem_u32(&full[k]), 1);
      ptx::mbar_init(ptx::smem_u32(&freeb[k]), 1);
    }
    sh_abort = 0;
    prod_done = 0;
    ptx::fence_barrier_init();
  }
  __syncthreads();

  // ================================================================== producer warp
  // Requests this block's slice of every layer for each phase kind (0 q/k/v, 2 wo, 3 gate/up, 4 down) into
  // that kind's own buffer, as soon as the compute warps have released the buffer.  A slice therefore has a
  // whole layer's time to arrive, HBM streams continuously under the dependency chain, and the time the copy
  // engine takes to accept the requests is not on the compute warps' path.
  if (warp == PK_WARPS) {
    if (lane != 0) return;
    int outstanding = 0, parity = 0;   // bit k: kind k has a request in flight / parity of its layer
    auto issue = [&](int l, int kind) {
      const uint32_t bar = ptx::smem_u32(&full[kind]);
      uint8_t* dst = smem + a.koff[kind];
      auto vec = [&](const float* w, uint32_t& off, uint32_t& total, bool count_only) {   // norm weights of layer l
        const uint32_t bytes = uint32_t(dim) * 4u;
        if (count_only) { total += bytes; return; }
        ptx::bulk_load(ptx::smem_u32(dst + off), w + size_t(l) * dim, bytes, bar);
        off += bytes;
      };
      auto one = [&](const float* W, int R, int K, uint32_t& off, uint32_t& total, bool count_only) {
        const int n = R == dim ? n_dim : (R == hd ? n_hd : n_kv);
        const int first = R == dim ? r0_dim : (R == hd ? r0_hd : r0_kv);
        const uint32_t bytes = uint32_t(n) * uint32_t(K) * 4u;
        if (bytes == 0) return;
        if (count_only) { total += bytes; return; }
        const uint8_t* src = reinterpret_cast<const uint8_t*>(W + (size_t(l) * R + first) * K);
        for (uint32_t done = 0; done < bytes; done += PK_COPY_CHUNK)
          ptx::bulk_load(ptx::smem_u32(dst + off + done), src + done, min(PK_COPY_CHUNK, bytes - done), bar);
        off += bytes;
      };
      for (int pass = 0; pass < 2; ++pass) {
        uint32_t off = 0, total = 0;
        const bool co = pass == 0;
        if (kind == 0) { vec(a.rms_att, off, total, co); one(a.wq, dim, dim, off, total, co); one(a.wk, kv, dim, off, total, co); one(a.wv, kv, dim, off, total, co); }
        if (kind == 2) one(a.wo, dim, dim, off, total, co);
        if (kind == 3) { vec(a.rms_ffn, off, total, co); one(a.w1, hd, dim, off, total, co); one(a.w3, hd, dim, off, total, co); }
        if (kind == 4) one(a.w2, dim, hd, off, total, co);
        if (co) {
          if (total == 0) { ptx::mbar_arrive(bar); return; }   // empty slice
          ptx::mbar_arrive_expect_tx(bar, total);
        }
      }
      outstanding |= 1 << kind;
      parity = (parity & ~(1 << kind)) | ((l & 1) << kind);
    };
    bool ok = true;
    for (int l = 0; l < a.n_layers && ok; ++l)
      for (int kind = 0; kind < 5 && ok; ++kind) {
        if (kind == 1) continue;
        if (l > 0) ok = ptx::mbar_wait(ptx::smem_u32(&freeb[kind]), uint32_t((l - 1) & 1), &sh_abort, a.status, 40 + kind);
        if (ok) issue(l, kind);
      }
    // Before this warp leaves, its last requests must have landed (they have, unless the kernel is being
    // abandoned; then the bounded wait keeps copies from arriving in shared memory that is no longer ours).
    for (int k = 0; k < 5; ++k)
      if (outstanding & (1 << k))
        for (int spin = 0; spin < 400000; ++spin)
          if (ptx::mbar_try_wait(ptx::smem_u32(&full[k]), uint32_t((parity >> k) & 1))) break;
    *reinterpret_cast<volatile int*>(&prod_done) = 1;
    return;
  }

  // ================================================================== compute warps
  auto wait_weights = [&](int l, int kind) {
    return ptx::mbar_wait(ptx::smem_u32(&full[kind]), uint32_t(l & 1), &sh_abort, a.status, 20 + kind);
  };
  // Error exit: raise the abort flag for the producer and give it a bounded time to see its copies land.
  auto drain = [&]() {
    if (threadIdx.x == 0) {
      *reinterpret_cast<volatile int*>(&sh_abort) = 1;
      for (int spin = 0; spin < 4000000 && *reinterpret_cast<volatile int*>(&prod_done) == 0; ++spin) {}
    }
    csync();
  };

  // ---- embedding: x = table[token] (each block copies a slice), then everyone may read x
  {
    const int64_t token = a.ctl[0];
    for (int i = b * PK_THREADS + threadIdx.x; i < dim; i += G * PK_THREADS) a.x[i] = a.tok_emb[token * dim + i];
  }
  if (!grid_sync(a.bar, epoch, &sh_abort, a.status, 0)) { drain(); return; }
  const int pos = a.ctl[1];

  for (int l = 0; l < a.n_layers; ++l) {
    // ------------------------------------------------------------------ phase 0: q/k/v
    {
      constexpr int kind = 0;
      const float r = stage_x_rms(a.x, xs, dim, red);
      if (!wait_weights(l, kind)) { drain(); return; }
      finish_rmsnorm(xs, reinterpret_cast<const float*>(smem + a.koff[kind]), r, dim);
      const int nq = n_dim, nk = n_kv, q0 = r0_dim, k0 = r0_kv;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind] + size_t(dim) * 4);
      const float4* xv = reinterpret_cast<const float4*>(xs);
      const int k4 = dim >> 2;
      const int nt = nq + 2 * nk;
      auto put = [&](int r, float v) {
        if (r < nq) a.q[q0 + r] = v;
        else if (r < nq + nk) a.k[k0 + r - nq] = v;
        else a.v[k0 + r - nq - nk] = v;
      };
      for (int r = 2 * warp; r < nt; r += 2 * PK_WARPS) {
        if (r + 1 < nt) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { put(r, v0); put(r + 1, v1); }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) put(r, v);
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(a.bar, epoch, &sh_abort, a.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 1: attention
    {
      const int S = a.nsplit;
      if (b < a.n_heads * S) {
        const int h = b / S, sp = b % S, kvh = h / a.kv_mul;
        if (int(threadIdx.x) < hs / 2) {
          const int i = 2 * threadIdx.x;
          const float freq = 1.0f / powf(10000.0f, float(i) / float(hs));
          const float val = float(pos) * freq;
          const float fcr = cosf(val), fci = sinf(val);
          const float q0 = __ldcg(a.q + h * hs + i), q1 = __ldcg(a.q + h * hs + i + 1);
          qs[i] = q0 * fcr - q1 * fci;
          qs[i + 1] = q0 * fci + q1 * fcr;
          const float k0 = __ldcg(a.k + kvh * hs + i), k1 = __ldcg(a.k + kvh * hs + i + 1);
          ks[i] = k0 * fcr - k1 * fci;
          ks[i + 1] = k0 * fci + k1 * fcr;
          vs[i] = __ldcg(a.v + kvh * hs + i);
          vs[i + 1] = __ldcg(a.v + kvh * hs + i + 1);
        }
        csync();
        float* kbase = a.kc + size_t(l) * a.seq_len * kv + kvh * hs;
        float* vbase = a.vc + size_t(l) * a.seq_len * kv + kvh * hs;
        if (sp == 0 && h % a.kv_mul == 0)
          for (int i = threadIdx.x; i < hs; i += PK_THREADS) {
            kbase[size_t(pos) * kv + i] = ks[i];
            vbase[size_t(pos) * kv + i] = vs[i];
          }
        const int len = pos + 1, per = (len + S - 1) / S;
        const int t0 = sp * per, t1 = min(len, t0 + per);
        const float div = sqrtf(float(hs));
        float qr[4], acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = lane + 32 * e;
          qr[e] = i < hs ? qs[i] : 0.0f;
          acc[e] = 0.0f;
        }
        float m = -INFINITY, s = 0.0f;
        constexpr int TU = 4;   // timesteps in flight per warp: their K/V rows are requested together
        for (int tb = t0 + warp; tb < t1; tb += PK_WARPS * TU) {
          float kr[TU][4], vr[TU][4];
#pragma unroll
          for (int u = 0; u < TU; ++u) {
            const int t = tb + u * PK_WARPS;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = lane + 32 * e;
              kr[u][e] = 0.0f; vr[u][e] = 0.0f;
              if (i < hs && t < t1) {
                if (t == pos) { kr[u][e] = ks[i]; vr[u][e] = vs[i]; }
                else { kr[u][e] = __ldcg(kbase + size_t(t) * kv + i); vr[u][e] = __ldcg(vbase + size_t(t) * kv + i); }
              }
            }
          }
#pragma unroll
          for (int u = 0; u < TU; ++u) {
            if (tb + u * PK_WARPS >= t1) break;
            float d = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) d = fmaf(qr[e], kr[u][e], d);
            const float score = warp_sum(d) / div;
            const float m_new = fmaxf(m, score);
            const float corr = expf(m - m_new);
            const float p = expf(score - m_new);
            s = s * corr + p;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[e] = acc[e] * corr + p * vr[u][e];
            m = m_new;
          }
        }
        if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = lane + 32 * e;
          if (i < hs) sm_acc[warp * 128 + i] = acc[e];
        }
        csync();
        float* mine = a.part + (size_t(h) * S + sp) * (hs + 2);
        if (warp == 0) {
          // lane w holds warp w's running maximum; one expf per lane, broadcast by shuffle
          const float mw = lane < PK_WARPS ? sm_m[lane] : -INFINITY;
          float M = mw;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
          const float scl = mw == -INFINITY ? 0.0f : expf(mw - M);
          float sc[PK_WARPS];
#pragma unroll
          for (int w = 0; w < PK_WARPS; ++w) sc[w] = __shfl_sync(0xffffffffu, scl, w);
          float Ssum = 0.0f;
#pragma unroll
          for (int w = 0; w < PK_WARPS; ++w) Ssum += sm_s[w] * sc[w];
          if (lane == 0) { mine[0] = M; mine[1] = Ssum; }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = lane + 32 * e;
            if (i < hs) {
              float v = 0.0f;
#pragma unroll
              for (int w = 0; w < PK_WARPS; ++w) v += sm_acc[w * 128 + i] * sc[w];
              mine[2 + i] = v;
            }
          }
        }
      }
      if (!grid_sync(a.bar, epoch, &sh_abort, a.status, 0)) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 2: wo + residual
    {
      constexpr int kind = 2;
      // merge the attention partials of every head into the staged vector
      const int S = a.nsplit;
      for (int i4 = threadIdx.x; i4 < (dim >> 2); i4 += PK_THREADS) {
        const int i = i4 << 2, h = i / hs, e = i - h * hs;
        const float* p = a.part + size_t(h) * S * (hs + 2);
        float pm[4], psum[4];
        float2 pa[4], pb[4];   // partials sit at an 8-byte (not 16-byte) aligned offset: two float2 loads
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const bool on = x < S;
          const float* px = p + x * (hs + 2);
          pm[x] = on ? __ldcg(px) : -INFINITY;
          psum[x] = on ? __ldcg(px + 1) : 0.0f;
          pa[x] = on ? __ldcg(reinterpret_cast<const float2*>(px + 2 + e)) : make_float2(0.0f, 0.0f);
          pb[x] = on ? __ldcg(reinterpret_cast<const float2*>(px + 4 + e)) : make_float2(0.0f, 0.0f);
        }
        const float M = fmaxf(fmaxf(pm[0], pm[1]), fmaxf(pm[2], pm[3]));
        float Ssum = 0.0f;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int x = 0; x < 4; ++x)
          if (pm[x] != -INFINITY) {
            const float wgt = expf(pm[x] - M);
            Ssum += psum[x] * wgt;
            v.x += pa[x].x * wgt; v.y += pa[x].y * wgt; v.z += pb[x].x * wgt; v.w += pb[x].y * wgt;
          }
        reinterpret_cast<float4*>(xs)[i4] = make_float4(v.x / Ssum, v.y / Ssum, v.z / Ssum, v.w / Ssum);
      }
      csync();
      if (!wait_weights(l, kind)) { drain(); return; }
      const int n = n_dim, r0 = r0_dim;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind]);
      const int k4 = dim >> 2;
      const float4* xv = reinterpret_cast<const float4*>(xs);
      for (int r = 2 * warp; r < n; r += 2 * PK_WARPS) {
        const float xr0 = __ldcg(a.x + r0 + r), xr1 = r + 1 < n ? __ldcg(a.x + r0 + r + 1) : 0.0f;
        if (r + 1 < n) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { a.x[r0 + r] = xr0 + v0; a.x[r0 + r + 1] = xr1 + v1; }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) a.x[r0 + r] = xr0 + v;
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(a.bar, epoch, &sh_abort, a.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 3: gate / up, silu * mul
    {
      constexpr int kind = 3;
      const float r = stage_x_rms(a.x, xs, dim, red);
      if (!wait_weights(l, kind)) { drain(); return; }
      finish_rmsnorm(xs, reinterpret_cast<const float*>(smem + a.koff[kind]), r, dim);
      const int n = n_hd, r0 = r0_hd;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind] + size_t(dim) * 4);
      const int k4 = dim >> 2;
      for (int r = warp; r < n; r += PK_WARPS) {
        float g, u;
        row_dot2(w + size_t(r) * k4, w + size_t(n + r) * k4, reinterpret_cast<const float4*>(xs), k4, lane, g, u);
        if (lane == 0) a.hb[r0 + r] = (g / (1.0f + expf(-g))) * u;
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(a.bar, epoch, &sh_abort, a.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
    // ------------------------------------------------------------------ phase 4: down + residual
    {
      constexpr int kind = 4;
      for (int i = threadIdx.x; i < (hd >> 2); i += PK_THREADS)
        reinterpret_cast<float4*>(xs)[i] = __ldcg(reinterpret_cast<const float4*>(a.hb) + i);
      csync();
      if (!wait_weights(l, kind)) { drain(); return; }
      const int n = n_dim, r0 = r0_dim;
      const float4* w = reinterpret_cast<const float4*>(smem + a.koff[kind]);
      const int k4 = hd >> 2;
      const float4* xv = reinterpret_cast<const float4*>(xs);
      for (int r = 2 * warp; r < n; r += 2 * PK_WARPS) {
        const float xr0 = __ldcg(a.x + r0 + r), xr1 = r + 1 < n ? __ldcg(a.x + r0 + r + 1) : 0.0f;
        if (r + 1 < n) {
          float v0, v1;
          row_dot2(w + size_t(r) * k4, w + size_t(r + 1) * k4, xv, k4, lane, v0, v1);
          if (lane == 0) { a.x[r0 + r] = xr0 + v0; a.x[r0 + r + 1] = xr1 + v1; }
        } else {
          const float v = row_dot(w + size_t(r) * k4, xv, k4, lane);
          if (lane == 0) a.x[r0 + r] = xr0 + v;
        }
      }
      // the barrier's leading block-wide sync also releases this kind's buffer to the producer warp
      if (!grid_sync(a.bar, epoch, &sh_abort, a.status, ptx::smem_u32(&freeb[kind]))) { drain(); return; }
    }
  }

  // ---------------------------------------------------------------------- classifier + argmax
  {
    const float r = stage_x_rms(a.x, xs, dim, red);
    finish_rmsnorm(xs, a.rms_final, r, dim);
  }
  {
    const int k4 = dim >> 2;
    const float4* xv = reinterpret_cast<const float4*>(xs);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    auto finish_row = [&](int row, float acc) {
      acc = warp_sum(acc);
      if (lane == 0) {
        a.logits[row] = acc;
        if (acc > best || (acc == best && row < best_i)) { best = acc; best_i = row; }
      }
    };
    const int row_step = G * PK_WARPS;
    if (k4 <= 8 * 32) {
      // Rows of up to 1024 elements: a lane holds a whole row slice in registers, and the next row's loads are
      // issued before the current row is reduced, so every warp always has a row in flight.
      float4 cur[8], nxt[8];
      auto load_row = [&](int row, float4 (&v)[8]) {
        const float4* wr = reinterpret_cast<const float4*>(a.wcls) + size_t(row) * k4;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          v[u] = (row < a.vocab && lane + 32 * u < k4) ? ld_stream_f4(wr + lane + 32 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      float4 xr[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) xr[u] = lane + 32 * u < k4 ? xv[lane + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
      int row = b * PK_WARPS + warp;
      load_row(row, cur);
      for (; row < a.vocab; row += row_step) {
        load_row(row + row_step, nxt);
        float acc = 0.0f;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc = fmaf(cur[u].x, xr[u].x, acc); acc = fmaf(cur[u].y, xr[u].y, acc);
          acc = fmaf(cur[u].z, xr[u].z, acc); acc = fmaf(cur[u].w, xr[u].w, acc);
        }
        finish_row(row, acc);
#pragma unroll
        for (int u = 0; u < 8; ++u) cur[u] = nxt[u];
      }
    } else {
      for (int row = b * PK_WARPS + warp; row < a.vocab; row += row_step) {
        const float4* wr = reinterpret_cast<const float4*>(a.wcls) + size_t(row) * k4;
        float acc = 0.0f;
        int i = lane;
        for (; i + 7 * 32 < k4; i += 8 * 32) {
          float4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = ld_stream_f4(wr + i + u * 32);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const float4 x4 = xv[i + u * 32];
            acc = fmaf(v[u].x, x4.x, acc); acc = fmaf(v[u].y, x4.y, acc);
            acc = fmaf(v[u].z, x4.z, acc); acc = fmaf(v[u].w, x4.w, acc);
          }
        }
        for (; i < k4; i += 32) {
          const float4 v = ld_stream_f4(wr + i), x4 = xv[i];
          acc = fmaf(v.x, x4.x, acc); acc = fmaf(v.y, x4.y, acc);
          acc = fmaf(v.z, x4.z, acc); acc = fmaf(v.w, x4.w, acc);
        }
        finish_row(row, acc);
      }
    }
    // block-level argmax (lane 0 of each warp holds a candidate)
    csync();
    if (lane == 0) { sm_m[warp] = best; reinterpret_cast<int*>(sm_s)[warp] = best_i; }
    csync();
    if (threadIdx.x == 0) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < PK_WARPS; ++w) {
        const float v = sm_m[w];
        const int i = reinterpret_cast<int*>(sm_s)[w];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      a.best_val[b] = bv;
      a.best_idx[b] = bi;
    }
  }
  if (!grid_sync(a.bar, epoch, &sh_abort, a.status, 0)) { drain(); return; }
  if (b == 0 && warp == 0) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int g = lane; g < G; g += 32) {
      const float v = __ldcg(a.best_val + g);
      const int i = __ldcg(a.best_idx + g);
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane != 0) return;
    if (bi == 0x7fffffff) bi = 0;
    const int npos = pos + 1, n_prompt = a.ctl[2];
    a.ctl[4] = bi;
    if (a.out_tokens && npos >= n_prompt) a.out_tokens[npos - n_prompt] = bi;
    a.ctl[0] = (a.prompt && npos < n_prompt) ? a.prompt[npos] : bi;
    a.ctl[1] = npos;
    a.ctl[3] = a.ctl[3] + 1;
  }
}

// ---------------------------------------------------------------------------------------------
// Shared-memory plan: one buffer per phase kind (sized for the largest row slice any block owns) followed by
// the staged-vector buffer, which doubles as the attention scratch.
struct PersistPlan {
  uint32_t koff[5];
  uint32_t xs_off;
  size_t total;
};
static PersistPlan persist_plan(const LlamaModel& m, int G) {
  const size_t dim = m.cfg.dim, hd = m.cfg.hidden_dim, kv = m.kv_dim;
  auto up = [&](size_t R) { return (R + G - 1) / G; };
  auto al = [](size_t v) { return (v + 127) & ~size_t(127); };
  const size_t bytes[5] = {(up(dim) + 2 * up(kv) + 1) * dim * 4, 0, up(dim) * dim * 4, (2 * up(hd) + 1) * dim * 4,
                           up(dim) * hd * 4};
  PersistPlan p{};
  size_t off = 0;
  for (int k = 0; k < 5; ++k) {
    p.koff[k] = uint32_t(off);
    off += al(bytes[k]);
  }
  p.xs_off = uint32_t(off);
  off += al(std::max<size_t>(std::max(dim, hd) * 4, size_t(PK_WARPS) * 128 * 4));
  p.total = off;
  return p;
}
static size_t persist_smem_bytes(const LlamaModel& m, int G) { return persist_plan(m, G).total; }

bool persistent_f32_supported(const LlamaModel& m) {
  if (m.cfg.w4 || m.tp > 1 || !ctx().ready) return false;
  const int G = ctx().sm_count;
  if (m.cfg.n_heads * 4 > G) return false;                 // one (head, split) item per block
  if (m.head_size > 128 || m.head_size % 4 || m.cfg.dim % 4 || m.cfg.hidden_dim % 4) return false;
  int coop = 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx().device) != cudaSuccess || !coop) return false;
  return persist_smem_bytes(m, G) <= PK_MAX_DYN_SMEM;
}

struct PersistScratch {
  unsigned* bar = nullptr;
  float* best_val = nullptr;
  int* best_idx = nullptr;
};
static PersistScratch g_ps;

int enqueue_token_persistent_f32(LlamaModel& m, cudaStream_t st) {
  const int G = ctx().sm_count;
  if (!g_ps.bar) {
    SIMP_CUDA(cudaMalloc(&g_ps.bar, 64));
    SIMP_CUDA(cudaMalloc(&g_ps.best_val, size_t(G) * 4));
    SIMP_CUDA(cudaMalloc(&g_ps.best_idx, size_t(G) * 4));
  }
  const simp_llama_config& c = m.cfg;
  PersistArgs a{};
  a.dim = int(c.dim); a.hd = int(c.hidden_dim); a.kv = int(m.kv_dim); a.hs = int(m.head_size);
  a.n_heads = int(c.n_heads); a.kv_mul = int(c.n_heads / c.n_kv_heads); a.n_layers = int(c.n_layers);
  a.vocab = int(c.vocab_size); a.seq_len = int(c.seq_len);
  a.nsplit = 4;
  while (a.nsplit > 1 && a.n_heads * a.nsplit > G) a.nsplit >>= 1;
  a.tok_emb = m.tok_emb; a.rms_att = m.rms_att; a.rms_ffn = m.rms_ffn; a.rms_final = m.rms_final; a.wcls = m.wcls;
  a.wq = m.wq; a.wk = m.wk; a.wv = m.wv; a.wo = m.wo; a.w1 = m.w1; a.w2 = m.w2; a.w3 = m.w3;
  a.x = m.x; a.xb = m.xb; a.hb = m.hb; a.q = m.q; a.k = m.k; a.v = m.v; a.logits = m.logits; a.kc = m.kc; a.vc = m.vc;
  a.part = m.attn_part;
  a.ctl = m.ctl; a.prompt = m.prompt; a.out_tokens = m.out_tokens;
  a.bar = g_ps.bar; a.best_val = g_ps.best_val; a.best_idx = g_ps.best_idx;
  a.status = ctx().dev_status;
  const PersistPlan plan = persist_plan(m, G);
  for (int k = 0; k < 5; ++k) a.koff[k] = plan.koff[k];
  a.xs_off = plan.xs_off;
  const size_t smem = plan.total;
  static bool attr_set = false;
  if (!attr_set) {
    SIMP_CUDA(cudaFuncSetAttribute(llama_f32_token_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(PK_MAX_DYN_SMEM)));
    attr_set = true;
  }
  SIMP_CUDA(cudaMemsetAsync(g_ps.bar, 0, 8, st));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(G));
  cfg.blockDim = dim3(PK_BLOCK);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  SIMP_CUDA(cudaLaunchKernelEx(&cfg, llama_f32_token_kernel, a));
  return SIMP_OK;
}

}  // namespace simp
