// llama_persistent.cuh -- pieces shared by the persistent per-token decode kernels (f32 weights:
// llama_persistent.cu, W4 weights: llama_persistent_w4.cu): the compute-warp barrier, the bounded grid
// barrier, the attention phase, the merge of its sequence splits, the classifier + greedy argmax.
//
// Block shape of both kernels: PK_WARPS compute warps followed by one producer warp that only requests
// weights.  Everything here is called by the compute warps (threadIdx.x < PK_THREADS).
#pragma once
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace simp {

constexpr int PK_THREADS = 512;
constexpr int PK_WARPS = PK_THREADS / 32;
constexpr int PK_BLOCK = PK_THREADS + 32;   // 16 compute warps + 1 producer warp (weight requests)
constexpr uint32_t PK_COPY_CHUNK = 16384;   // bytes per bulk copy request
constexpr size_t PK_SMEM_LIMIT = 227 * 1024;

// Model geometry and device state both kernels use.
struct PkCommon {
  int dim, hd, kv, hs, n_heads, kv_mul, n_layers, vocab, seq_len, nsplit;
  const float *tok_emb, *rms_att, *rms_ffn, *rms_final, *wcls;
  float *x, *hb, *q, *k, *v, *logits, *kc, *vc, *part;
  int* ctl;
  const int32_t* prompt;
  int32_t* out_tokens;
  unsigned* bar;    // [0] arrivals, [1] error word
  float* best_val;  // per-block argmax partials
  int* best_idx;
  int* status;      // library-wide device status word
};

// Small statically sized shared state of a block.
struct PkStatic {
  float red[33];
  int sh_abort, prod_done;
  float sm_m[PK_WARPS], sm_s[PK_WARPS];
  float qs[128], ks[128], vs[128];
  int halves[2][4 * PK_WARPS];   // int8 kernel: partial row sums of two warps sharing a row (double-buffered by tile)
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

// Attention of layer l for this block's (head, sequence split) item, if it has one: RoPE on q and k, the new
// K/V row stored to the cache, online softmax over the split's timesteps (16 warps, 4 timesteps in flight
// each), the (max, sum, weighted V) partial written to c.part.  sm_acc: PK_WARPS x 128 floats of scratch.
__device__ __forceinline__ void pk_attention(const PkCommon& c, PkStatic& S, float* sm_acc, int l, int pos) {
  const int b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hs = c.hs, kv = c.kv;
  const int NS = c.nsplit;
  if (b < c.n_heads * NS) {
    const int h = b / NS, sp = b % NS, kvh = h / c.kv_mul;
    if (int(threadIdx.x) < hs / 2) {
      const int i = 2 * threadIdx.x;
      const float freq = 1.0f / powf(10000.0f, float(i) / float(hs));
      const float val = float(pos) * freq;
      const float fcr = cosf(val), fci = sinf(val);
      const float q0 = __ldcg(c.q + h * hs + i), q1 = __ldcg(c.q + h * hs + i + 1);
      S.qs[i] = q0 * fcr - q1 * fci;
      S.qs[i + 1] = q0 * fci + q1 * fcr;
      const float k0 = __ldcg(c.k + kvh * hs + i), k1 = __ldcg(c.k + kvh * hs + i + 1);
      S.ks[i] = k0 * fcr - k1 * fci;
      S.ks[i + 1] = k0 * fci + k1 * fcr;
      S.vs[i] = __ldcg(c.v + kvh * hs + i);
      S.vs[i + 1] = __ldcg(c.v + kvh * hs + i + 1);
    }
    csync();
    float* kbase = c.kc + size_t(l) * c.seq_len * kv + kvh * hs;
    float* vbase = c.vc + size_t(l) * c.seq_len * kv + kvh * hs;
    if (sp == 0 && h % c.kv_mul == 0)
      for (int i = threadIdx.x; i < hs; i += PK_THREADS) {
        kbase[size_t(pos) * kv + i] = S.ks[i];
        vbase[size_t(pos) * kv + i] = S.vs[i];
      }
    const int len = pos + 1, per = (len + NS - 1) / NS;
    const int t0 = sp * per, t1 = min(len, t0 + per);
    const float div = sqrtf(float(hs));
    float qr[4], acc[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = lane + 32 * e;
      qr[e] = i < hs ? S.qs[i] : 0.0f;
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
            if (t == pos) { kr[u][e] = S.ks[i]; vr[u][e] = S.vs[i]; }
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
    if (lane == 0) { S.sm_m[warp] = m; S.sm_s[warp] = s; }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = lane + 32 * e;
      if (i < hs) sm_acc[warp * 128 + i] = acc[e];
    }
    csync();
    float* mine = c.part + (size_t(h) * NS + sp) * (hs + 2);
    if (warp == 0) {
      // lane w holds warp w's running maximum; one expf per lane, broadcast by shuffle
      const float mw = lane < PK_WARPS ? S.sm_m[lane] : -INFINITY;
      float M = mw;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
      const float scl = mw == -INFINITY ? 0.0f : expf(mw - M);
      float sc[PK_WARPS];
#pragma unroll
      for (int w = 0; w < PK_WARPS; ++w) sc[w] = __shfl_sync(0xffffffffu, scl, w);
      float Ssum = 0.0f;
#pragma unroll
      for (int w = 0; w < PK_WARPS; ++w) Ssum += S.sm_s[w] * sc[w];
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
}

// Merges the sequence splits of every head into the normalised attention output (dim floats at `out`,
// shared memory).  head_size must be a multiple of 4.
__device__ __forceinline__ void pk_merge_heads(const PkCommon& c, float* out) {
  const int dim = c.dim, hs = c.hs;
    const int S = c.nsplit;
  for (int i4 = threadIdx.x; i4 < (dim >> 2); i4 += PK_THREADS) {
    const int i = i4 << 2, h = i / hs, e = i - h * hs;
    const float* p = c.part + size_t(h) * S * (hs + 2);
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
    reinterpret_cast<float4*>(out)[i4] = make_float4(v.x / Ssum, v.y / Ssum, v.z / Ssum, v.w / Ssum);
  }
}

// Classifier rows streamed from HBM against the normalised vector xs (shared), logits stored, and this
// block's argmax candidate (strict '>', lowest index wins) written to c.best_val / c.best_idx.
__device__ __forceinline__ void pk_classifier(const PkCommon& c, PkStatic& S, const float* xs) {
  const int G = gridDim.x, b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dim = c.dim;
  {
    const int k4 = dim >> 2;
    const float4* xv = reinterpret_cast<const float4*>(xs);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    auto finish_row = [&](int row, float acc) {
      acc = warp_sum(acc);
      if (lane == 0) {
        c.logits[row] = acc;
        if (acc > best || (acc == best && row < best_i)) { best = acc; best_i = row; }
      }
    };
    const int row_step = G * PK_WARPS;
    if (k4 <= 8 * 32) {
      // Rows of up to 1024 elements: a lane holds a whole row slice in registers, and the next row's loads are
      // issued before the current row is reduced, so every warp always has a row in flight.
      float4 cur[8], nxt[8];
      auto load_row = [&](int row, float4 (&v)[8]) {
        const float4* wr = reinterpret_cast<const float4*>(c.wcls) + size_t(row) * k4;
#pragma unroll
        for (int u = 0; u < 8; ++u)
          v[u] = (row < c.vocab && lane + 32 * u < k4) ? ld_stream_f4(wr + lane + 32 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
      };
      float4 xr[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) xr[u] = lane + 32 * u < k4 ? xv[lane + 32 * u] : make_float4(0.f, 0.f, 0.f, 0.f);
      int row = b * PK_WARPS + warp;
      load_row(row, cur);
      for (; row < c.vocab; row += row_step) {
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
      for (int row = b * PK_WARPS + warp; row < c.vocab; row += row_step) {
        const float4* wr = reinterpret_cast<const float4*>(c.wcls) + size_t(row) * k4;
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
    if (lane == 0) { S.sm_m[warp] = best; reinterpret_cast<int*>(S.sm_s)[warp] = best_i; }
    csync();
    if (threadIdx.x == 0) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int w = 0; w < PK_WARPS; ++w) {
        const float v = S.sm_m[w];
        const int i = reinterpret_cast<int*>(S.sm_s)[w];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      c.best_val[b] = bv;
      c.best_idx[b] = bi;
    }
  }
}

// After the last grid barrier: block 0 reduces the per-block candidates and advances the control words
// (step++, pos++, token = pos < n_prompt ? prompt[pos] : argmax; generated tokens are recorded).
__device__ __forceinline__ void pk_advance(const PkCommon& c, int pos) {
  const int G = gridDim.x, b = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (b == 0 && warp == 0) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int g = lane; g < G; g += 32) {
      const float v = __ldcg(c.best_val + g);
      const int i = __ldcg(c.best_idx + g);
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
    const int npos = pos + 1, n_prompt = c.ctl[2];
    c.ctl[4] = bi;
    if (c.out_tokens && npos >= n_prompt) c.out_tokens[npos - n_prompt] = bi;
    c.ctl[0] = (c.prompt && npos < n_prompt) ? c.prompt[npos] : bi;
    c.ctl[1] = npos;
    c.ctl[3] = c.ctl[3] + 1;
  }
}

// Host side (llama_persistent.cu): fills PkCommon from a model; checks what both kernels need of the
// device and the model; zeroes the barrier words and launches a kernel cooperatively, one block per SM.
struct LlamaModel;
int pk_fill_common(LlamaModel& m, PkCommon& c);
bool pk_device_ok(const LlamaModel& m);
int pk_launch(const void* kernel, void* args_struct, unsigned* bar, size_t smem, cudaStream_t st);

}  // namespace simp
