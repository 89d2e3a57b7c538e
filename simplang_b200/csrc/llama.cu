// llama.cu -- whole-token LLaMA decode on the device: the model drivers that define the f32 110M and
// W4 3B decode workloads (examples/llama2/stories110M.sl:5-247, examples/llama2/llama2_quant.sl:7-198)
// as one CUDA graph of this library's kernels per token.
//
// Per layer: rmsnorm -> q/k/v GEMV (one launch, three matrices) -> RoPE + KV-cache store ->
// decode attention (scores, softmax, weighted sum per head, split over the sequence) -> wo GEMV with
// the residual add fused -> rmsnorm -> gate/up GEMV pair with silu*mul fused -> down GEMV with the
// residual add fused; then final rmsnorm, classifier GEMV, greedy argmax (strict '>', lowest index
// wins ties as examples/llama2/generate_stories110M.cpp:73-83).  Token id and position live in device
// memory, so the same graph is replayed for every token and the host never synchronises inside a
// generation.
//
// Deviations from the .sl text (all mirrored by the CPU oracle): the score divisor is sqrt(head_size)
// rather than the literal 8.0 (identical for head_size 64); the W4 model applies RoPE like the f32
// one (the reference's W4 model has none); W4 projections use scale_mode 1 (per-matrix scale index).
#include <cuda.h>

#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "gemv_f32_core.cuh"
#include "w4_core.cuh"
#include "llama_model.hpp"

namespace simp {


// ---------------------------------------------------------------------------------------------
// x = embedding row of the current token.
// (Tensor parallel: x is a vector of tagged words, see TpLL; every rank fills its own copy, tag id 1.)
__global__ void __launch_bounds__(256) embed_kernel(float* __restrict__ x, const float* __restrict__ table,
                                                    const int* __restrict__ ctl, int dim, const TpLL tp) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t token = ctl[0];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  if (tp.n > 1) ll_store_sys(reinterpret_cast<ll_word*>(x) + i, table[token * dim + i], ll_tag_base(tp) + 1u);
  else x[i] = table[token * dim + i];
}

// rmsnorm of one row before the classifier: y = (x / sqrt(ss/n + eps)) * w (the arithmetic of rmsnorm_any_kernel).
__global__ void __launch_bounds__(1024) dec_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           float* __restrict__ y, int n, float eps, const TpLL tp, uint32_t id_x,
                                                           int* status) {
  __shared__ float red[33];
  extern __shared__ float xs_ll[];   // tensor parallel: x as it arrives (n floats)
  pdl_launch_dependents();
  const uint32_t tbase = ll_tag_base(tp);
  pdl_wait();
  float ss = 0.0f;
  if (tp.n > 1) {   // x is a vector of tagged words that the peers fill
    const uint32_t tag = tbase + id_x;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      const float v = ll_get(reinterpret_cast<const ll_word*>(x) + i, tag, status, 81);
      xs_ll[i] = v;
      ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = sqrtf(ss / float(n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) y[i] = (xs_ll[i] / r) * w[i];
    return;
  }
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
  ss = block_sum(ss, red);
  const float r = sqrtf(ss / float(n) + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) y[i] = (x[i] / r) * w[i];
}

// Decode attention of one layer in a single launch: grid (heads, nsplit), one block of 16 warps per head and
// slice of the sequence.  Built for latency (at batch 1 the kernel is a dependency chain, not a stream):
//   * everything that does not depend on this token's q/k/v happens BEFORE the wait for the projection kernel:
//     the position, the rotation angles, and asynchronous copies (cp.async, no registers held) of ALL cached K and
//     V rows of the block's slice into shared memory -- rows of earlier positions are final; they were evicted
//     from L2 by a token's worth of weights, so their HBM latency is spent while the projection still runs;
//   * RoPE on (even, odd) pairs of this head's q and k (examples/llama2/stories110M.sl:86-112:
//     freq = 1 / 10000^((i % hs)/hs), angle = pos * freq), held in shared memory; the block (split 0, first
//     head of a KV group) stores the rotated k and v into the caches at `pos` (stories110M.sl:115-121) and every
//     block whose slice holds `pos` puts them into its shared-memory rows, so no block depends on another
//     block's cache write;
//   * three short phases out of shared memory instead of an online softmax carried through every timestep (whose
//     max / exp / rescale chain every lane of a warp repeats per timestep):
//     (A) raw scores: four threads per timestep, a quarter of the head dimension each (a warp per timestep with a
//         five-step shuffle reduction took 4.3 us for 143 timesteps);
//     (B) softmax numerators, one thread per timestep: block maximum, expf, sum;
//     (C) weighted values: thread (g, i) sums p[t] * v[t][i] over t = g, g+4, ...; the four partial sums of an
//         element meet in shared memory;
//   * a slice is at most `cap` positions (what fits in shared memory, at most 256): up to there a head is ONE
//     block, which writes the normalised head output directly -- no partials in global memory, no counter, no
//     second round trip.  Longer sequences use one block per `cap` positions (at most nsplit; beyond nsplit * cap a
//     block walks its slice in rounds); their partials (m, s, acc[hs]) go to `part`, and the last block of a head
//     to finish (atomic counter, no waiting) merges them in split order.
constexpr int ATT_WARPS = 16;
constexpr int ATT_MAX_CAP = 256;
constexpr size_t ATT_SMEM_BUDGET = 200 * 1024;
inline int att_cap(int hs) {   // timesteps per block and round
  const int fit = int(ATT_SMEM_BUDGET / (size_t(hs) * 8));
  return (fit < ATT_MAX_CAP ? fit : ATT_MAX_CAP) / 16 * 16;
}
inline size_t att_smem_bytes(int hs) { return size_t(att_cap(hs)) * hs * 8; }

constexpr int ATT_BOX_ROWS = 16;   // rows per tiled load
__global__ void __launch_bounds__(ATT_WARPS * 32)
    attn_fused_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap, int use_tma,
                      const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
                      float* __restrict__ kc, float* __restrict__ vc, float* __restrict__ part, int* __restrict__ counters,
                      float* __restrict__ out, const int* __restrict__ ctl, int hs, int kv_dim, int kv_mul, int seq_len,
                      int layer, int nsplit, int cap, int* status, const TpLL tp, uint32_t id_out, uint32_t out_off
#ifdef SIMP_W4_TRACE
                      , unsigned long long* trace
#define ATT_MARK(k) do { if (trace && threadIdx.x == 0 && blockIdx.y == 0) trace[size_t(blockIdx.x) * 16 + (k)] = ptx::globaltimer_ns(); } while (0)
#else
#define ATT_MARK(k) do { } while (0)
#endif
                      ) {
  ATT_MARK(0);
  extern __shared__ __align__(128) float att_rows[];   // [cap][hs] K rows, then [cap][hs] V rows
  __shared__ __align__(8) uint64_t row_bar;
  __shared__ int abort_flag;
  __shared__ float qs[128], ks[128], vs[128];
  __shared__ float sc_s[ATT_MAX_CAP];            // scores, then softmax numerators, of the round's timesteps
  __shared__ float red_m[ATT_WARPS], red_s[ATT_WARPS];
  __shared__ float sm_acc[4][128];
  __shared__ int is_last;
  __shared__ float rc[64], rs[64];
  const int h = blockIdx.x, sp = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  const int pos = ctl[1];   // written by the previous token's last kernel, long complete
  const uint32_t tag_out = ll_tag_base(tp) + id_out;
  const int len = pos + 1;
  const int kvh = h / kv_mul;
  float* kbase = kc + int64_t(layer) * seq_len * kv_dim + kvh * hs;
  float* vbase = vc + int64_t(layer) * seq_len * kv_dim + kvh * hs;
  const int eff = min(nsplit, (len + cap - 1) / cap);
  if (sp >= eff) return;
  const int per = (len + eff - 1) / eff;
  const int t0 = sp * per, t1 = min(len, t0 + per);
  const int nrounds = (per + cap - 1) / cap;   // > 1 only when nsplit blocks of `cap` cannot cover the sequence
  float* ksm = att_rows;
  float* vsm = att_rows + size_t(cap) * hs;
  if (use_tma) {
    if (threadIdx.x == 0) {
      ptx::mbar_init(ptx::smem_u32(&row_bar), 1);
      abort_flag = 0;
      ptx::fence_barrier_init();
      ptx::prefetch_tensormap(&kmap);
      ptx::prefetch_tensormap(&vmap);
    }
    __syncthreads();
  }
  // async copies of the rows [r0, r0 + rn) (without `pos`) into shared memory; 16 bytes at a time when rows are
  // 16-byte aligned (hs % 4 == 0 and an aligned cache), else 4 bytes
  const bool vec16 = (hs & 3) == 0 && (kv_dim & 3) == 0 && ((reinterpret_cast<uintptr_t>(kbase) | reinterpret_cast<uintptr_t>(vbase)) & 15u) == 0;
  // Tiled loads (TMA) of the rows [r0, r0 + rn) of this head: boxes of ATT_BOX_ROWS rows x hs floats straight into
  // the row-major shared-memory arrays, one request per box by lane 0 of successive warps; the copy engine keeps
  // far more bytes in flight per SM than per-thread copies do (those took 8 us for 115 KB).  The box that holds
  // `pos` brings a stale row, which is overwritten after the loads have landed.
  auto fetch_rows = [&](int r0, int rn) {
    if (use_tma) {
      const int nbox = (rn + ATT_BOX_ROWS - 1) / ATT_BOX_ROWS;
      const uint32_t bar = ptx::smem_u32(&row_bar), box_bytes = uint32_t(ATT_BOX_ROWS * hs * 4);
      if (threadIdx.x == 0) ptx::mbar_arrive_expect_tx(bar, uint32_t(nbox) * 2u * box_bytes);
      if (lane == 0)
        for (int b = warp; b < nbox; b += ATT_WARPS) {
          const int y = layer * seq_len + r0 + b * ATT_BOX_ROWS;
          ptx::tma_load_2d(ptx::smem_u32(ksm) + uint32_t(b) * box_bytes, &kmap, bar, kvh * hs, y);
          ptx::tma_load_2d(ptx::smem_u32(vsm) + uint32_t(b) * box_bytes, &vmap, bar, kvh * hs, y);
        }
      return;
    }
    if (vec16) {
      const int per_row = hs >> 2, n = rn * per_row;
      for (int e = threadIdx.x; e < n; e += blockDim.x) {
        const int r = e / per_row, c4 = e - r * per_row;
        if (r0 + r == pos) continue;
        const size_t go = size_t(r0 + r) * kv_dim + c4 * 4;
        const uint32_t so = uint32_t(r * hs + c4 * 4) * 4u;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(ksm) + so), "l"(kbase + go) : "memory");
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(vsm) + so), "l"(vbase + go) : "memory");
      }
    } else {
      const int n = rn * hs;
      for (int e = threadIdx.x; e < n; e += blockDim.x) {
        const int r = e / hs, c1 = e - r * hs;
        if (r0 + r == pos) continue;
        const size_t go = size_t(r0 + r) * kv_dim + c1;
        const uint32_t so = uint32_t(r * hs + c1) * 4u;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(ksm) + so), "l"(kbase + go) : "memory");
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(vsm) + so), "l"(vbase + go) : "memory");
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch_rows(t0, min(cap, t1 - t0));   // in flight while the projection kernel finishes
  if (int(threadIdx.x) < hs / 2) {
    const int i = 2 * threadIdx.x;
    const float freq = 1.0f / powf(10000.0f, float(i) / float(hs));
    const float val = float(pos) * freq;
    rc[threadIdx.x] = cosf(val);
    rs[threadIdx.x] = sinf(val);
  }
  ATT_MARK(2);
  pdl_wait();
  ATT_MARK(3);
  if (int(threadIdx.x) < hs / 2) {
    const int i = 2 * threadIdx.x;
    const float fcr = rc[threadIdx.x], fci = rs[threadIdx.x];
    const float2 qq = __ldcg(reinterpret_cast<const float2*>(q + h * hs + i));
    const float2 kk = __ldcg(reinterpret_cast<const float2*>(k + kvh * hs + i));
    const float2 vv = __ldcg(reinterpret_cast<const float2*>(v + kvh * hs + i));
    qs[i] = qq.x * fcr - qq.y * fci;
    qs[i + 1] = qq.x * fci + qq.y * fcr;
    ks[i] = kk.x * fcr - kk.y * fci;
    ks[i + 1] = kk.x * fci + kk.y * fcr;
    vs[i] = vv.x;
    vs[i + 1] = vv.y;
  }
  __syncthreads();
  ATT_MARK(4);
  if (sp == 0 && h % kv_mul == 0) {
    for (int i = threadIdx.x; i < hs; i += blockDim.x) {
      kbase[int64_t(pos) * kv_dim + i] = ks[i];
      vbase[int64_t(pos) * kv_dim + i] = vs[i];
    }
  }
  const float div = sqrtf(float(hs));
  const int cg = threadIdx.x >> 7, ci = threadIdx.x & 127;   // phase C: group of timesteps, head element
  float acc = 0.0f;                                          // running weighted value of element ci, timesteps = cg mod 4
  float Mrun = -INFINITY, Srun = 0.0f;                       // running (max, sum) over the rounds
  for (int rd = 0; rd < nrounds; ++rd) {
    const int r0 = t0 + rd * cap;                  // first timestep of the round
    const int rn = max(0, min(cap, t1 - r0));      // timesteps in the round
    if (rd > 0) {
      __syncthreads();   // the previous round's rows and scores are no longer read
      fetch_rows(r0, rn);
    }
    if (use_tma) {
      if (!ptx::mbar_wait(ptx::smem_u32(&row_bar), uint32_t(rd) & 1u, &abort_flag, status, 70)) return;   // block-wide flag
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    ATT_MARK(7);
    // the row of `pos` comes from this token's rotated k and v
    if (pos >= r0 && pos < r0 + rn)
      for (int i = threadIdx.x; i < hs; i += blockDim.x) {
        ksm[(pos - r0) * hs + i] = ks[i];
        vsm[(pos - r0) * hs + i] = vs[i];
      }
    __syncthreads();
    // ---- (A) raw scores: four threads per timestep, each a quarter of the head dimension (row pitches of 64 or 100
    // floats keep the 32 lanes of a warp on 32 different banks), two shuffles per timestep
    {
      const int part = threadIdx.x & 3, qsz = (hs + 3) >> 2;
      const int i0 = part * qsz, i1 = min(hs, i0 + qsz);
      for (int base = 0; base < rn; base += ATT_WARPS * 8) {   // warp-uniform trip count
        const int r = base + int(threadIdx.x >> 2);
        float d = 0.0f;
        if (r < rn) {
          const float* kr = ksm + r * hs;
          for (int i = i0; i < i1; ++i) d = fmaf(qs[i], kr[i], d);
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        if (r < rn && part == 0) sc_s[r] = d / div;
      }
    }
    __syncthreads();
    ATT_MARK(8);
    // ---- (B) softmax numerators of the round: block maximum, expf, sum
    const float x = int(threadIdx.x) < rn ? sc_s[threadIdx.x] : -INFINITY;
    float mx = x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red_m[warp] = mx;
    __syncthreads();
    float M = red_m[0];
#pragma unroll
    for (int w = 1; w < ATT_WARPS; ++w) M = fmaxf(M, red_m[w]);
    const float Mnew = fmaxf(Mrun, M);
    const float pnum = int(threadIdx.x) < rn ? expf(x - Mnew) : 0.0f;
    if (int(threadIdx.x) < rn) sc_s[threadIdx.x] = pnum;
    const float ps = warp_sum(pnum);
    if (lane == 0) red_s[warp] = ps;
    __syncthreads();
    float S = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) S += red_s[w];
    const float corr = Mrun == -INFINITY ? 0.0f : expf(Mrun - Mnew);   // rescales earlier rounds
    Srun = Srun * corr + S;
    Mrun = Mnew;
    ATT_MARK(9);
    // ---- (C) weighted values
    acc *= corr;
    if (ci < hs)
      for (int r = cg; r < rn; r += 4) acc = fmaf(sc_s[r], vsm[r * hs + ci], acc);
  }
  ATT_MARK(5);
  if (ci < hs) sm_acc[cg][ci] = acc;
  __syncthreads();
  float* mine = part + (int64_t(h) * nsplit + sp) * (hs + 2);
  if (int(threadIdx.x) < hs) {
    const int i = threadIdx.x;
    const float a = (sm_acc[0][i] + sm_acc[1][i]) + (sm_acc[2][i] + sm_acc[3][i]);
    if (eff == 1) {   // the whole sequence was this block's: normalised output, done
      const float val = a / Srun;
      if (tp.n > 1) ll_store_all(tp, out_off + uint32_t(h * hs + i) * 8u, val, tag_out);   // every rank's copy
      else out[h * hs + i] = val;
    } else {
      if (i == 0) {
        mine[0] = Mrun;
        mine[1] = Srun;
      }
      mine[2 + i] = a;
    }
  }
  ATT_MARK(6);
  if (eff == 1) return;
  // last block of this head merges (writes above are published by the fence + atomic)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[h], 1) == eff - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // all partial maxima and sums are requested together, then all values of an element: one round trip each
  constexpr int MAXS = 8;   // nsplit never exceeds 8
  const float* p = part + int64_t(h) * nsplit * (hs + 2);
  float mm[MAXS], ssum[MAXS], ex[MAXS];
#pragma unroll
  for (int x2 = 0; x2 < MAXS; ++x2) {
    mm[x2] = x2 < eff ? __ldcg(p + x2 * (hs + 2)) : -INFINITY;
    ssum[x2] = x2 < eff ? __ldcg(p + x2 * (hs + 2) + 1) : 0.0f;
  }
  float M = -INFINITY;
#pragma unroll
  for (int x2 = 0; x2 < MAXS; ++x2) M = fmaxf(M, mm[x2]);
  float S = 0.0f;
#pragma unroll
  for (int x2 = 0; x2 < MAXS; ++x2) {
    ex[x2] = mm[x2] != -INFINITY ? expf(mm[x2] - M) : 0.0f;
    if (mm[x2] != -INFINITY) S += ssum[x2] * ex[x2];
  }
  for (int i = threadIdx.x; i < hs; i += blockDim.x) {
    float val[MAXS];
#pragma unroll
    for (int x2 = 0; x2 < MAXS; ++x2) val[x2] = x2 < eff ? __ldcg(p + x2 * (hs + 2) + 2 + i) : 0.0f;
    float a = 0.0f;
#pragma unroll
    for (int x2 = 0; x2 < MAXS; ++x2)
      if (mm[x2] != -INFINITY) a += val[x2] * ex[x2];
    const float res = a / S;
    if (tp.n > 1) ll_store_all(tp, out_off + uint32_t(h * hs + i) * 8u, res, tag_out);
    else out[h * hs + i] = res;
  }
  if (threadIdx.x == 0) counters[h] = 0;
}

// Greedy argmax (strict '>', lowest index wins) + bookkeeping for the next step:
// step++, pos++, token = pos < n_prompt ? prompt[pos] : argmax; generated tokens are recorded.
// ARGMAX_BLOCKS blocks each reduce a contiguous slice of the logits to one (value, index) pair; the last block to
// finish (ticket in ctl[8], reset for the next launch; nobody waits) reduces the pairs and does the bookkeeping.
constexpr int ARGMAX_BLOCKS = 32;
__device__ __forceinline__ void argmax_merge(float& best, int& idx, float ov, int oi) {
  if (ov > best || (ov == best && oi < idx)) {
    best = ov;
    idx = oi;
  }
}
__global__ void __launch_bounds__(1024) argmax_advance_kernel(const float* __restrict__ logits, int n, int* ctl,
                                                              const int32_t* __restrict__ prompt,
                                                              int32_t* __restrict__ out_tokens, float* __restrict__ part_val,
                                                              int* __restrict__ part_idx) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  __shared__ int is_last;
  pdl_launch_dependents();
  pdl_wait();
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int i0 = blockIdx.x * per, i1 = min(n, i0 + per);
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) argmax_merge(best, idx, logits[i], i);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
  if (lane == 0) {
    bv[warp] = best;
    bi[warp] = idx;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < (blockDim.x >> 5) ? bv[lane] : -INFINITY;
    idx = lane < (blockDim.x >> 5) ? bi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) {
      part_val[blockIdx.x] = best;
      part_idx[blockIdx.x] = idx;
      __threadfence();
      is_last = atomicAdd(ctl + 8, 1) == int(gridDim.x) - 1;
    }
  }
  __syncthreads();
  if (!is_last || warp != 0) return;
  __threadfence();
  best = lane < int(gridDim.x) ? __ldcg(part_val + lane) : -INFINITY;
  idx = lane < int(gridDim.x) ? __ldcg(part_idx + lane) : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
  if (lane == 0) {
    if (idx == 0x7fffffff) idx = 0;  // all-NaN logits: the host loop would keep index 0
    const int pos = ctl[1] + 1, n_prompt = ctl[2], step = ctl[3];
    ctl[4] = idx;
    if (out_tokens && pos >= n_prompt) out_tokens[pos - n_prompt] = idx;
    ctl[0] = (prompt && pos < n_prompt) ? prompt[pos] : idx;
    ctl[1] = pos;
    ctl[3] = step + 1;
    ctl[8] = 0;
    ctl[10] = ctl[10] + 1;   // tokens completed since the model was created (never reset: arrival counts build on it)
  }
}

// ---------------------------------------------------------------------------------------------
// Tensor map of a key / value cache viewed as [rows, kv_dim] f32 with boxes of ATT_BOX_ROWS rows x hs columns.
static int make_cache_map(CUtensorMap* map, const float* base, int64_t rows, int64_t kv_dim, int64_t hs) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn enc = nullptr;
  if (!enc) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      enc = reinterpret_cast<EncodeFn>(sym);
  }
  SIMP_REQUIRE(enc != nullptr, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {cuuint64_t(kv_dim), cuuint64_t(rows)};
  cuuint64_t strides[1] = {cuuint64_t(kv_dim) * 4};
  cuuint32_t box[2] = {cuuint32_t(hs), cuuint32_t(ATT_BOX_ROWS)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SIMP_REQUIRE(r == CUDA_SUCCESS, SIMP_ERR_CUDA, "cuTensorMapEncodeTiled (kv cache) failed with CUresult %d", int(r));
  return SIMP_OK;
}

static int dev_alloc(void** p, size_t bytes) {
  SIMP_CUDA(cudaMalloc(p, bytes ? bytes : 16));
  return SIMP_OK;
}

#define LAUNCH_OR_FAIL(...)                                                                         \
  do {                                                                                              \
    cudaError_t e__ = launch_kernel(__VA_ARGS__);                                                   \
    if (e__ != cudaSuccess)                                                                         \
      return set_error(SIMP_ERR_CUDA, "decode launch failed: %s (%s:%d)", cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)

// Enqueues one token.  Every launch after the first uses programmatic dependent launch: each kernel
// requests its first weights, then waits for its predecessor before touching activations.
static int enqueue_token_tp(LlamaModel& m, cudaStream_t st);
bool dist_symm_peers(const void* local, uint8_t** peers8);   // dist.cu

// Decode form on one GPU.  f32 model: the single cooperative kernel per token whenever the model fits its
// shared-memory plan, unless SIMP_DECODE_MODE=graph asks for the per-op kernels.  W4 model and tensor-parallel
// models: the per-op kernels (a cooperative W4 kernel was built and measured at 1333 us per 3B token against
// 1049 for the per-op graph of that time; it was removed).
static bool use_persistent(const LlamaModel& m) {
  const char* e = getenv("SIMP_DECODE_MODE");
  if (e && !strcmp(e, "graph")) return false;
  return !m.cfg.w4 && persistent_f32_supported(m);
}

static int enqueue_token(LlamaModel& m, cudaStream_t st) {
  const simp_llama_config& c = m.cfg;
  if (use_persistent(m)) return enqueue_token_persistent_f32(m, st);
  if (c.w4) return enqueue_token_tp(m, st);  // the per-op W4 path is shared by 1 and R ranks
  const int dim = int(c.dim), hd = int(c.hidden_dim), kv = int(m.kv_dim), hs = int(m.head_size);
  const int sms = ctx().sm_count;
  const bool pdl = true;
  LAUNCH_OR_FAIL(embed_kernel, dim3((dim + 255) / 256), dim3(256), 0, st, false, m.x, m.tok_emb, m.ctl, dim, TpLL{});
  for (int64_t l = 0; l < c.n_layers; ++l) {
    {
      GemvDecArgs g{};
      g.seg[0] = GemvSeg{m.wq + l * dim * dim, m.q, dim};
      g.seg[1] = GemvSeg{m.wk + l * int64_t(kv) * dim, m.k, kv};
      g.seg[2] = GemvSeg{m.wv + l * int64_t(kv) * dim, m.v, kv};
      g.nseg = 3; g.k4 = dim / 4; g.x = m.x; g.norm_w = m.rms_att + l * dim; g.eps = 1e-5f;
      if (int rc = gemv_f32_dec_launch<GEMV_STORE>(g, st, sms, pdl)) return rc;
    }
    LAUNCH_OR_FAIL(attn_fused_kernel, dim3(unsigned(c.n_heads), unsigned(m.nsplit)), dim3(ATT_WARPS * 32), att_smem_bytes(hs), st, pdl,
                   m.kmap, m.vmap, int(m.kv_tma), (const float*)m.q, (const float*)m.k, (const float*)m.v, m.kc, m.vc, m.attn_part, m.attn_cnt, m.xb,
                   (const int*)m.ctl, hs, kv, int(c.n_heads / c.n_kv_heads), int(c.seq_len), int(l), m.nsplit, att_cap(hs), ctx().dev_status, TpLL{}, 0u, 0u
#ifdef SIMP_W4_TRACE
                   , (unsigned long long*)nullptr
#endif
                   );
    {
      GemvDecArgs o{};
      o.seg[0] = GemvSeg{m.wo + l * dim * dim, m.x, dim};
      o.nseg = 1; o.k4 = dim / 4; o.x = m.xb;
      if (int rc = gemv_f32_dec_launch<GEMV_ACCUM>(o, st, sms, pdl)) return rc;
      GemvDecArgs g{};
      g.seg[0] = GemvSeg{m.w1 + l * int64_t(hd) * dim, m.hb, hd};
      g.seg[1] = GemvSeg{m.w3 + l * int64_t(hd) * dim, nullptr, hd};
      g.nseg = 2; g.k4 = dim / 4; g.x = m.x; g.norm_w = m.rms_ffn + l * dim; g.eps = 1e-5f;
      if (int rc = gemv_f32_dec_launch<GEMV_GATE_UP>(g, st, sms, pdl)) return rc;
      GemvDecArgs d{};
      d.seg[0] = GemvSeg{m.w2 + l * int64_t(dim) * hd, m.x, dim};
      d.nseg = 1; d.k4 = hd / 4; d.x = m.hb;
      if (int rc = gemv_f32_dec_launch<GEMV_ACCUM>(d, st, sms, pdl)) return rc;
    }
  }
  LAUNCH_OR_FAIL(dec_rmsnorm_kernel, dim3(1), dim3(1024), 0, st, pdl, (const float*)m.x, (const float*)m.rms_final, m.xb,
                 dim, 1e-5f, TpLL{}, 0u, ctx().dev_status);
  {
    GemvArgs g{};
    g.seg[0] = GemvSeg{m.wcls, m.logits, int(c.vocab_size)};
    g.nseg = 1; g.k4 = dim / 4; g.x = m.xb;
    if (int rc = gemv_f32_launch<GEMV_STORE>(g, st, sms)) return rc;
  }
  LAUNCH_OR_FAIL(argmax_advance_kernel, dim3(ARGMAX_BLOCKS), dim3(1024), 0, st, false, (const float*)m.logits,
                 int(c.vocab_size), m.ctl, (const int32_t*)m.prompt, m.out_tokens, m.pk_best_val, m.pk_best_idx);
  return SIMP_OK;
}

// W4 token, single GPU (R = 1) or tensor-parallel: every projection computes this rank's output rows from the full,
// replicated input vector, and the row slices are exchanged with in-place all-gathers.  Every projection kernel
// packs its (gathered) input vector itself and folds the preceding rmsnorm in, so each output element keeps the
// single-GPU arithmetic.
#ifdef SIMP_W4_TRACE
static unsigned long long* g_w4_trace = nullptr;   // instrumented builds: [4 projections of layer 1][148 blocks][16 marks]
#endif

static int enqueue_token_tp(LlamaModel& m, cudaStream_t st) {
  const simp_llama_config& c = m.cfg;
#ifdef SIMP_W4_TRACE
  if (!g_w4_trace) {
    cudaMalloc(&g_w4_trace, 5 * 148 * 16 * 8);
    cudaMemset(g_w4_trace, 0, 5 * 148 * 16 * 8);
  }
#define W4_TRACE_SET(args, which) (args).trace = (l == 1) ? g_w4_trace + size_t(which) * 148 * 16 : nullptr
#else
#define W4_TRACE_SET(args, which) do { } while (0)
#endif
  const int R = m.tp, rk = m.rank;
  const int dim = int(c.dim), hd = int(c.hidden_dim), kv = int(m.kv_dim), hs = int(m.head_size);
  const int dim_l = dim / R, kv_l = kv / R, hd_l = hd / R, V_l = int(c.vocab_size) / R, heads_l = int(c.n_heads) / R;
  const int sms = ctx().sm_count;
  const int log2_cpg = __builtin_ctzll(uint64_t(c.group_size / 32));
  // Tensor parallel: x, xb and hb are vectors of tagged words inside the symmetric arena; every producing kernel
  // stores its slice into every rank's copy and every consuming kernel polls its own copy (see TpLL).  No exchange
  // kernels in between, so every launch can be a programmatic dependent, as on one GPU.
  const bool chain = true;
  TpLL tp;
  if (R > 1) {
    tp.n = R; tp.rank = rk;
    for (int r = 0; r < R; ++r) tp.arena[r] = m.tp_peer[r];
    tp.tokens = m.ctl + 10;
    tp.per_token = uint32_t(4 * c.n_layers + 2);
  }
  auto arena_off = [&](const float* p) { return uint32_t(reinterpret_cast<const uint8_t*>(p) - static_cast<const uint8_t*>(m.tp_arena)); };
  // tag ids of a token: 1 = embedding; per layer: attention output, x after wo, hidden, x after down
  auto id_xb = [](int64_t l) { return uint32_t(2 + 4 * l); };
  auto id_xwo = [](int64_t l) { return uint32_t(3 + 4 * l); };
  auto id_hb = [](int64_t l) { return uint32_t(4 + 4 * l); };
  auto id_xdn = [](int64_t l) { return l < 0 ? 1u : uint32_t(5 + 4 * l); };
  // a slice of a vector that holds 4-byte floats on one GPU and 8-byte tagged words under tensor parallelism
  auto slice = [&](float* vec, int64_t first) { return R > 1 ? vec + 2 * first : vec + first; };
  LAUNCH_OR_FAIL(embed_kernel, dim3((dim + 255) / 256), dim3(256), 0, st, false, m.x, m.tok_emb, m.ctl, dim, tp);
  auto w4seg = [&](int fam, int64_t layer, int64_t rows_l, int64_t cols, float* out) {
    const int64_t o = m.loff[fam] + layer * rows_l * cols;
    return W4Seg{m.qweights + o / 2, m.scales + o / c.group_size, m.zeros ? m.zeros + o / c.group_size : nullptr, out,
                 int(rows_l)};
  };
  // weights and scales of (family, layer) as L2 prefetch regions i, i+1 of a launch's arguments
  auto next_weights = [&](W4Args& a, int i, int fam, int64_t layer, int64_t rows_l, int64_t cols) {
    if (layer >= c.n_layers || m.zeros) return;
    const int64_t o = m.loff[fam] + layer * rows_l * cols;
    a.nx_base[i] = m.qweights + o / 2;
    a.nx_bytes[i] = uint32_t(rows_l * cols / 2);
    a.nx_base[i + 1] = reinterpret_cast<const uint8_t*>(m.scales + o / c.group_size);
    a.nx_bytes[i + 1] = uint32_t(rows_l * cols / c.group_size * 4);
  };
  // input vector x; norm_w != nullptr folds rmsnorm(x, norm_w) into the projection
  auto w4args = [&](int cols, const float* x, const float* norm_w) {
    W4Args a{};
    a.cols = cols; a.log2_cpg = log2_cpg; a.groups_per_row = int(cols / c.group_size);
    a.x = x; a.mul = norm_w; a.norm = norm_w != nullptr;
    a.eps = 1e-5f; a.ss_div = float(dim);
    a.tp = tp;
    return a;
  };
  // exchange of this rank's slice [rk * n, (rk + 1) * n) of an activation vector: peer stores inside the model's
  // symmetric arena (default) or an in-place NCCL all-gather (SIMP_TP_ALLGATHER=nccl, or no arena)
  // the logits (plain floats, once per token) are gathered by the one-block peer-store exchange kernel
  auto gather_logits = [&]() -> int {
    if (R == 1) return SIMP_OK;
    return simp_dist_allgather_peer(m.tp_arena, arena_off(m.logits), size_t(V_l) * 4);
  };
#define TP_CUDA(e) do { cudaError_t e__ = (e); if (e__ != cudaSuccess) return set_error(SIMP_ERR_CUDA, "tp decode launch failed: %s", cudaGetErrorString(e__)); } while (0)
  for (int64_t l = 0; l < c.n_layers; ++l) {
    {
      W4Args a = w4args(dim, m.x, m.rms_att + l * dim);
      a.seg[0] = w4seg(0, l, dim_l, dim, m.q);
      a.seg[1] = w4seg(1, l, kv_l, dim, m.k);
      a.seg[2] = w4seg(2, l, kv_l, dim, m.v);
      a.nseg = 3;
      // the attention kernel that follows reads this layer's cached keys / values of all earlier positions; they were
      // evicted from L2 by a token's worth of weights, so this launch requests them into L2 while it streams
      a.pf_len = m.ctl + 1;
      a.pf_base[0] = reinterpret_cast<const uint8_t*>(m.kc + size_t(l) * c.seq_len * kv_l);
      a.pf_base[1] = reinterpret_cast<const uint8_t*>(m.vc + size_t(l) * c.seq_len * kv_l);
      a.pf_row_bytes = kv_l * 4;
      a.id_x = id_xdn(l - 1);
      next_weights(a, 0, 3, l, dim_l, dim);   // wo
      W4_TRACE_SET(a, 0);
      if (int rc = w4_launch<W4_STORE>(a, st, sms, chain)) return rc;
    }
    LAUNCH_OR_FAIL(attn_fused_kernel, dim3(unsigned(heads_l), unsigned(m.nsplit)), dim3(ATT_WARPS * 32), att_smem_bytes(hs), st, true,
                   m.kmap, m.vmap, int(m.kv_tma), (const float*)m.q, (const float*)m.k, (const float*)m.v, m.kc, m.vc, m.attn_part, m.attn_cnt,
                   m.xb + rk * dim_l, (const int*)m.ctl, hs, kv_l, int(c.n_heads / c.n_kv_heads), int(c.seq_len), int(l),
                   m.nsplit, att_cap(hs), ctx().dev_status, tp, id_xb(l), R > 1 ? arena_off(slice(m.xb, rk * dim_l)) : 0u
#ifdef SIMP_W4_TRACE
                   , (unsigned long long*)(l == 1 ? g_w4_trace + size_t(4) * 148 * 16 : nullptr)
#endif
                   );
    {
      W4Args a = w4args(dim, m.xb, nullptr);
      a.seg[0] = w4seg(3, l, dim_l, dim, slice(m.x, rk * dim_l));
      a.nseg = 1; a.res = slice(m.x, rk * dim_l);
      a.id_x = id_xb(l); a.id_res = id_xdn(l - 1); a.id_out = id_xwo(l);
      a.out_off = R > 1 ? arena_off(slice(m.x, rk * dim_l)) : 0u;
      next_weights(a, 0, 4, l, hd_l, dim);    // gate
      next_weights(a, 2, 6, l, hd_l, dim);    // up
      W4_TRACE_SET(a, 1);
      if (int rc = w4_launch<W4_ADD>(a, st, sms, chain)) return rc;
    }
    {
      W4Args g = w4args(dim, m.x, m.rms_ffn + l * dim);
      g.seg[0] = w4seg(4, l, hd_l, dim, slice(m.hb, rk * hd_l));
      g.seg[1] = w4seg(6, l, hd_l, dim, nullptr);
      g.nseg = 2;
      g.id_x = id_xwo(l); g.id_out = id_hb(l);
      g.out_off = R > 1 ? arena_off(slice(m.hb, rk * hd_l)) : 0u;
      next_weights(g, 0, 5, l, dim_l, hd);    // down
      W4_TRACE_SET(g, 2);
      if (int rc = w4_launch<W4_GATE_UP>(g, st, sms, chain)) return rc;
    }
    {
      W4Args d = w4args(hd, m.hb, nullptr);
      d.seg[0] = w4seg(5, l, dim_l, hd, slice(m.x, rk * dim_l));
      d.nseg = 1; d.res = slice(m.x, rk * dim_l);
      d.id_x = id_hb(l); d.id_res = id_xwo(l); d.id_out = id_xdn(l);
      d.out_off = R > 1 ? arena_off(slice(m.x, rk * dim_l)) : 0u;
      next_weights(d, 0, 0, l + 1, dim_l, dim);   // the next layer's q | k | v
      next_weights(d, 2, 1, l + 1, kv_l, dim);
      next_weights(d, 4, 2, l + 1, kv_l, dim);
      W4_TRACE_SET(d, 3);
      if (int rc = w4_launch<W4_ADD>(d, st, sms, chain)) return rc;
    }
  }
  // final rmsnorm into a plain vector (under tensor parallelism its own buffer: xb holds tagged words there)
  float* xn = R > 1 ? m.tp_xn : m.xb;
  LAUNCH_OR_FAIL(dec_rmsnorm_kernel, dim3(1), dim3(1024), R > 1 ? size_t(dim) * 4 : 0, st, chain, (const float*)m.x,
                 (const float*)m.rms_final, xn, dim, 1e-5f, tp, id_xdn(c.n_layers - 1), ctx().dev_status);
  {
    GemvArgs g{};
    g.seg[0] = GemvSeg{m.wcls, m.logits + int64_t(rk) * V_l, V_l};
    g.nseg = 1; g.k4 = dim / 4; g.x = xn;
    if (int rc = gemv_f32_launch<GEMV_STORE>(g, st, sms)) return rc;
  }
  if (int rc = gather_logits()) return rc;
  LAUNCH_OR_FAIL(argmax_advance_kernel, dim3(ARGMAX_BLOCKS), dim3(1024), 0, st, false, (const float*)m.logits,
                 int(c.vocab_size), m.ctl, (const int32_t*)m.prompt, m.out_tokens, m.pk_best_val, m.pk_best_idx);
#undef TP_CUDA
  return SIMP_OK;
}

static int ensure_graph(LlamaModel& m) {
  if (m.graph) return SIMP_OK;
  cudaStream_t st = ctx().stream;
  {
    static bool att_attr_set = false;   // the attention kernel stages its K / V rows in dynamic shared memory
    if (!att_attr_set) {
      SIMP_CUDA(cudaFuncSetAttribute(attn_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ATT_SMEM_BUDGET)));
      att_attr_set = true;
    }
  }
  // one eager pass first (sets function attributes, surfaces launch errors outside capture); it
  // rewrites the same cache row the replay will write, so it is harmless
  int ctl_save[5];
  SIMP_CUDA(cudaMemcpyAsync(ctl_save, m.ctl, sizeof(ctl_save), cudaMemcpyDeviceToHost, st));
  if (m.tp > 1)
    if (int rc = simp_dist_barrier()) return rc;   // the eager pass exchanges with the peers: start it together
  SIMP_CUDA(cudaStreamSynchronize(st));
  if (int rc = (m.tp > 1 ? enqueue_token_tp(m, st) : enqueue_token(m, st))) return rc;
  SIMP_CUDA(cudaStreamSynchronize(st));
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, ctl_save, sizeof(ctl_save), cudaMemcpyHostToDevice, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  cudaGraph_t g = nullptr;
  SIMP_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  const int rc = m.tp > 1 ? enqueue_token_tp(m, st) : enqueue_token(m, st);
  cudaError_t e = cudaStreamEndCapture(st, &g);
  if (rc != SIMP_OK) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  SIMP_REQUIRE(e == cudaSuccess, SIMP_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  {
    size_t n_nodes = 0;
    m.graph_kernels = 0;
    if (cudaGraphGetNodes(g, nullptr, &n_nodes) == cudaSuccess && n_nodes > 0) {
      std::vector<cudaGraphNode_t> nodes(n_nodes);
      if (cudaGraphGetNodes(g, nodes.data(), &n_nodes) == cudaSuccess)
        for (size_t i = 0; i < n_nodes; ++i) {
          cudaGraphNodeType t;
          if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++m.graph_kernels;
        }
    }
  }
  e = cudaGraphInstantiate(&m.graph, g, 0);
  cudaGraphDestroy(g);
  SIMP_REQUIRE(e == cudaSuccess, SIMP_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_llama_create(const simp_llama_config* cfg, void** model) {
  SIMP_REQUIRE(cfg && model, SIMP_ERR_ARG, "llama_create: null pointer");
  if (int rc = ensure_ready()) return rc;
  const simp_llama_config& c = *cfg;
  SIMP_REQUIRE(c.dim > 0 && c.hidden_dim > 0 && c.n_layers > 0 && c.n_heads > 0 && c.n_kv_heads > 0 &&
                   c.vocab_size > 0 && c.seq_len > 0,
               SIMP_ERR_ARG, "llama_create: non-positive dimension");
  SIMP_REQUIRE(c.dim % c.n_heads == 0 && c.n_heads % c.n_kv_heads == 0, SIMP_ERR_SHAPE,
               "llama_create: dim %% n_heads or n_heads %% n_kv_heads != 0");
  const int64_t hs = c.dim / c.n_heads;
  SIMP_REQUIRE(hs % 2 == 0 && hs <= 128, SIMP_ERR_SHAPE, "llama_create: head_size %lld must be even and <= 128",
               (long long)hs);
  SIMP_REQUIRE(c.dim % 4 == 0 && c.hidden_dim % 4 == 0, SIMP_ERR_SHAPE, "llama_create: dim, hidden_dim must be multiples of 4");
  if (c.w4) {
    const int64_t gs = c.group_size;
    SIMP_REQUIRE(gs == 32 || gs == 64 || gs == 128 || gs == 256 || gs == 512 || gs == 1024, SIMP_ERR_SHAPE,
                 "llama_create: W4 group_size must be 32..1024 and a power of two");
    SIMP_REQUIRE(c.dim % gs == 0 && c.hidden_dim % gs == 0 && c.dim <= 16384 && c.hidden_dim <= 16384, SIMP_ERR_SHAPE,
                 "llama_create: W4 needs dim and hidden_dim to be multiples of group_size and <= 16384");
  }
  const int tp = c.tp_size > 1 ? int(c.tp_size) : 1;
  if (tp > 1) {
    SIMP_REQUIRE(c.w4 != 0, SIMP_ERR_UNSUPPORTED, "llama_create: tensor parallelism is implemented for the W4 model only");
    SIMP_REQUIRE(tp == simp_dist_world(), SIMP_ERR_STATE, "llama_create: tp_size %d but simp_dist_init world is %d", tp,
                 simp_dist_world());
    SIMP_REQUIRE(c.n_heads % tp == 0 && c.n_kv_heads % tp == 0 && c.hidden_dim % tp == 0 && c.vocab_size % tp == 0,
                 SIMP_ERR_SHAPE, "llama_create: heads, kv heads, hidden_dim and vocab_size must be multiples of tp_size");
    SIMP_REQUIRE(((c.dim / tp) * (c.dim / c.group_size)) % 4 == 0 && ((c.hidden_dim / tp) * (c.dim / c.group_size)) % 4 == 0 &&
                     ((c.dim / tp) * (c.hidden_dim / c.group_size)) % 4 == 0,
                 SIMP_ERR_SHAPE, "llama_create: row slices leave the scale arrays misaligned (need 16-byte multiples)");
  }
  LlamaModel* m = new LlamaModel();
  m->cfg = c;
  m->tp = tp;
  m->rank = tp > 1 ? simp_dist_rank() : 0;
  m->head_size = hs;
  m->kv_dim = c.dim * c.n_kv_heads / c.n_heads;
  m->nsplit = int(c.seq_len >= 1024 ? 8 : (c.seq_len >= 256 ? 4 : 1));
  int rc = SIMP_OK;
  auto A = [&](void** p, size_t n) { if (rc == SIMP_OK) rc = dev_alloc(p, n); };
  const size_t mx = size_t(c.dim > c.hidden_dim ? c.dim : c.hidden_dim);
  if (tp > 1) {
    // the exchanged vectors live in one symmetric arena so that ranks can store their slices straight into each
    // other's copies: x, xb and hb as tagged 64-bit words (see TpLL; zero = no tag yet), the logits as plain floats
    auto al = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t o_xb = al(size_t(c.dim) * 8), o_hb = o_xb + al(size_t(c.dim) * 8), o_lg = o_hb + al(size_t(c.hidden_dim) * 8);
    const size_t total = o_lg + al(size_t(c.vocab_size) * 4);
    if (rc == SIMP_OK) rc = simp_dist_symm_alloc(total, &m->tp_arena);
    if (rc == SIMP_OK && !dist_symm_peers(m->tp_arena, m->tp_peer)) rc = set_error(SIMP_ERR_STATE, "llama_create: arena peers missing");
    if (rc == SIMP_OK) {
      // nobody may store into a peer's copy before every rank's words are zero
      if (cudaMemsetAsync(m->tp_arena, 0, total, ctx().stream) != cudaSuccess) rc = SIMP_ERR_CUDA;
      if (rc == SIMP_OK) rc = simp_dist_barrier();
      if (rc == SIMP_OK && cudaStreamSynchronize(ctx().stream) != cudaSuccess) rc = SIMP_ERR_CUDA;
    }
    if (rc == SIMP_OK) {
      uint8_t* base = static_cast<uint8_t*>(m->tp_arena);
      m->x = reinterpret_cast<float*>(base);
      m->xb = reinterpret_cast<float*>(base + o_xb);
      m->hb = reinterpret_cast<float*>(base + o_hb);
      m->logits = reinterpret_cast<float*>(base + o_lg);
      // first use of the peer exchange (logits) allocates its epoch words (a collective): here, outside any capture
      rc = simp_dist_allgather_peer(m->tp_arena, o_lg, 16);
    }
    A((void**)&m->tp_xn, size_t(c.dim) * 4);
  } else {
    A((void**)&m->x, c.dim * 4); A((void**)&m->xb, mx * 4); A((void**)&m->hb, c.hidden_dim * 4);
  }
  A((void**)&m->q, c.dim * 4); A((void**)&m->k, m->kv_dim * 4); A((void**)&m->v, m->kv_dim * 4);
  if (tp == 1) A((void**)&m->logits, c.vocab_size * 4);
  const size_t kv_bytes = size_t(c.n_layers) * c.seq_len * (m->kv_dim / tp) * 4;  // this rank's heads only
  A((void**)&m->kc, kv_bytes);
  A((void**)&m->vc, kv_bytes);
  A((void**)&m->attn_part, size_t(c.n_heads) * (m->nsplit > 4 ? m->nsplit : 4) * (hs + 2) * 4);
  A((void**)&m->attn_cnt, size_t(c.n_heads) * 4);
  A((void**)&m->ctl, 64);
  if (rc == SIMP_OK && cudaMemset(m->ctl, 0, 64) != cudaSuccess) rc = SIMP_ERR_CUDA;   // ctl[8]: argmax ticket
  A((void**)&m->pk_bar, 64);
  A((void**)&m->pk_best_val, size_t(ctx().sm_count) * 4);
  A((void**)&m->pk_best_idx, size_t(ctx().sm_count) * 4);
  if (rc == SIMP_OK) {
    // tiled loads of cache rows need 16-byte multiples everywhere: head_size and the per-rank row length % 4 == 0
    const int64_t kv_l = m->kv_dim / tp;
    memset(&m->kmap, 0, sizeof(m->kmap));
    memset(&m->vmap, 0, sizeof(m->vmap));
    m->kv_tma = hs % 4 == 0 && kv_l % 4 == 0;
    if (m->kv_tma) {
      rc = make_cache_map(&m->kmap, m->kc, c.n_layers * c.seq_len, kv_l, hs);
      if (rc == SIMP_OK) rc = make_cache_map(&m->vmap, m->vc, c.n_layers * c.seq_len, kv_l, hs);
    }
  }
  if (rc != SIMP_OK) { simp_llama_destroy(m); return rc; }
  cudaMemsetAsync(m->ctl, 0, 64, ctx().stream);
  cudaMemsetAsync(m->attn_cnt, 0, size_t(c.n_heads) * 4, ctx().stream);
  cudaMemsetAsync(m->kc, 0, kv_bytes, ctx().stream);
  cudaMemsetAsync(m->vc, 0, kv_bytes, ctx().stream);
  *model = m;
  return SIMP_OK;
}

SIMP_API int simp_llama_load(void* model, const char* name, const void* host, size_t bytes) {
  SIMP_REQUIRE(model && name && host, SIMP_ERR_ARG, "llama_load: null pointer");
  LlamaModel& m = *static_cast<LlamaModel*>(model);
  const simp_llama_config& c = m.cfg;
  const std::string n(name);
  const size_t d = c.dim, h = c.hidden_dim, L = c.n_layers, V = c.vocab_size, kv = m.kv_dim;
  void** slot = nullptr;
  size_t want = 0;
  if (n == "token_embedding") { slot = (void**)&m.tok_emb; want = V * d * 4; }
  else if (n == "rms_att_w") { slot = (void**)&m.rms_att; want = L * d * 4; }
  else if (n == "rms_ffn_w") { slot = (void**)&m.rms_ffn; want = L * d * 4; }
  else if (n == "rms_final_w") { slot = (void**)&m.rms_final; want = d * 4; }
  else if (n == "wcls") { slot = (void**)&m.wcls; want = V * d * 4; }
  else if (n == "wq") { slot = (void**)&m.wq; want = L * d * d * 4; }
  else if (n == "wk") { slot = (void**)&m.wk; want = L * kv * d * 4; }
  else if (n == "wv") { slot = (void**)&m.wv; want = L * kv * d * 4; }
  else if (n == "wo") { slot = (void**)&m.wo; want = L * d * d * 4; }
  else if (n == "w1") { slot = (void**)&m.w1; want = L * h * d * 4; }
  else if (n == "w2") { slot = (void**)&m.w2; want = L * d * h * 4; }
  else if (n == "w3") { slot = (void**)&m.w3; want = L * h * d * 4; }
  else if (n == "qweights") { slot = (void**)&m.qweights; want = bytes; }
  else if (n == "scales") { slot = (void**)&m.scales; want = bytes; }
  else if (n == "zeros") { slot = (void**)&m.zeros; want = bytes; }
  SIMP_REQUIRE(slot != nullptr, SIMP_ERR_ARG, "llama_load: unknown tensor name '%s'", name);
  SIMP_REQUIRE(bytes == want, SIMP_ERR_SHAPE, "llama_load: '%s' needs %zu bytes, got %zu", name, want, bytes);
  if (m.tp > 1 && (n == "qweights" || n == "scales" || n == "zeros" || n == "wcls")) {
    // keep this rank's rows only
    cudaStream_t st = ctx().stream;
    if (*slot) { cudaStreamSynchronize(st); cudaFree(*slot); *slot = nullptr; }
    if (n == "wcls") {
      const size_t rows_l = V / m.tp;
      if (int rc = dev_alloc(slot, rows_l * d * 4)) return rc;
      SIMP_CUDA(cudaMemcpyAsync(*slot, static_cast<const float*>(host) + size_t(m.rank) * rows_l * d, rows_l * d * 4,
                                cudaMemcpyHostToDevice, st));
    } else {
      SIMP_REQUIRE(m.offsets_set, SIMP_ERR_STATE, "llama_load: call simp_llama_set_w4_offsets before loading '%s'", name);
      const size_t fam_rows[7] = {d, kv, kv, d, h, d, h}, fam_cols[7] = {d, d, d, d, d, h, d};
      const size_t gs = size_t(c.group_size);
      size_t total_l = 0;
      for (int f = 0; f < 7; ++f) total_l += L * (fam_rows[f] / m.tp) * fam_cols[f];
      const bool is_q = n == "qweights";
      if (int rc = dev_alloc(slot, is_q ? total_l / 2 : total_l / gs * 4)) return rc;
      for (int f = 0; f < 7; ++f) {
        const size_t rows_l = fam_rows[f] / m.tp, cols = fam_cols[f];
        for (size_t l = 0; l < L; ++l) {
          const size_t src = size_t(m.off[f]) + l * fam_rows[f] * cols + size_t(m.rank) * rows_l * cols;  // elements
          const size_t dst = size_t(m.loff[f]) + l * rows_l * cols;
          const size_t cnt = rows_l * cols;
          if (is_q) {
            SIMP_REQUIRE((src + cnt) / 2 <= bytes, SIMP_ERR_SHAPE, "llama_load: qweights shorter than the offsets imply");
            SIMP_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(*slot) + dst / 2, static_cast<const uint8_t*>(host) + src / 2,
                                      cnt / 2, cudaMemcpyHostToDevice, st));
          } else {
            SIMP_REQUIRE((src + cnt) / gs * 4 <= bytes, SIMP_ERR_SHAPE, "llama_load: '%s' shorter than the offsets imply", name);
            SIMP_CUDA(cudaMemcpyAsync(static_cast<float*>(*slot) + dst / gs, static_cast<const float*>(host) + src / gs,
                                      cnt / gs * 4, cudaMemcpyHostToDevice, st));
          }
        }
      }
    }
    SIMP_CUDA(cudaStreamSynchronize(st));
    if (m.graph) { cudaGraphExecDestroy(m.graph); m.graph = nullptr; }
    return SIMP_OK;
  }
  if (*slot) { cudaStreamSynchronize(ctx().stream); cudaFree(*slot); *slot = nullptr; }
  if (int rc = dev_alloc(slot, bytes)) return rc;
  SIMP_CUDA(cudaMemcpyAsync(*slot, host, bytes, cudaMemcpyHostToDevice, ctx().stream));
  SIMP_CUDA(cudaStreamSynchronize(ctx().stream));
  if (m.graph) { cudaGraphExecDestroy(m.graph); m.graph = nullptr; }
  return SIMP_OK;
}

SIMP_API int simp_llama_set_w4_offsets(void* model, const int64_t* offsets7) {
  SIMP_REQUIRE(model && offsets7, SIMP_ERR_ARG, "llama_set_w4_offsets: null pointer");
  LlamaModel& m = *static_cast<LlamaModel*>(model);
  for (int i = 0; i < 7; ++i) {
    SIMP_REQUIRE(offsets7[i] >= 0 && offsets7[i] % m.cfg.group_size == 0 && offsets7[i] % 32 == 0, SIMP_ERR_SHAPE,
                 "llama_set_w4_offsets: offset %d (%lld) must be a multiple of group_size and of 32", i,
                 (long long)offsets7[i]);
    m.off[i] = offsets7[i];
  }
  if (m.tp > 1) {
    const int64_t d = m.cfg.dim, h = m.cfg.hidden_dim, kv = m.kv_dim, L = m.cfg.n_layers;
    const int64_t fam_rows[7] = {d, kv, kv, d, h, d, h}, fam_cols[7] = {d, d, d, d, d, h, d};
    int64_t acc = 0;
    for (int f = 0; f < 7; ++f) {
      m.loff[f] = acc;
      acc += L * (fam_rows[f] / m.tp) * fam_cols[f];
    }
  } else {
    for (int i = 0; i < 7; ++i) m.loff[i] = m.off[i];
  }
  m.offsets_set = true;
  if (m.graph) { cudaGraphExecDestroy(m.graph); m.graph = nullptr; }
  return SIMP_OK;
}

static int check_loaded(const LlamaModel& m) {
  const bool common = m.tok_emb && m.rms_att && m.rms_ffn && m.rms_final && m.wcls;
  const bool proj = m.cfg.w4 ? (m.qweights && m.scales) : (m.wq && m.wk && m.wv && m.wo && m.w1 && m.w2 && m.w3);
  SIMP_REQUIRE(common && proj, SIMP_ERR_STATE, "llama: not all tensors are loaded");
  SIMP_REQUIRE(!m.cfg.w4 || m.offsets_set, SIMP_ERR_STATE, "llama: call simp_llama_set_w4_offsets for the W4 model");
  return SIMP_OK;
}

SIMP_API int simp_llama_forward(void* model, int64_t token, int64_t pos, float* logits_host) {
  SIMP_REQUIRE(model != nullptr, SIMP_ERR_ARG, "llama_forward: null model");
  LlamaModel& m = *static_cast<LlamaModel*>(model);
  SIMP_REQUIRE(token >= 0 && token < m.cfg.vocab_size && pos >= 0 && pos < m.cfg.seq_len, SIMP_ERR_ARG,
               "llama_forward: token %lld or pos %lld out of range", (long long)token, (long long)pos);
  if (int rc = check_loaded(m)) return rc;
  cudaStream_t st = ctx().stream;
  const int ctl[5] = {int(token), int(pos), 0, 0, 0};
  if (m.out_tokens || m.prompt) {  // a forward() is not part of a generation: detach the buffers
    cudaStreamSynchronize(st);
    cudaFree(m.out_tokens); cudaFree(m.prompt);
    m.out_tokens = nullptr; m.prompt = nullptr; m.out_cap = m.prompt_cap = 0;
    if (m.graph) { cudaGraphExecDestroy(m.graph); m.graph = nullptr; }
  }
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, ctl, sizeof(ctl), cudaMemcpyHostToDevice, st));
  if (int rc = ensure_graph(m)) return rc;
  if (m.tp > 1)
    if (int rc = simp_dist_barrier()) return rc;
  SIMP_CUDA(cudaGraphLaunch(m.graph, st));
  if (logits_host)
    SIMP_CUDA(cudaMemcpyAsync(logits_host, m.logits, size_t(m.cfg.vocab_size) * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  return simp_gpu_check_device_status();
}

// Teacher-forces `prompt` (positions 0..n_prompt-1), then generates n_new tokens greedily.
// tokens_out[n_new] receives the generated ids; logits_trace (optional, host) receives the logits of
// every step, (n_prompt + n_new - 1) x vocab.  ms_out (optional) = device time of the whole generation.
SIMP_API int simp_llama_generate(void* model, const int32_t* prompt, int64_t n_prompt, int64_t n_new,
                                 int32_t* tokens_out, float* logits_trace, float* ms_out) {
  SIMP_REQUIRE(model && prompt && tokens_out, SIMP_ERR_ARG, "llama_generate: null pointer");
  LlamaModel& m = *static_cast<LlamaModel*>(model);
  SIMP_REQUIRE(n_prompt >= 1 && n_new >= 1 && n_prompt + n_new - 1 <= m.cfg.seq_len, SIMP_ERR_ARG,
               "llama_generate: need n_prompt >= 1, n_new >= 1, n_prompt + n_new - 1 <= seq_len");
  for (int64_t i = 0; i < n_prompt; ++i)
    SIMP_REQUIRE(prompt[i] >= 0 && prompt[i] < m.cfg.vocab_size, SIMP_ERR_ARG, "llama_generate: prompt token out of range");
  if (int rc = check_loaded(m)) return rc;
  cudaStream_t st = ctx().stream;
  if (m.prompt_cap < n_prompt || m.out_cap < n_new) {
    cudaStreamSynchronize(st);
    cudaFree(m.prompt); cudaFree(m.out_tokens);
    m.prompt = nullptr; m.out_tokens = nullptr;
    m.prompt_cap = n_prompt > 64 ? n_prompt : 64;
    m.out_cap = n_new > 2048 ? n_new : 2048;
    if (int rc = dev_alloc((void**)&m.prompt, size_t(m.prompt_cap) * 4)) return rc;
    if (int rc = dev_alloc((void**)&m.out_tokens, size_t(m.out_cap) * 4)) return rc;
    if (m.graph) { cudaGraphExecDestroy(m.graph); m.graph = nullptr; }
  }
  SIMP_CUDA(cudaMemcpyAsync(m.prompt, prompt, size_t(n_prompt) * 4, cudaMemcpyHostToDevice, st));
  const int ctl[5] = {int(prompt[0]), 0, int(n_prompt), 0, 0};
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, ctl, sizeof(ctl), cudaMemcpyHostToDevice, st));
  if (int rc = ensure_graph(m)) return rc;
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, ctl, sizeof(ctl), cudaMemcpyHostToDevice, st));
  // Tensor parallel: the ranks meet on the host side of the stream before the tokens start, so that the bounded
  // device-side waits of the exchange only ever cover kernel skew, not a rank that is still loading or capturing.
  if (m.tp > 1)
    if (int rc = simp_dist_barrier()) return rc;
  const int64_t steps = n_prompt + n_new - 1;
  cudaEvent_t e0, e1;
  SIMP_CUDA(cudaEventCreate(&e0));
  SIMP_CUDA(cudaEventCreate(&e1));
  SIMP_CUDA(cudaEventRecord(e0, st));
  for (int64_t s = 0; s < steps; ++s) {
    SIMP_CUDA(cudaGraphLaunch(m.graph, st));
    if (logits_trace)
      SIMP_CUDA(cudaMemcpyAsync(logits_trace + s * m.cfg.vocab_size, m.logits, size_t(m.cfg.vocab_size) * 4,
                                cudaMemcpyDeviceToHost, st));
  }
  SIMP_CUDA(cudaEventRecord(e1, st));
  SIMP_CUDA(cudaMemcpyAsync(tokens_out, m.out_tokens, size_t(n_new) * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  if (ms_out) SIMP_CUDA(cudaEventElapsedTime(ms_out, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return simp_gpu_check_device_status();   // a bounded device-side wait that gave up makes the tokens meaningless
}

SIMP_API int simp_llama_kernels_per_token(void* model, int64_t* kernels) {
  SIMP_REQUIRE(model && kernels, SIMP_ERR_ARG, "llama_kernels_per_token: null pointer");
  LlamaModel& m = *static_cast<LlamaModel*>(model);
  SIMP_REQUIRE(m.graph != nullptr, SIMP_ERR_STATE, "llama_kernels_per_token: no token graph yet (run forward or generate first)");
  *kernels = m.graph_kernels;
  return SIMP_OK;
}

SIMP_API int simp_llama_destroy(void* model) {
  if (!model) return SIMP_OK;
  LlamaModel* m = static_cast<LlamaModel*>(model);
  if (ctx().ready) cudaStreamSynchronize(ctx().stream);
  if (m->graph) cudaGraphExecDestroy(m->graph);
  if (m->tp_arena) {   // x, xb, hb and logits live inside the symmetric arena
    simp_dist_symm_free(m->tp_arena);
    m->x = m->xb = m->hb = m->logits = nullptr;
  }
  void* ptrs[] = {m->tok_emb, m->rms_att, m->rms_ffn, m->rms_final, m->wcls, m->wq, m->wk, m->wv, m->wo, m->w1, m->w2,
                  m->w3, m->qweights, m->scales, m->zeros, m->x, m->xb, m->hb, m->q, m->k, m->v, m->logits, m->kc,
                  m->vc, m->attn_part, m->attn_cnt, m->ctl, m->prompt, m->out_tokens,
                  m->pk_bar, m->pk_best_val, m->pk_best_idx, m->tp_xn};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  delete m;
  return SIMP_OK;
}

#ifdef SIMP_W4_TRACE
SIMP_API int simp_debug_w4_trace(unsigned long long* host_out, size_t words) {
  SIMP_REQUIRE(simp::g_w4_trace != nullptr, SIMP_ERR_STATE, "no trace yet");
  SIMP_CUDA(cudaMemcpy(host_out, simp::g_w4_trace, words * 8, cudaMemcpyDeviceToHost));
  return SIMP_OK;
}
#endif
