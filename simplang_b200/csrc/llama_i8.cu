// llama_i8.cu -- token forward of the int8 LLaMA-3.2-1B-style model
// (examples/llama2/llama32_1b_int8_tensor.sl:16-305): f32 residual stream and norms, int8 activations,
// int8 weights pre-transposed [N, K] with i32 accumulation (tensor_matmul_nt at M = 1), int8 KV cache,
// grouped-query attention, f32 classifier.  One CUDA graph per token, programmatic dependent launch
// between the kernels; the position lives in device memory.
//
// Kernels per layer (5):
//   gemv_i8_kernel<PRO_NORM, EPI_STORE>   rmsnorm + quantise folded into the prologue, q | k | v rows (i32)
//   attn_i8_kernel                        KV store (acc / 256 -> i8), scores / 8.0, softmax, weighted sum,
//                                         (i32) trunc, requantise clamp(v / 256.0) -> i8
//   gemv_i8_kernel<PRO_I8, EPI_RESID>     wo: x += (f32)acc / 65536
//   gemv_i8_kernel<PRO_NORM, EPI_GATEUP>  w1 | w3 pairs: (i8)(silu(g / 65536) * (u / 65536) * 127), no clamp
//   gemv_i8_kernel<PRO_I8, EPI_RESID>     w2: x += (f32)acc / 65536
// The GEMV is a streaming kernel (HBM-bound: every weight byte is read once per token): a warp owns RPW
// rows, lanes read 16-byte pieces of the K-contiguous rows with no-allocate loads, four independent
// pieces per row in flight, dp4a.s32.s32 against the int8 input vector staged in shared memory, one
// shuffle reduction per row.  Integer accumulation is exact, so q, k, v, wo, gate, up and down match the CPU
// reference bit for bit whenever their int8 inputs do; differences can only enter through the f32 sums of
// the norms and of the attention (different summation order) at a quantisation boundary.
#include <algorithm>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "gemv_f32_core.cuh"
#include "llama_i8_model.hpp"

namespace simp {

enum { PRO_NORM = 0, PRO_I8 = 1 };
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_GATEUP = 2 };
constexpr int GI8_WARPS = 8;

struct GemvI8Seg {
  const int8_t* w;   // [rows, K]
  int32_t* out;      // EPI_STORE
  int rows;
};
struct GemvI8Args {
  GemvI8Seg seg[3];
  int nseg, K;
  const float* x_f32;     // PRO_NORM: vector to normalise; EPI_RESID: residual stream (updated in place)
  const float* norm_w;    // PRO_NORM
  const int8_t* x_i8;     // PRO_I8
  float* resid;           // EPI_RESID: x[row] += acc / 65536
  int8_t* hb;             // EPI_GATEUP: seg[0] = w1, seg[1] = w3
  int total_rows;         // rows over all segments (EPI_GATEUP: rows of one matrix)
};

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
// f32 -> i8 as the model text does it: clamp to [-128, 127], truncate toward zero.
__device__ __forceinline__ int8_t quant_clamped(float v) {
  v = fminf(v, 127.0f);
  v = fmaxf(v, -128.0f);
  return int8_t(__float2int_rz(v));
}

template <int PRO, int EPI, int RPW>
__global__ void __launch_bounds__(GI8_WARPS * 32) gemv_i8_kernel(const GemvI8Args a) {
  extern __shared__ __align__(16) uint8_t gi8_smem[];   // K int8 inputs
  __shared__ float red[33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = a.K, k16 = K >> 4;
  constexpr int NM = EPI == EPI_GATEUP ? 2 : 1;
  constexpr int U = 4;   // 16-byte pieces per row in flight per lane
  pdl_launch_dependents();
  // rows of this warp: (segment, row) pairs; a warp's RPW rows never straddle segments when every segment's
  // row count is a multiple of RPW (checked on the host)
  const int row0 = (blockIdx.x * GI8_WARPS + warp) * RPW;
  const bool active = row0 < a.total_rows;
  int s = 0, r_in = row0;
  if (EPI != EPI_GATEUP)
    while (s + 1 < a.nseg && r_in >= a.seg[s].rows) { r_in -= a.seg[s].rows; ++s; }
  const uint4* wrow[NM][RPW];
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int r = 0; r < RPW; ++r)
      wrow[m][r] = reinterpret_cast<const uint4*>(a.seg[EPI == EPI_GATEUP ? m : s].w + size_t(active ? r_in + r : 0) * K);
  uint4 w[NM][RPW][U];
  auto load_batch = [&](int j0) {
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
      for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int j = j0 + 32 * u;
          w[m][r][u] = (active && j < k16) ? ldg_stream_u4(wrow[m][r] + j) : make_uint4(0u, 0u, 0u, 0u);
        }
  };
  // Weights never change: the first pieces of every row are requested before waiting for the producer of the
  // input vector, so they stream in under the predecessor's tail and under the prologue below.
  load_batch(lane);
  // ... and so are the norm weights (first NW_REG per thread; longer vectors read the rest after the wait)
  constexpr int NW_REG = 8;
  float nw[NW_REG];
  if (PRO == PRO_NORM) {
#pragma unroll
    for (int u = 0; u < NW_REG; ++u) {
      const int i = threadIdx.x + u * (GI8_WARPS * 32);
      nw[u] = i < K ? __ldg(a.norm_w + i) : 0.0f;
    }
  }
  pdl_wait();
  // residual rows are requested now so that their latency is not paid in the epilogue (lane r holds row r's)
  float resid_pre = 0.0f;
  if (EPI == EPI_RESID && active && lane < RPW) resid_pre = __ldcg(a.resid + r_in + lane);
  // ---- prologue: the int8 input vector in shared memory
  if (PRO == PRO_NORM) {
    // y = (x / r) * w, r = sqrt(mean(x^2) + 1e-5); v = y * 127 clamped, truncated (llama32_1b_int8_tensor.sl:93-103)
    float xr[NW_REG];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < NW_REG; ++u) {
      const int i = threadIdx.x + u * (GI8_WARPS * 32);
      xr[u] = i < K ? a.x_f32[i] : 0.0f;
      ss += xr[u] * xr[u];
    }
    for (int i = threadIdx.x + NW_REG * (GI8_WARPS * 32); i < K; i += blockDim.x) {
      const float t = a.x_f32[i];
      ss += t * t;
    }
    ss = block_sum(ss, red);
    const float r = sqrtf(ss / float(K) + 1e-5f);
#pragma unroll
    for (int u = 0; u < NW_REG; ++u) {
      const int i = threadIdx.x + u * (GI8_WARPS * 32);
      if (i < K) reinterpret_cast<int8_t*>(gi8_smem)[i] = quant_clamped(((xr[u] / r) * nw[u]) * 127.0f);
    }
    for (int i = threadIdx.x + NW_REG * (GI8_WARPS * 32); i < K; i += blockDim.x)
      reinterpret_cast<int8_t*>(gi8_smem)[i] = quant_clamped(((a.x_f32[i] / r) * a.norm_w[i]) * 127.0f);
  } else {
    for (int i = threadIdx.x; i < k16; i += blockDim.x)
      reinterpret_cast<uint4*>(gi8_smem)[i] = reinterpret_cast<const uint4*>(a.x_i8)[i];
  }
  __syncthreads();
  if (!active) return;
  const uint4* xs = reinterpret_cast<const uint4*>(gi8_smem);
  int acc[NM][RPW];
#pragma unroll
  for (int m = 0; m < NM; ++m)
#pragma unroll
    for (int r = 0; r < RPW; ++r) acc[m][r] = 0;
  for (int j0 = lane; j0 < k16; j0 += 32 * U) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = j0 + 32 * u;
      const uint4 xv = j < k16 ? xs[j] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
          int t = acc[m][r];
          t = dp4a_ss(w[m][r][u].x, xv.x, t);
          t = dp4a_ss(w[m][r][u].y, xv.y, t);
          t = dp4a_ss(w[m][r][u].z, xv.z, t);
          t = dp4a_ss(w[m][r][u].w, xv.w, t);
          acc[m][r] = t;
        }
    }
    if (j0 + 32 * U < k16) load_batch(j0 + 32 * U);
  }
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    int v0 = acc[0][r], v1 = NM == 2 ? acc[NM - 1][r] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      v0 += __shfl_xor_sync(0xffffffffu, v0, o);
      if (NM == 2) v1 += __shfl_xor_sync(0xffffffffu, v1, o);
    }
    const float resid_r = __shfl_sync(0xffffffffu, resid_pre, r);
    if (lane == 0) {
      const int row = r_in + r;
      if (EPI == EPI_STORE) a.seg[s].out[row] = v0;
      if (EPI == EPI_RESID) a.resid[row] = resid_r + float(v0) / 65536.0f;
      if (EPI == EPI_GATEUP) {
        const float gate_f = float(v0) / 65536.0f;
        const float silu = gate_f / (1.0f + expf(0.0f - gate_f));
        const float up_f = float(v1) / 65536.0f;
        float hb = silu * up_f * 127.0f;
        hb = fmaxf(fminf(hb, 2147483520.0f), -2147483648.0f);   // keeps the conversion defined
        a.hb[row] = int8_t(uint8_t(uint32_t(__float2int_rz(hb)) & 0xffu));
      }
    }
  }
}

// x_f32[i] = (f32) x_i8[i]  (llama32_1b_int8_tensor.sl:78-82)
__global__ void i8_input_kernel(const int8_t* __restrict__ x_i8, float* __restrict__ x, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] = float(x_i8[i]) * 1.0f;
}

// Attention of one layer (llama32_1b_int8_tensor.sl:142-215): grid (query heads, sequence splits).
// The new K/V row is derived by every block from the i32 projections (so no block depends on another block's
// cache write); split 0 of the first head of each KV group stores it.  A cache row of head_dim int8 values is
// read as 16-byte pieces: a lane owns (timestep within a group of 32 / pieces, piece), converts to f32 and
// multiplies as the model text does -- scores[t] = sum_d f32(q_d) * f32(k_td) / 8.0 -- then the split's
// exp-weights and weighted V sums are formed; the block that arrives last for its head merges the splits
// (online-softmax algebra), truncates to i32 (attn_out) and requantises clamp(out / 256.0) for the next
// projection.  With one split the arithmetic is p = e / sum, out = sum_t p_t * v_t as in the text.
constexpr int AI8_WARPS = 8;
constexpr int AI8_MAX_SPLITS = 16;
__global__ void __launch_bounds__(AI8_WARPS * 32) attn_i8_kernel(const int32_t* __restrict__ Q, const int32_t* __restrict__ Kp,
                                                                  const int32_t* __restrict__ Vp, int8_t* __restrict__ kc,
                                                                  int8_t* __restrict__ vc, int8_t* __restrict__ xb_i8,
                                                                  float* __restrict__ part, int* __restrict__ counters,
                                                                  const int* __restrict__ ctl, int hs, int kv_dim, int n_rep,
                                                                  int max_seq, int layer, int nsplit) {
  extern __shared__ float scores[];   // timesteps of this split
  __shared__ float qf[128], knew[128], vnew[128], red[33];
  __shared__ float wpart[AI8_WARPS][128];
  __shared__ bool is_last;
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, sp = blockIdx.y, kvh = h / n_rep;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = ctl[0], seq = pos + 1;
  // splits actually used: one per 64 positions of the current context, so short contexts do not pay for the
  // merge of up to 16 nearly empty splits; the blocks of unused splits leave at once
  nsplit = min(nsplit, (seq + 63) / 64);
  if (sp >= nsplit) return;
  const int per = (seq + nsplit - 1) / nsplit;
  const int t0 = sp * per, t1 = min(seq, t0 + per), len = max(0, t1 - t0);
  int8_t* kbase = kc + size_t(layer) * max_seq * kv_dim + kvh * hs;
  int8_t* vbase = vc + size_t(layer) * max_seq * kv_dim + kvh * hs;
  for (int d = threadIdx.x; d < hs; d += blockDim.x) {
    qf[d] = float(Q[h * hs + d]);
    const int8_t k8 = int8_t(uint8_t(uint32_t(Kp[kvh * hs + d] / 256) & 0xffu));
    const int8_t v8 = int8_t(uint8_t(uint32_t(Vp[kvh * hs + d] / 256) & 0xffu));
    knew[d] = float(k8);
    vnew[d] = float(v8);
    if (sp == 0 && h % n_rep == 0) {
      kbase[size_t(pos) * kv_dim + d] = k8;
      vbase[size_t(pos) * kv_dim + d] = v8;
    }
  }
  __syncthreads();
  const int pieces = hs >> 4;              // 16-byte pieces per cache row (1, 2, 4 or 8)
  const int tpw = 32 / pieces;             // timesteps a warp covers per iteration
  const int piece = lane % pieces, tsub = lane / pieces;
  float q_r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) q_r[i] = qf[piece * 16 + i];
  auto load_row = [&](const int8_t* base, const float* fresh, int t, float (&f)[16]) {
    if (t == pos) {
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = fresh[piece * 16 + i];
    } else {
      const uint4 raw = *reinterpret_cast<const uint4*>(base + size_t(t) * kv_dim + piece * 16);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 16; ++i) f[i] = float(int8_t(uint8_t(w[i >> 2] >> (8 * (i & 3)))));
    }
  };
  // The V piece of this lane's first timestep is requested together with its K piece, so the second pass does
  // not start with a fresh round trip (short contexts have one timestep per lane).
  const int t_first = t0 + warp * tpw + tsub;
  uint4 v_first = make_uint4(0u, 0u, 0u, 0u);
  if (t_first < t1 && t_first != pos)
    v_first = *reinterpret_cast<const uint4*>(vbase + size_t(t_first) * kv_dim + piece * 16);
  // ---- scores of this split
  for (int tb = t0 + warp * tpw; tb < t1; tb += AI8_WARPS * tpw) {
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
  __syncthreads();
  // ---- exp-weights of the split
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < len; i += blockDim.x) mx = fmaxf(mx, scores[i]);
  mx = block_max(mx, red);
  float sum = 0.0f;
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    const float e = expf(scores[i] - mx);
    scores[i] = e;
    sum += e;
  }
  sum = block_sum(sum, red);
  // ---- weighted sums of V (with one split the weights are the probabilities themselves, as in the text)
  const bool single = nsplit == 1;
  float acc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.0f;
  for (int tb = t0 + warp * tpw; tb < t1; tb += AI8_WARPS * tpw) {
    const int t = tb + tsub;
    if (t < t1) {
      float vf[16];
      if (t == t_first && t != pos) {
        const uint32_t w[4] = {v_first.x, v_first.y, v_first.z, v_first.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) vf[i] = float(int8_t(uint8_t(w[i >> 2] >> (8 * (i & 3)))));
      } else {
        load_row(vbase, vnew, t, vf);
      }
      const float p = single ? scores[t - t0] / sum : scores[t - t0];
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
    for (int i = 0; i < 16; ++i) wpart[warp][piece * 16 + i] = acc[i];
  }
  __syncthreads();
  float* mine = part + (size_t(h) * nsplit + sp) * (hs + 2);
  for (int d = threadIdx.x; d < hs; d += blockDim.x) {
    float val = 0.0f;
#pragma unroll
    for (int w = 0; w < AI8_WARPS; ++w) val += wpart[w][d];
    if (single) {
      const int32_t out = __float2int_rz(val);                 // attn_out = val as i32
      xb_i8[h * hs + d] = quant_clamped(float(out) / 256.0f);   // next projection's input
    } else {
      mine[2 + d] = val;
    }
  }
  if (single) return;
  if (threadIdx.x == 0) { mine[0] = len > 0 ? mx : -INFINITY; mine[1] = len > 0 ? sum : 0.0f; }
  // last block of this head merges (writes above are published by the fence + atomic)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(&counters[h], 1) == nsplit - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // all partial maxima and sums are requested together, then all values of an element: one round trip each
  constexpr int MAXS = 16;   // the number of sequence splits never exceeds 16
  const float* p0 = part + size_t(h) * nsplit * (hs + 2);
  float mm[MAXS], ssum[MAXS], ex[MAXS];
#pragma unroll
  for (int x = 0; x < MAXS; ++x) {
    mm[x] = x < nsplit ? __ldcg(p0 + x * (hs + 2)) : -INFINITY;
    ssum[x] = x < nsplit ? __ldcg(p0 + x * (hs + 2) + 1) : 0.0f;
  }
  float M = -INFINITY;
#pragma unroll
  for (int x = 0; x < MAXS; ++x) M = fmaxf(M, mm[x]);
  float total = 0.0f;
#pragma unroll
  for (int x = 0; x < MAXS; ++x) {
    ex[x] = mm[x] != -INFINITY ? expf(mm[x] - M) : 0.0f;
    if (mm[x] != -INFINITY) total += ssum[x] * ex[x];
  }
  for (int d = threadIdx.x; d < hs; d += blockDim.x) {
    float pv[MAXS];
#pragma unroll
    for (int x = 0; x < MAXS; ++x) pv[x] = x < nsplit ? __ldcg(p0 + x * (hs + 2) + 2 + d) : 0.0f;
    float val = 0.0f;
#pragma unroll
    for (int x = 0; x < MAXS; ++x)
      if (mm[x] != -INFINITY) val += pv[x] * ex[x];
    const int32_t out = __float2int_rz(val / total);
    xb_i8[h * hs + d] = quant_clamped(float(out) / 256.0f);
  }
  if (threadIdx.x == 0) counters[h] = 0;
}

// xb = rmsnorm(x) * w for the classifier (one block).
__global__ void __launch_bounds__(1024) i8_final_norm_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                             float* __restrict__ y, int n) {
  __shared__ float red[33];
  pdl_launch_dependents();
  pdl_wait();
  float ss = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += x[i] * x[i];
  ss = block_sum(ss, red);
  const float r = sqrtf(ss / float(n) + 1e-5f);
  for (int i = threadIdx.x; i < n; i += blockDim.x) y[i] = (x[i] / r) * w[i];
}
__global__ void i8_advance_kernel(int* ctl) { ctl[0] = ctl[0] + 1; }

// ---------------------------------------------------------------------------------------------
#define I8_LAUNCH(...)                                                                                  \
  do {                                                                                                  \
    cudaError_t e__ = launch_kernel(__VA_ARGS__);                                                       \
    if (e__ != cudaSuccess)                                                                             \
      return set_error(SIMP_ERR_CUDA, "int8 decode launch failed: %s (%s:%d)", cudaGetErrorString(e__), __FILE__, __LINE__); \
  } while (0)

template <int PRO, int EPI>
static int gemv_i8_launch(GemvI8Args a, cudaStream_t st, int sms, bool pdl) {
  // rows per warp: 4 when that still leaves two blocks per SM, else 2, else 1 (all segment row counts must
  // divide; they are multiples of 16 here)
  int rpw = 4;
  bool div4 = true, div2 = true;
  for (int s = 0; s < (EPI == EPI_GATEUP ? 1 : a.nseg); ++s) {
    div4 = div4 && a.seg[s].rows % 4 == 0;
    div2 = div2 && a.seg[s].rows % 2 == 0;
  }
  while (rpw > 1 && ((rpw == 4 && !div4) || (rpw == 2 && !div2) || a.total_rows / (GI8_WARPS * rpw) < 2 * sms)) rpw >>= 1;
  if (EPI == EPI_GATEUP && rpw > 2) rpw = 2;   // two matrices per row: keep the loads in flight per lane bounded
  const int grid = (a.total_rows + GI8_WARPS * rpw - 1) / (GI8_WARPS * rpw);
  const size_t smem = size_t(a.K);
  cudaError_t e;
  if (rpw == 4) e = launch_kernel(gemv_i8_kernel<PRO, EPI, (EPI == EPI_GATEUP ? 2 : 4)>, dim3(grid), dim3(GI8_WARPS * 32), smem, st, pdl, a);
  else if (rpw == 2) e = launch_kernel(gemv_i8_kernel<PRO, EPI, 2>, dim3(grid), dim3(GI8_WARPS * 32), smem, st, pdl, a);
  else e = launch_kernel(gemv_i8_kernel<PRO, EPI, 1>, dim3(grid), dim3(GI8_WARPS * 32), smem, st, pdl, a);
  if (e != cudaSuccess) return set_error(SIMP_ERR_CUDA, "gemv_i8 launch failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

// shared memory of the attention kernel: the scores of one sequence split
static size_t i8_attn_smem(const LlamaI8Model& m) {
  return size_t((m.cfg.max_seq_len + m.nsplit - 1) / m.nsplit + 1) * 4;
}

static int i8_enqueue_token(LlamaI8Model& m, cudaStream_t st) {
  const simp_llama_i8_config& c = m.cfg;
  // (a single cooperative kernel per token was built for this model too: 698 us at position 0 against 641 for the
  // per-op kernels below, so it was removed)
  const int dim = int(c.dim), hd = int(c.hidden_dim), kv = int(m.kv_dim), hs = int(c.head_dim);
  const int sms = ctx().sm_count;
  I8_LAUNCH(i8_input_kernel, dim3((dim + 255) / 256), dim3(256), 0, st, false, (const int8_t*)m.x_i8, m.x, dim);
  for (int64_t l = 0; l < c.n_layers; ++l) {
    {
      GemvI8Args a{};
      a.seg[0] = GemvI8Seg{m.wq + l * dim * dim, m.q, dim};
      a.seg[1] = GemvI8Seg{m.wk + l * int64_t(kv) * dim, m.k, kv};
      a.seg[2] = GemvI8Seg{m.wv + l * int64_t(kv) * dim, m.v, kv};
      a.nseg = 3; a.K = dim; a.x_f32 = m.x; a.norm_w = m.rms_att + l * dim; a.total_rows = dim + 2 * kv;
      if (int rc = gemv_i8_launch<PRO_NORM, EPI_STORE>(a, st, sms, true)) return rc;
    }
    I8_LAUNCH(attn_i8_kernel, dim3(unsigned(c.n_heads), unsigned(m.nsplit)), dim3(AI8_WARPS * 32),
              i8_attn_smem(m), st, true, (const int32_t*)m.q, (const int32_t*)m.k, (const int32_t*)m.v, m.kc, m.vc, m.xb_i8,
              m.attn_part, m.attn_cnt, (const int*)m.ctl, hs, kv, int(c.n_heads / c.n_kv_heads), int(c.max_seq_len), int(l),
              m.nsplit);
    {
      GemvI8Args a{};
      a.seg[0] = GemvI8Seg{m.wo + l * dim * dim, nullptr, dim};
      a.nseg = 1; a.K = dim; a.x_i8 = m.xb_i8; a.resid = m.x; a.total_rows = dim;
      if (int rc = gemv_i8_launch<PRO_I8, EPI_RESID>(a, st, sms, true)) return rc;
    }
    {
      GemvI8Args a{};
      a.seg[0] = GemvI8Seg{m.w1 + l * int64_t(hd) * dim, nullptr, hd};
      a.seg[1] = GemvI8Seg{m.w3 + l * int64_t(hd) * dim, nullptr, hd};
      a.nseg = 2; a.K = dim; a.x_f32 = m.x; a.norm_w = m.rms_ffn + l * dim; a.hb = m.ffn_hb; a.total_rows = hd;
      if (int rc = gemv_i8_launch<PRO_NORM, EPI_GATEUP>(a, st, sms, true)) return rc;
    }
    {
      GemvI8Args a{};
      a.seg[0] = GemvI8Seg{m.w2 + l * int64_t(dim) * hd, nullptr, dim};
      a.nseg = 1; a.K = hd; a.x_i8 = m.ffn_hb; a.resid = m.x; a.total_rows = dim;
      if (int rc = gemv_i8_launch<PRO_I8, EPI_RESID>(a, st, sms, true)) return rc;
    }
  }
  I8_LAUNCH(i8_final_norm_kernel, dim3(1), dim3(1024), 0, st, true, (const float*)m.x, (const float*)m.rms_final, m.xb, dim);
  {
    GemvArgs g{};
    g.seg[0] = GemvSeg{m.wcls, m.logits, int(c.vocab_size)};
    g.nseg = 1; g.k4 = dim / 4; g.x = m.xb;
    if (int rc = gemv_f32_launch<GEMV_STORE>(g, st, sms)) return rc;
  }
  I8_LAUNCH(i8_advance_kernel, dim3(1), dim3(1), 0, st, false, m.ctl);
  return SIMP_OK;
}

static int i8_ensure_graph(LlamaI8Model& m) {
  if (m.graph) return SIMP_OK;
  cudaStream_t st = ctx().stream;
  // one eager pass first (sets attributes, surfaces launch errors outside capture); it writes the cache row
  // of the current position, which the replay writes again with the same values
  int pos_save = 0;
  SIMP_CUDA(cudaMemcpyAsync(&pos_save, m.ctl, 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  SIMP_CUDA(cudaFuncSetAttribute(attn_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(i8_attn_smem(m))));
  if (int rc = i8_enqueue_token(m, st)) return rc;
  SIMP_CUDA(cudaStreamSynchronize(st));
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, &pos_save, 4, cudaMemcpyHostToDevice, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  cudaGraph_t g = nullptr;
  SIMP_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  const int rc = i8_enqueue_token(m, st);
  cudaError_t e = cudaStreamEndCapture(st, &g);
  if (rc != SIMP_OK) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  SIMP_REQUIRE(e == cudaSuccess, SIMP_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(&m.graph, g, 0);
  cudaGraphDestroy(g);
  SIMP_REQUIRE(e == cudaSuccess, SIMP_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
  return SIMP_OK;
}

// ---------------------------------------------------------------------------------------------
// Prefill over M tokens at once (examples/llama2/llama32_1b_int8_prefill.sl:11-232).  The seven projections of
// a layer are int8 GEMMs on the tensor cores (gemm_i8_run: tcgen05 kind::i8, A = activations [M, K] s8,
// B = weights [N, K] s8 K-major); the steps between them are small row kernels that restate the text.
int gemm_i8_run(const void* A, const int8_t* B, int32_t* C, int64_t M, int64_t K, int64_t N, int a_unsigned,
                int b_transposed, int32_t* const* peer_c, int n_peers, int64_t ldc, int64_t col_offset, int self_rank = 0);

// f32 -> i8 without a clamp: truncate to i32, keep the low 8 bits (what the compiled reference does on x86).
__device__ __forceinline__ int8_t narrow_f32_to_i8(float v) {
  v = fmaxf(fminf(v, 2147483520.0f), -2147483648.0f);
  return int8_t(uint8_t(uint32_t(__float2int_rz(v)) & 0xffu));
}

// x_f32 = (f32) x_i8 over M * dim elements (prefill.sl:23-27); rows = 1 block each for the norm below.
__global__ void pf_input_kernel(const int8_t* __restrict__ x_i8, float* __restrict__ x, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = float(x_i8[i]) * 1.0f;
}
// One block per token: ss = 1 / sqrt(mean(x^2) + 1e-5); xb = x * ss * w; xb_i8 = (i8)(xb * 127) unclamped (:33-51).
__global__ void __launch_bounds__(256) pf_norm_quant_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                            int8_t* __restrict__ xb_i8, int dim) {
  __shared__ float red[33];
  const float* xr = x + size_t(blockIdx.x) * dim;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, red);
  ss = 1.0f / sqrtf(ss / (float(dim) * 1.0f) + 0.00001f);
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    xb_i8[size_t(blockIdx.x) * dim + i] = narrow_f32_to_i8((xr[i] * ss * w[i]) * 127.0f);
}
// cache[layer][t][i] = (i8)(acc / 256) for K and V (:69-79); the device cache keeps its [max_seq, kv_dim] layout.
__global__ void pf_kv_store_kernel(const int32_t* __restrict__ K, const int32_t* __restrict__ V, int8_t* __restrict__ kc,
                                   int8_t* __restrict__ vc, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    kc[i] = int8_t(uint8_t(uint32_t(K[i] / 256) & 0xffu));
    vc[i] = int8_t(uint8_t(uint32_t(V[i] / 256) & 0xffu));
  }
}
// Causal attention, one block per (head, query position) (:81-141): thread t scores key t, block softmax with
// the division of the text, thread d sums dim d; attn_out = (i32) trunc, next input = (i8)(attn_out / 256.0).
__global__ void __launch_bounds__(256) pf_attn_kernel(const int32_t* __restrict__ Q, const int8_t* __restrict__ kc,
                                                      const int8_t* __restrict__ vc, int8_t* __restrict__ xb_i8, int dim,
                                                      int hs, int kv_dim, int n_rep) {
  __shared__ float qf[128], probs[256], red[33];
  const int h = blockIdx.x, q_pos = blockIdx.y, ko = (h / n_rep) * hs;
  for (int d = threadIdx.x; d < hs; d += blockDim.x) qf[d] = float(Q[size_t(q_pos) * dim + h * hs + d]);
  __syncthreads();
  const int t = threadIdx.x;
  float score = -INFINITY;
  if (t <= q_pos) {
    const uint4* kr = reinterpret_cast<const uint4*>(kc + size_t(t) * kv_dim + ko);   // head_dim is a multiple of 16
    float sc = 0.0f;
    for (int d16 = 0; d16 < (hs >> 4); ++d16) {
      const uint4 raw = kr[d16];
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 16; ++i)
        sc = sc + qf[d16 * 16 + i] * 1.0f * float(int8_t(uint8_t(w[i >> 2] >> (8 * (i & 3))))) * 1.0f;
    }
    score = sc / 8.0f;
  }
  const float mx = block_max(score, red);
  const float e = t <= q_pos ? expf(score - mx) : 0.0f;
  const float sum = block_sum(e, red);
  probs[t] = t <= q_pos ? e / sum : 0.0f;
  __syncthreads();
  if (t < hs) {
    float val = 0.0f;
    int vi = 0;
    for (; vi + 8 <= q_pos + 1; vi += 8) {   // eight rows requested together; the sum keeps its order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = float(vc[size_t(vi + u) * kv_dim + ko + t]);
#pragma unroll
      for (int u = 0; u < 8; ++u) val = val + probs[vi + u] * v[u] * 1.0f;
    }
    for (; vi <= q_pos; ++vi) val = val + probs[vi] * float(vc[size_t(vi) * kv_dim + ko + t]) * 1.0f;
    const int32_t out = __float2int_rz(val);
    xb_i8[size_t(q_pos) * dim + h * hs + t] = narrow_f32_to_i8(float(out) * 1.0f / 256.0f);
  }
}
// x += (f32) acc / 65536 (:160-167, :220-227)
__global__ void pf_resid_kernel(float* __restrict__ x, const int32_t* __restrict__ acc, int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = x[i] + float(acc[i]) * 1.0f / 65536.0f;
}
// ffn_hb = (i8)(silu(gate / 65536) * (up / 65536) * 127) unclamped (:203-213)
__global__ void pf_swiglu_kernel(const int32_t* __restrict__ gate, const int32_t* __restrict__ up, int8_t* __restrict__ hb,
                                 int64_t n) {
  const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    const float gate_f = float(gate[i]) * 1.0f / 65536.0f;
    const float silu = gate_f / (1.0f + expf(0.0f - gate_f));
    const float up_f = float(up[i]) * 1.0f / 65536.0f;
    hb[i] = narrow_f32_to_i8(silu * up_f * 127.0f);
  }
}

static int i8_prefill_run(LlamaI8Model& m, int64_t M, float* x, int8_t* x_i8, int8_t* xb_i8, int8_t* hb, int32_t* acc0,
                          int32_t* acc1, cudaStream_t st) {
  const simp_llama_i8_config& c = m.cfg;
  const int64_t dim = c.dim, hd = c.hidden_dim, kv = m.kv_dim;
  auto blocks = [](int64_t n) { return dim3(unsigned((n + 255) / 256)); };
  pf_input_kernel<<<blocks(M * dim), 256, 0, st>>>(x_i8, x, M * dim);
  for (int64_t l = 0; l < c.n_layers; ++l) {
    pf_norm_quant_kernel<<<dim3(unsigned(M)), 256, 0, st>>>(x, m.rms_att + l * dim, xb_i8, int(dim));
    int32_t *Q = acc0, *K = acc1, *V = acc1 + M * kv;
    if (int rc = gemm_i8_run(xb_i8, m.wq + l * dim * dim, Q, M, dim, dim, 0, 1, nullptr, 0, dim, 0)) return rc;
    if (int rc = gemm_i8_run(xb_i8, m.wk + l * kv * dim, K, M, dim, kv, 0, 1, nullptr, 0, kv, 0)) return rc;
    if (int rc = gemm_i8_run(xb_i8, m.wv + l * kv * dim, V, M, dim, kv, 0, 1, nullptr, 0, kv, 0)) return rc;
    int8_t* kc = m.kc + size_t(l) * c.max_seq_len * kv;
    int8_t* vc = m.vc + size_t(l) * c.max_seq_len * kv;
    pf_kv_store_kernel<<<blocks(M * kv), 256, 0, st>>>(K, V, kc, vc, M * kv);
    pf_attn_kernel<<<dim3(unsigned(c.n_heads), unsigned(M)), 256, 0, st>>>(Q, kc, vc, xb_i8, int(dim), int(c.head_dim), int(kv),
                                                                        int(c.n_heads / c.n_kv_heads));
    if (int rc = gemm_i8_run(xb_i8, m.wo + l * dim * dim, acc0, M, dim, dim, 0, 1, nullptr, 0, dim, 0)) return rc;
    pf_resid_kernel<<<blocks(M * dim), 256, 0, st>>>(x, acc0, M * dim);
    pf_norm_quant_kernel<<<dim3(unsigned(M)), 256, 0, st>>>(x, m.rms_ffn + l * dim, xb_i8, int(dim));
    if (int rc = gemm_i8_run(xb_i8, m.w1 + l * hd * dim, acc0, M, dim, hd, 0, 1, nullptr, 0, hd, 0)) return rc;
    if (int rc = gemm_i8_run(xb_i8, m.w3 + l * hd * dim, acc1, M, dim, hd, 0, 1, nullptr, 0, hd, 0)) return rc;
    pf_swiglu_kernel<<<blocks(M * hd), 256, 0, st>>>(acc0, acc1, hb, M * hd);
    if (int rc = gemm_i8_run(hb, m.w2 + l * dim * hd, acc0, M, hd, dim, 0, 1, nullptr, 0, dim, 0)) return rc;
    pf_resid_kernel<<<blocks(M * dim), 256, 0, st>>>(x, acc0, M * dim);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_llama_i8_destroy(void* model) {
  if (!model) return SIMP_OK;
  LlamaI8Model* m = static_cast<LlamaI8Model*>(model);
  if (ctx().ready) cudaStreamSynchronize(ctx().stream);
  if (m->graph) cudaGraphExecDestroy(m->graph);
  for (auto& pl : m->plans) {
    if (pl.graph) cudaGraphExecDestroy(pl.graph);
    void* pp[] = {pl.x, pl.x_i8, pl.xb_i8, pl.hb, pl.acc0, pl.acc1};
    for (void* p : pp)
      if (p) cudaFree(p);
  }
  void* ptrs[] = {m->rms_att, m->rms_ffn, m->rms_final, m->wcls, m->wq, m->wk, m->wv, m->wo, m->w1, m->w2, m->w3,
                  m->x_i8, m->xb_i8, m->ffn_hb, m->kc, m->vc, m->x, m->xb, m->logits, m->q, m->k, m->v, m->ctl,
                  m->attn_part, m->attn_cnt};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  delete m;
  return SIMP_OK;
}

SIMP_API int simp_llama_i8_create(const simp_llama_i8_config* cfg, void** model) {
  SIMP_REQUIRE(cfg && model, SIMP_ERR_ARG, "llama_i8_create: null pointer");
  if (int rc = ensure_ready()) return rc;
  const simp_llama_i8_config& c = *cfg;
  SIMP_REQUIRE(c.dim > 0 && c.hidden_dim > 0 && c.n_layers > 0 && c.n_heads > 0 && c.n_kv_heads > 0 && c.vocab_size > 0 &&
                   c.max_seq_len > 0 && c.head_dim > 0,
               SIMP_ERR_ARG, "llama_i8_create: non-positive dimension");
  SIMP_REQUIRE(c.n_heads * c.head_dim == c.dim && c.n_heads % c.n_kv_heads == 0, SIMP_ERR_SHAPE,
               "llama_i8_create: n_heads * head_dim must equal dim and n_kv_heads must divide n_heads");
  SIMP_REQUIRE(c.dim % 16 == 0 && c.hidden_dim % 16 == 0 && c.dim <= 65536 && c.hidden_dim <= 65536, SIMP_ERR_SHAPE,
               "llama_i8_create: dim and hidden_dim must be multiples of 16 and at most 65536");
  SIMP_REQUIRE((c.head_dim == 16 || c.head_dim == 32 || c.head_dim == 64 || c.head_dim == 128) && c.max_seq_len <= 131072,
               SIMP_ERR_SHAPE, "llama_i8_create: head_dim must be 16, 32, 64 or 128; max_seq_len at most 131072");
  LlamaI8Model* m = new LlamaI8Model();
  m->cfg = c;
  m->kv_dim = c.n_kv_heads * c.head_dim;
  int rc = SIMP_OK;
  auto A = [&](void** p, size_t n) {
    if (rc != SIMP_OK) return;
    cudaError_t e = cudaMalloc(p, n ? n : 16);
    if (e != cudaSuccess) rc = set_error(SIMP_ERR_CUDA, "llama_i8_create: cudaMalloc of %zu bytes failed: %s", n, cudaGetErrorString(e));
  };
  const size_t kv_bytes = size_t(c.n_layers) * c.max_seq_len * m->kv_dim;
  A((void**)&m->x_i8, c.dim); A((void**)&m->xb_i8, c.dim); A((void**)&m->ffn_hb, c.hidden_dim);
  A((void**)&m->kc, kv_bytes); A((void**)&m->vc, kv_bytes);
  A((void**)&m->x, c.dim * 4); A((void**)&m->xb, c.dim * 4); A((void**)&m->logits, c.vocab_size * 4);
  A((void**)&m->q, c.dim * 4); A((void**)&m->k, m->kv_dim * 4); A((void**)&m->v, m->kv_dim * 4);
  A((void**)&m->ctl, 64);
  // one sequence split per 256 positions of context, at most 16: (heads x splits) blocks keep the SMs busy
  m->nsplit = int(std::min<int64_t>(AI8_MAX_SPLITS, std::max<int64_t>(1, c.max_seq_len / 256)));
  A((void**)&m->attn_part, size_t(c.n_heads) * m->nsplit * (c.head_dim + 2) * 4);
  A((void**)&m->attn_cnt, size_t(c.n_heads) * 4);
  if (rc != SIMP_OK) { simp_llama_i8_destroy(m); return rc; }
  cudaMemsetAsync(m->ctl, 0, 64, ctx().stream);
  cudaMemsetAsync(m->attn_cnt, 0, size_t(c.n_heads) * 4, ctx().stream);
  cudaMemsetAsync(m->kc, 0, kv_bytes, ctx().stream);
  cudaMemsetAsync(m->vc, 0, kv_bytes, ctx().stream);
  *model = m;
  return SIMP_OK;
}

SIMP_API int simp_llama_i8_load(void* model, const char* name, const void* host, size_t bytes) {
  SIMP_REQUIRE(model && name && host, SIMP_ERR_ARG, "llama_i8_load: null pointer");
  LlamaI8Model& m = *static_cast<LlamaI8Model*>(model);
  const simp_llama_i8_config& c = m.cfg;
  const std::string n(name);
  const size_t d = c.dim, h = c.hidden_dim, L = c.n_layers, V = c.vocab_size, kv = m.kv_dim;
  void** slot = nullptr;
  size_t want = 0;
  if (n == "rms_att_w") { slot = (void**)&m.rms_att; want = L * d * 4; }
  else if (n == "rms_ffn_w") { slot = (void**)&m.rms_ffn; want = L * d * 4; }
  else if (n == "rms_final_w") { slot = (void**)&m.rms_final; want = d * 4; }
  else if (n == "wcls") { slot = (void**)&m.wcls; want = V * d * 4; }
  else if (n == "wq_t") { slot = (void**)&m.wq; want = L * d * d; }
  else if (n == "wk_t") { slot = (void**)&m.wk; want = L * kv * d; }
  else if (n == "wv_t") { slot = (void**)&m.wv; want = L * kv * d; }
  else if (n == "wo_t") { slot = (void**)&m.wo; want = L * d * d; }
  else if (n == "w1_t") { slot = (void**)&m.w1; want = L * h * d; }
  else if (n == "w2_t") { slot = (void**)&m.w2; want = L * d * h; }
  else if (n == "w3_t") { slot = (void**)&m.w3; want = L * h * d; }
  SIMP_REQUIRE(slot != nullptr, SIMP_ERR_ARG, "llama_i8_load: unknown tensor '%s'", name);
  SIMP_REQUIRE(bytes == want, SIMP_ERR_SHAPE, "llama_i8_load: '%s' has %zu bytes, the configuration needs %zu", name, bytes, want);
  if (!*slot) SIMP_CUDA(cudaMalloc(slot, want));
  SIMP_CUDA(cudaMemcpyAsync(*slot, host, want, cudaMemcpyHostToDevice, ctx().stream));
  SIMP_CUDA(cudaStreamSynchronize(ctx().stream));
  return SIMP_OK;
}

static int i8_check_loaded(const LlamaI8Model& m) {
  SIMP_REQUIRE(m.rms_att && m.rms_ffn && m.rms_final && m.wcls && m.wq && m.wk && m.wv && m.wo && m.w1 && m.w2 && m.w3,
               SIMP_ERR_STATE, "llama_i8: not every tensor has been loaded");
  return SIMP_OK;
}

SIMP_API int simp_llama_i8_reset_cache(void* model) {
  SIMP_REQUIRE(model, SIMP_ERR_ARG, "llama_i8_reset_cache: null model");
  LlamaI8Model& m = *static_cast<LlamaI8Model*>(model);
  const size_t kv_bytes = size_t(m.cfg.n_layers) * m.cfg.max_seq_len * m.kv_dim;
  SIMP_CUDA(cudaMemsetAsync(m.kc, 0, kv_bytes, ctx().stream));
  SIMP_CUDA(cudaMemsetAsync(m.vc, 0, kv_bytes, ctx().stream));
  return SIMP_OK;
}

SIMP_API int simp_llama_i8_decode_loop(void* model, const int8_t* x_i8_host, int64_t start_pos, int64_t n_tokens,
                                       float* logits_host, float* ms_out) {
  SIMP_REQUIRE(model && x_i8_host, SIMP_ERR_ARG, "llama_i8: null pointer");
  LlamaI8Model& m = *static_cast<LlamaI8Model*>(model);
  if (int rc = i8_check_loaded(m)) return rc;
  SIMP_REQUIRE(n_tokens >= 1 && start_pos >= 0 && start_pos + n_tokens <= m.cfg.max_seq_len, SIMP_ERR_ARG,
               "llama_i8: positions %lld .. %lld outside [0, %lld)", (long long)start_pos, (long long)(start_pos + n_tokens - 1),
               (long long)m.cfg.max_seq_len);
  cudaStream_t st = ctx().stream;
  const int pos32 = int(start_pos);
  SIMP_CUDA(cudaMemcpyAsync(m.x_i8, x_i8_host, size_t(m.cfg.dim), cudaMemcpyHostToDevice, st));
  SIMP_CUDA(cudaMemcpyAsync(m.ctl, &pos32, 4, cudaMemcpyHostToDevice, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  if (int rc = i8_ensure_graph(m)) return rc;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ms_out) {
    SIMP_CUDA(cudaEventCreate(&e0));
    SIMP_CUDA(cudaEventCreate(&e1));
    SIMP_CUDA(cudaEventRecord(e0, st));
  }
  for (int64_t i = 0; i < n_tokens; ++i) SIMP_CUDA(cudaGraphLaunch(m.graph, st));
  if (ms_out) SIMP_CUDA(cudaEventRecord(e1, st));
  if (logits_host)
    SIMP_CUDA(cudaMemcpyAsync(logits_host, m.logits, size_t(m.cfg.vocab_size) * 4, cudaMemcpyDeviceToHost, st));
  SIMP_CUDA(cudaStreamSynchronize(st));
  if (ms_out) {
    SIMP_CUDA(cudaEventElapsedTime(ms_out, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return simp_gpu_check_device_status();
}

SIMP_API int simp_llama_i8_forward(void* model, const int8_t* x_i8_host, int64_t pos, float* logits_host) {
  return simp_llama_i8_decode_loop(model, x_i8_host, pos, 1, logits_host, nullptr);
}

// Scratch and graph of a prefill length, created on first use: one eager pass (sets kernel attributes, surfaces
// launch errors outside capture), then the same enqueue captured.  The host work of a prefill -- 112 GEMM calls
// with three tensor-map encodes each -- would otherwise cost more than the device work at small seq_len.
static int i8_prefill_plan(LlamaI8Model& m, int64_t M, LlamaI8Model::PrefillPlan** out) {
  for (auto& pl : m.plans)
    if (pl.M == M) { *out = &pl; return SIMP_OK; }
  const simp_llama_i8_config& c = m.cfg;
  const int64_t dim = c.dim, hd = c.hidden_dim, kv = m.kv_dim;
  LlamaI8Model::PrefillPlan pl;
  pl.M = M;
  const size_t acc_elems = size_t(M) * size_t(std::max<int64_t>(hd, std::max<int64_t>(dim, 2 * kv)));
  int rc = SIMP_OK;
  auto A = [&](void** p, size_t n) {
    if (rc != SIMP_OK) return;
    cudaError_t e = cudaMalloc(p, n);
    if (e != cudaSuccess) rc = set_error(SIMP_ERR_CUDA, "llama_i8_prefill: cudaMalloc of %zu bytes failed: %s", n, cudaGetErrorString(e));
  };
  A((void**)&pl.x, size_t(M) * dim * 4); A((void**)&pl.x_i8, size_t(M) * dim); A((void**)&pl.xb_i8, size_t(M) * dim);
  A((void**)&pl.hb, size_t(M) * hd); A((void**)&pl.acc0, acc_elems * 4); A((void**)&pl.acc1, acc_elems * 4);
  cudaStream_t st = ctx().stream;
  if (rc == SIMP_OK) {
    cudaMemsetAsync(pl.x_i8, 0, size_t(M) * dim, st);
    rc = i8_prefill_run(m, M, pl.x, pl.x_i8, pl.xb_i8, pl.hb, pl.acc0, pl.acc1, st);
    if (rc == SIMP_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = set_error(SIMP_ERR_CUDA, "llama_i8_prefill: eager pass failed");
  }
  if (rc == SIMP_OK) {
    cudaGraph_t g = nullptr;
    if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess)
      rc = set_error(SIMP_ERR_CUDA, "llama_i8_prefill: begin capture failed");
    if (rc == SIMP_OK) {
      const int rr = i8_prefill_run(m, M, pl.x, pl.x_i8, pl.xb_i8, pl.hb, pl.acc0, pl.acc1, st);
      cudaError_t e = cudaStreamEndCapture(st, &g);
      if (rr != SIMP_OK) rc = rr;
      else if (e != cudaSuccess) rc = set_error(SIMP_ERR_CUDA, "llama_i8_prefill: capture failed: %s", cudaGetErrorString(e));
      else if ((e = cudaGraphInstantiate(&pl.graph, g, 0)) != cudaSuccess)
        rc = set_error(SIMP_ERR_CUDA, "llama_i8_prefill: graph instantiate failed: %s", cudaGetErrorString(e));
      if (g) cudaGraphDestroy(g);
    }
  }
  if (rc != SIMP_OK) {
    void* pp[] = {pl.x, pl.x_i8, pl.xb_i8, pl.hb, pl.acc0, pl.acc1};
    for (void* p : pp)
      if (p) cudaFree(p);
    return rc;
  }
  m.plans.push_back(pl);
  *out = &m.plans.back();
  return SIMP_OK;
}

SIMP_API int simp_llama_i8_prefill(void* model, const int8_t* x_i8_host, int64_t seq_len, float* x_fp32_host,
                                   int8_t* k_cache_host, int8_t* v_cache_host, float* ms_out) {
  SIMP_REQUIRE(model && x_i8_host, SIMP_ERR_ARG, "llama_i8_prefill: null pointer");
  LlamaI8Model& m = *static_cast<LlamaI8Model*>(model);
  if (int rc = i8_check_loaded(m)) return rc;
  const simp_llama_i8_config& c = m.cfg;
  const int64_t M = seq_len, dim = c.dim, kv = m.kv_dim;
  SIMP_REQUIRE(M >= 1 && M <= 256 && M <= c.max_seq_len, SIMP_ERR_ARG,
               "llama_i8_prefill: seq_len %lld outside [1, min(256, max_seq_len)]", (long long)M);
  LlamaI8Model::PrefillPlan* pl = nullptr;
  if (int rc = i8_prefill_plan(m, M, &pl)) return rc;
  cudaStream_t st = ctx().stream;
  SIMP_CUDA(cudaMemcpyAsync(pl->x_i8, x_i8_host, size_t(M) * dim, cudaMemcpyHostToDevice, st));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (ms_out) {
    SIMP_CUDA(cudaEventCreate(&e0));
    SIMP_CUDA(cudaEventCreate(&e1));
    SIMP_CUDA(cudaEventRecord(e0, st));
  }
  SIMP_CUDA(cudaGraphLaunch(pl->graph, st));
  if (ms_out) SIMP_CUDA(cudaEventRecord(e1, st));
  if (x_fp32_host) SIMP_CUDA(cudaMemcpyAsync(x_fp32_host, pl->x, size_t(M) * dim * 4, cudaMemcpyDeviceToHost, st));
  for (int64_t l = 0; l < c.n_layers; ++l) {   // cache rows 0 .. M-1 of every layer, packed [n_layers, M, kv_dim]
    const size_t src = size_t(l) * c.max_seq_len * kv, dst = size_t(l) * M * kv;
    if (k_cache_host) SIMP_CUDA(cudaMemcpyAsync(k_cache_host + dst, m.kc + src, size_t(M) * kv, cudaMemcpyDeviceToHost, st));
    if (v_cache_host) SIMP_CUDA(cudaMemcpyAsync(v_cache_host + dst, m.vc + src, size_t(M) * kv, cudaMemcpyDeviceToHost, st));
  }
  SIMP_CUDA(cudaStreamSynchronize(st));
  if (ms_out) {
    SIMP_CUDA(cudaEventElapsedTime(ms_out, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  }
  return simp_gpu_check_device_status();
}
