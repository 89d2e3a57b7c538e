// simp_oracle.cpp -- CPU restatement of the SimpLang tensor hot path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the *checker* for the CUDA library:
// the test-suite, the smoke check and the CPU-baseline leg of the benchmark
// are the only callers.  Nothing the CUDA library ships may link, import or
// fall back to anything in this directory.
//
// Every function restates, in plain sequential loops, what one lowering
// pattern of the reference compiler emits (paths are relative to the
// reference project root).  Parity status per function is given in its
// comment: "pinned" means one of the reference's own known-answer tests or
// its own compiled CPU code is checked against this restatement by the test
// suite; "parity unpinned" means the reference holds no test for the op and
// the restatement follows the lowering source only.
//
// Build: see oracle/Makefile (g++ -O2 -fopenmp -shared -fPIC).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API extern "C" __attribute__((visibility("default")))

namespace {
inline int clamp_threads(int threads) {
#ifdef _OPENMP
  if (threads <= 0) return omp_get_max_threads();
  return threads;
#else
  (void)threads;
  return 1;
#endif
}
}  // namespace

ORACLE_API int simp_oracle_max_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Sets the OpenMP team size used by later parallel regions started from the calling thread (every library
// in the process that links the same OpenMP runtime follows it, the compiled reference kernels included).
// Launchers that export OMP_NUM_THREADS=1 to every rank would otherwise pin the CPU legs to one core.
ORACLE_API int simp_oracle_set_threads(int threads) {
#ifdef _OPENMP
  if (threads > 0) omp_set_num_threads(threads);
  return omp_get_max_threads();
#else
  (void)threads;
  return 1;
#endif
}

// ---------------------------------------------------------------------------
// simp.matmul : C[coff + i*n + j] += sum_p A[aoff + i*k + p] * B[boff + p*n + j]
// Follows MatMulOpLowering (src/mlir/lowering/ConvertSimpToMemRef.cpp:1794-1920):
// a linalg.matmul on reinterpret-cast views, which ACCUMULATES into C; the
// callers zero C first (examples/llama2/stories110M.sl:66-83).
// Pinned by tests/mlir/integration/test_matmul_simple.sl:24-27 (2x2 -> 19).
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_matmul_f32(const float* A, int64_t aoff, const float* B, int64_t boff,
                                       float* C, int64_t coff, int64_t m, int64_t k, int64_t n,
                                       int threads) {
  const int nt = clamp_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      float acc = C[coff + i * n + j];
      for (int64_t p = 0; p < k; ++p) acc += A[aoff + i * k + p] * B[boff + p * n + j];
      C[coff + i * n + j] = acc;
    }
  }
}

// ---------------------------------------------------------------------------
// tensor_matmul on f32 / f64: fresh zero-filled result, then C[i,j] += A[i,p]*B[p,j]
// (ConvertSimpToMemRef.cpp:2926-2933 zero fill, :3280-3291 linalg.matmul).
// b_transposed selects tensor_matmul_nt (:3373-3486), B given as [N,K].
// Pinned by tests/test_tensor_matmul.sl:4-65 (4x3 * 3x2 -> C[0,0] = 22).
// ---------------------------------------------------------------------------
template <typename T>
static void tensor_matmul_fp(const T* A, const T* B, T* C, int64_t M, int64_t K, int64_t N,
                             int b_transposed, int threads) {
  const int nt = clamp_threads(threads);
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      T acc = T(0);
      for (int64_t p = 0; p < K; ++p)
        acc += A[i * K + p] * (b_transposed ? B[j * K + p] : B[p * N + j]);
      C[i * N + j] = acc;
    }
  }
}
ORACLE_API void simp_oracle_tensor_matmul_f32(const float* A, const float* B, float* C, int64_t M,
                                              int64_t K, int64_t N, int b_transposed, int threads) {
  tensor_matmul_fp<float>(A, B, C, M, K, N, b_transposed, threads);
}
ORACLE_API void simp_oracle_tensor_matmul_f64(const double* A, const double* B, double* C,
                                              int64_t M, int64_t K, int64_t N, int b_transposed,
                                              int threads) {
  tensor_matmul_fp<double>(A, B, C, M, K, N, b_transposed, threads);
}

// ---------------------------------------------------------------------------
// tensor_matmul on i8: C[i,j] (i32, wrap-around) = sum_p ext(A[i,p]) * sext(B[p,j]).
// a_unsigned == 0: the op as lowered -- both operands sign-extended
//   (ConvertSimpToMemRef.cpp:3220-3247; the VNNI rewrite's sign flip and
//   128*sum(B) correction cancel exactly, src/mlir/passes/VNNIPass.cpp:819-830,
//   899-906).
// a_unsigned == 1: the raw vpdpbusd form, A zero-extended
//   (simptensor/tests/test_vnni_correctness.cpp:28-42).
// b_transposed == 1: B is [N,K] (tensor_matmul_nt, ConvertSimpToMemRef.cpp:3417-3443).
// Accumulation is modulo 2^32 (vpdpbusd does not saturate,
// test_vnni_correctness.cpp:248-277); done here in uint32_t.
// Pinned against the reference's own compiled VNNI kernels (oracle/ref_shim.cpp)
// and the checksum test on the ((i*N+j)%127)-64 fill
// (simptensor/benchmarks/bench_int8_matmul_omp_runner.cpp:36-64).
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_tensor_matmul_i8(const void* A_, const int8_t* B, int32_t* C,
                                             int64_t M, int64_t K, int64_t N, int a_unsigned,
                                             int b_transposed, int threads) {
  const int nt = clamp_threads(threads);
  const int8_t* As = static_cast<const int8_t*>(A_);
  const uint8_t* Au = static_cast<const uint8_t*>(A_);
  // Work on a [N,K] copy of B so the inner loop is contiguous (same values, same sums).
  std::vector<int8_t> bt;
  const int8_t* Bt = B;
  if (!b_transposed) {
    bt.resize(size_t(N) * size_t(K));
    for (int64_t p = 0; p < K; ++p)
      for (int64_t j = 0; j < N; ++j) bt[j * K + p] = B[p * N + j];
    Bt = bt.data();
  }
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      uint32_t acc = 0;
      const int8_t* brow = Bt + j * K;
      if (a_unsigned) {
        const uint8_t* arow = Au + i * K;
        for (int64_t p = 0; p < K; ++p) acc += uint32_t(int32_t(arow[p]) * int32_t(brow[p]));
      } else {
        const int8_t* arow = As + i * K;
        for (int64_t p = 0; p < K; ++p) acc += uint32_t(int32_t(arow[p]) * int32_t(brow[p]));
      }
      C[i * N + j] = int32_t(acc);
    }
  }
}

// i32 checksum of C the way the benchmark kernels fold it
// (simptensor/benchmarks/bench_int8_matmul.sl:29-40): wrap-around i32 sum.
ORACLE_API int32_t simp_oracle_checksum_i32(const int32_t* C, int64_t count) {
  uint32_t s = 0;
  for (int64_t i = 0; i < count; ++i) s += uint32_t(C[i]);
  return int32_t(s);
}

// ---------------------------------------------------------------------------
// dequant_w4: byte = qw[idx>>1]; q = idx odd ? high nibble : low nibble;
// w = float(q) * scale[idx/gs] + zero[idx/gs]
// (DequantW4OpLowering, ConvertSimpToMemRef.cpp:2384-2424; note the code is
// q*scale+zero, not (q-zero)*scale as the op description says).
// zeros == nullptr is this project's symmetric extension: zero = -8*scale.
// Parity unpinned: no reference test exercises the op.
// ---------------------------------------------------------------------------
static inline float dequant_one(const uint8_t* qw, const float* sc, const float* zr, int64_t idx,
                                int64_t sidx) {
  const uint32_t byte = qw[idx >> 1];
  const uint32_t q = (idx & 1) ? ((byte >> 4) & 15u) : (byte & 15u);
  const float s = sc[sidx];
  const float z = zr ? zr[sidx] : -8.0f * s;
  return float(q) * s + z;
}
ORACLE_API void simp_oracle_dequant_w4(const uint8_t* qw, const float* sc, const float* zr,
                                       int64_t idx0, int64_t count, int64_t gs, float* out) {
  for (int64_t t = 0; t < count; ++t) {
    const int64_t idx = idx0 + t;
    out[t] = dequant_one(qw, sc, zr, idx, idx / gs);
  }
}

// ---------------------------------------------------------------------------
// matmul_quant (MatMulQuantOpLowering, ConvertSimpToMemRef.cpp:3906-4005):
//   for i < rows: out[i] = 0
//     for g < cols/gs:                       (integer division, :3916)
//       scale/zero index = (i*cols)/gs + g   (:3923-3926; `offset` NOT added)
//       acc = 0
//       for t < 8, j < 16:                   (8 tiles of 16 hard-coded, :3928-3936)
//         kk = g*gs + t*16 + j
//         w  = dequant(weight index offset + i*cols + kk)
//         if kk < cols: acc += w * x[kk]
//       out[i] += acc
// scale_mode 0 = exactly that ("reference").  scale_mode 1 ("per_matrix") is
// the self-consistent variant used for the 3B configuration: every weight of
// the group [g*gs, (g+1)*gs) is visited once and the scale/zero index is
// (offset + i*cols)/gs + g.  For gs == 128 and offset == 0 the two coincide.
// Parity unpinned: no reference test exercises the op
// (examples/llama2/test_quant_host.cpp only prints an RMSE of a user-level kernel).
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_matmul_quant(const uint8_t* qw, const float* sc, const float* zr,
                                         const float* x, float* out, int64_t rows, int64_t cols,
                                         int64_t gs, int64_t offset, int scale_mode, int threads) {
  const int nt = clamp_threads(threads);
  const int64_t ngroups = cols / gs;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < rows; ++i) {
    float o = 0.0f;
    const int64_t row_off = i * cols;
    for (int64_t g = 0; g < ngroups; ++g) {
      const int64_t sidx = (scale_mode == 0 ? row_off : offset + row_off) / gs + g;
      const int64_t span = (scale_mode == 0) ? 128 : gs;
      float acc = 0.0f;
      for (int64_t e = 0; e < span; ++e) {
        const int64_t kk = g * gs + e;
        if (kk < cols) acc += dequant_one(qw, sc, zr, offset + row_off + kk, sidx) * x[kk];
      }
      o += acc;
    }
    out[i] = o;
  }
}

// Asymmetric W4 quantiser of the reference's host
// (examples/llama2/bench_llama_quant.cpp:51-93): flat groups of gs weights,
// scale = (max-min)/15 floored at 1e-8, zero = min, q = clamp(round((w-min)/scale), 0, 15),
// low nibble = even flat index.  Writes count/2 bytes and ceil(count/gs) scale/zero pairs.
ORACLE_API void simp_oracle_quantize_w4(const float* w, int64_t count, int64_t gs, uint8_t* qw,
                                        float* sc, float* zr) {
  const int64_t ngroups = (count + gs - 1) / gs;
  std::memset(qw, 0, size_t((count + 1) / 2));
  for (int64_t g = 0; g < ngroups; ++g) {
    const int64_t s = g * gs, e = std::min(s + gs, count);
    float mn = w[s], mx = w[s];
    for (int64_t i = s; i < e; ++i) {
      mn = std::min(mn, w[i]);
      mx = std::max(mx, w[i]);
    }
    float scale = (mx - mn) / 15.0f;
    if (scale < 1e-8f) scale = 1e-8f;
    sc[g] = scale;
    zr[g] = mn;
    for (int64_t i = s; i < e; ++i) {
      int q = int(std::round((w[i] - mn) / scale));
      q = std::max(0, std::min(15, q));
      if ((i & 1) == 0)
        qw[i >> 1] = uint8_t(q);
      else
        qw[i >> 1] |= uint8_t(q << 4);
    }
  }
}

// ---------------------------------------------------------------------------
// rmsnorm (RMSNormOpLowering, ConvertSimpToMemRef.cpp:2192-2230):
//   ss = sum x[i]^2 (sequential f32); r = sqrtf(ss/n + eps); y[i] = (x[i]/r) * w[woff+i]
// Pinned by examples/llama2/kernels/test_rmsnorm.sl:13-39 ([1,2,3,4], w=1).
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_rmsnorm(const float* x, const float* w, float* y, int64_t n, float eps,
                                    int64_t woff) {
  float ss = 0.0f;
  for (int64_t i = 0; i < n; ++i) ss += x[i] * x[i];
  const float r = std::sqrt(ss / float(n) + eps);
  for (int64_t i = 0; i < n; ++i) y[i] = (x[i] / r) * w[woff + i];
}

// ---------------------------------------------------------------------------
// softmax (SoftmaxOpLowering, ConvertSimpToMemRef.cpp:2264-2316):
//   m = x[xoff]; for i in 1..n-1: if x[xoff+i] > m (ordered): m = x[xoff+i]
//   y[yoff+i] = expf(x[xoff+i]-m); s += y[yoff+i];  y[yoff+i] /= s
// Pinned by examples/llama2/kernels/test_softmax_host.cpp:34-38.
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_softmax(const float* x, float* y, int64_t n, int64_t xoff,
                                    int64_t yoff) {
  if (n <= 0) return;
  float m = x[xoff];
  for (int64_t i = 1; i < n; ++i)
    if (x[xoff + i] > m) m = x[xoff + i];
  float s = 0.0f;
  for (int64_t i = 0; i < n; ++i) {
    const float e = std::exp(x[xoff + i] - m);
    y[yoff + i] = e;
    s += e;
  }
  for (int64_t i = 0; i < n; ++i) y[yoff + i] = y[yoff + i] / s;
}

// ---------------------------------------------------------------------------
// silu (SiLUOpLowering, ConvertSimpToMemRef.cpp:2345-2354): y = x / (1 + expf(-x)).
// mul != nullptr is the SwiGLU product every model applies right after
// (examples/llama2/stories110M.sl:202-212): y = silu(x) * mul.
// Pinned by examples/llama2/kernels/test_silu_host.cpp:31-36 and test_swiglu_host.cpp:33-41.
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_silu(const float* x, const float* mul, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const float s = x[i] / (1.0f + std::exp(-x[i]));
    y[i] = mul ? s * mul[i] : s;
  }
}

// ---------------------------------------------------------------------------
// int8 quantise / dequantise: scalar model code, not ops
// (examples/llama2/llama32_1b_int8_tensor.sl:96-103, 227; the prefill variant
// omits the clamp, llama32_1b_int8_prefill.sl:48; f32->int cast truncates toward
// zero, src/mlir/mlir_codegen.cpp:866-869).
//   quantise : v = x*scale; clamp ? v = min(max(v,-128),127); y = (int8) trunc(v)
//              (without the clamp the i32 truncation is narrowed modulo 256)
//   dequant  : y = float(acc) / divisor                   (65536.0 in the model)
// Parity unpinned beyond the formulas: the reference has no test for them.
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_quantize_i8(const float* x, int8_t* y, int64_t n, float scale,
                                        int clamp) {
  for (int64_t i = 0; i < n; ++i) {
    float v = x[i] * scale;
    if (clamp) {
      if (v < -128.0f) v = -128.0f;
      if (v > 127.0f) v = 127.0f;
      y[i] = int8_t(int32_t(v));
    } else {
      // keep the conversion defined for the test ranges: saturate to i32 first
      if (v < -2147483648.0f) v = -2147483648.0f;
      if (v > 2147483520.0f) v = 2147483520.0f;
      y[i] = int8_t(uint8_t(uint32_t(int32_t(v)) & 0xffu));
    }
  }
}
ORACLE_API void simp_oracle_dequantize_i32(const int32_t* acc, float* y, int64_t n, float divisor) {
  for (int64_t i = 0; i < n; ++i) y[i] = float(acc[i]) / divisor;
}

// ---------------------------------------------------------------------------
// Whole-token LLaMA forward, f32 weights (examples/llama2/stories110M.sl:5-247)
// and W4 weights (examples/llama2/llama2_quant.sl:7-198), one restatement with
// the projection step switched.  Deviations from the .sl text, all stated in
// the project's design notes:
//   * the score divisor is sqrtf(head_size) instead of the literal 8.0
//     (identical for head_size 64; llama2_quant.sl:112 already uses sqrt);
//   * the W4 model applies the same RoPE as the f32 one (the reference's W4
//     model has none, llama2_quant.sl:81-93);
//   * W4 projections use scale_mode 1 of simp_oracle_matmul_quant.
// Tensor order and layouts follow the .sl argument list: per-layer matrices
// are stacked [n_layers, rows, cols]; KV cache is [n_layers, seq_len, kv_dim].
// Parity unpinned: the reference only checks that logits are finite
// (examples/llama2/test_stories110M.cpp:186-187).
// ---------------------------------------------------------------------------
struct SimpOracleLlama {
  int64_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len;
  int64_t w4;          // 0: f32 projections, 1: W4 projections
  int64_t group_size;  // W4 only
  // f32 tensors
  const float* token_embedding;  // [vocab, dim]
  const float* rms_att_w;        // [L, dim]
  const float* rms_ffn_w;        // [L, dim]
  const float* rms_final_w;      // [dim]
  const float* wcls;             // [vocab, dim]
  // f32 projections (w4 == 0)
  const float *wq, *wk, *wv, *wo, *w1, *w2, *w3;
  // W4 projections (w4 == 1): one byte array + scale/zero arrays, element offsets per family
  const uint8_t* qweights;
  const float* scales;
  const float* zeros;  // may be null (symmetric)
  int64_t wq_off, wk_off, wv_off, wo_off, w1_off, w2_off, w3_off;
  // state
  float* key_cache;    // [L, seq_len, kv_dim]
  float* value_cache;  // [L, seq_len, kv_dim]
  float* logits;       // [vocab]
  int32_t threads;
};

static void proj(const SimpOracleLlama& m, const float* wf, int64_t w4_off, int64_t layer,
                 int64_t rows, int64_t cols, const float* x, float* out) {
  if (m.w4) {
    simp_oracle_matmul_quant(m.qweights, m.scales, m.zeros, x, out, rows, cols, m.group_size,
                             w4_off + layer * rows * cols, 1, m.threads);
  } else {
    std::fill(out, out + rows, 0.0f);
    simp_oracle_matmul_f32(wf, layer * rows * cols, x, 0, out, 0, rows, cols, 1, m.threads);
  }
}

ORACLE_API int simp_oracle_llama_forward(const SimpOracleLlama* mp, int64_t token, int64_t pos) {
  const SimpOracleLlama& m = *mp;
  const int64_t dim = m.dim, hd = m.hidden_dim, hs = dim / m.n_heads;
  const int64_t kv_dim = dim * m.n_kv_heads / m.n_heads;
  if (pos < 0 || pos >= m.seq_len || token < 0 || token >= m.vocab_size) return -1;
  std::vector<float> x(dim), xb(dim), xb2(std::max(dim, hd)), hb(hd), hbs(hd), q(dim),
      k(kv_dim), v(kv_dim), att(m.seq_len), atts(m.seq_len);
  for (int64_t i = 0; i < dim; ++i) x[i] = m.token_embedding[token * dim + i];
  const float inv_div = std::sqrt(float(hs));
  for (int64_t l = 0; l < m.n_layers; ++l) {
    simp_oracle_rmsnorm(x.data(), m.rms_att_w, xb.data(), dim, 1e-5f, l * dim);
    proj(m, m.wq, m.wq_off, l, dim, dim, xb.data(), q.data());
    proj(m, m.wk, m.wk_off, l, kv_dim, dim, xb.data(), k.data());
    proj(m, m.wv, m.wv_off, l, kv_dim, dim, xb.data(), v.data());
    // RoPE on (even, odd) pairs (stories110M.sl:86-112)
    for (int64_t i = 0; i < dim; i += 2) {
      const float freq = 1.0f / std::pow(10000.0f, float(i % hs) / float(hs));
      const float val = float(pos) * freq;
      const float fcr = std::cos(val), fci = std::sin(val);
      const float q0 = q[i], q1 = q[i + 1];
      q[i] = q0 * fcr - q1 * fci;
      q[i + 1] = q0 * fci + q1 * fcr;
      if (i < kv_dim) {
        const float k0 = k[i], k1 = k[i + 1];
        k[i] = k0 * fcr - k1 * fci;
        k[i + 1] = k0 * fci + k1 * fcr;
      }
    }
    float* kc = m.key_cache + l * m.seq_len * kv_dim;
    float* vc = m.value_cache + l * m.seq_len * kv_dim;
    for (int64_t i = 0; i < kv_dim; ++i) {
      kc[pos * kv_dim + i] = k[i];
      vc[pos * kv_dim + i] = v[i];
    }
    for (int64_t h = 0; h < m.n_heads; ++h) {
      const int64_t qo = h * hs;
      const int64_t kvo = (h * m.n_kv_heads / m.n_heads) * hs;
      for (int64_t t = 0; t <= pos; ++t) {
        float score = 0.0f;
        for (int64_t i = 0; i < hs; ++i) score += q[qo + i] * kc[t * kv_dim + kvo + i];
        att[t] = score / inv_div;
      }
      simp_oracle_softmax(att.data(), atts.data(), pos + 1, 0, 0);
      for (int64_t i = 0; i < hs; ++i) {
        float val = 0.0f;
        for (int64_t t = 0; t <= pos; ++t) val += atts[t] * vc[t * kv_dim + kvo + i];
        xb[qo + i] = val;
      }
    }
    proj(m, m.wo, m.wo_off, l, dim, dim, xb.data(), xb2.data());
    for (int64_t i = 0; i < dim; ++i) x[i] += xb2[i];
    simp_oracle_rmsnorm(x.data(), m.rms_ffn_w, xb.data(), dim, 1e-5f, l * dim);
    proj(m, m.w1, m.w1_off, l, hd, dim, xb.data(), hb.data());
    simp_oracle_silu(hb.data(), nullptr, hbs.data(), hd);
    proj(m, m.w3, m.w3_off, l, hd, dim, xb.data(), xb2.data());
    for (int64_t i = 0; i < hd; ++i) hb[i] = hbs[i] * xb2[i];
    proj(m, m.w2, m.w2_off, l, dim, hd, hb.data(), xb.data());
    for (int64_t i = 0; i < dim; ++i) x[i] += xb[i];
  }
  simp_oracle_rmsnorm(x.data(), m.rms_final_w, xb.data(), dim, 1e-5f, 0);
  std::fill(m.logits, m.logits + m.vocab_size, 0.0f);
  simp_oracle_matmul_f32(m.wcls, 0, xb.data(), 0, m.logits, 0, m.vocab_size, dim, 1, m.threads);
  return 0;
}

// argmax with the host's tie rule: strict '>' so the lowest index wins
// (examples/llama2/generate_stories110M.cpp:73-83).
ORACLE_API int64_t simp_oracle_argmax(const float* v, int64_t n) {
  int64_t best = 0;
  for (int64_t i = 1; i < n; ++i)
    if (v[i] > v[best]) best = i;
  return best;
}

// ---------------------------------------------------------------------------
// Whole-token forward of the int8 LLaMA-3.2-1B-style model
// (examples/llama2/llama32_1b_int8_tensor.sl:16-305): f32 residual stream and norms, int8
// activations and weights ([N,K] pre-transposed), i32 accumulation (tensor_matmul_nt), int8 KV
// cache, grouped-query attention, f32 classifier.  Restated literally, including what the .sl
// text leaves out or hard-codes:
//   * no RoPE is applied (the loop at :124-140 computes the angles and discards them);
//   * the score divisor is the literal 8.0 (:178), whatever head_dim is;
//   * K and V enter the cache as (i8)(acc / 256) -- integer division truncating toward zero, then
//     a narrowing that keeps the low 8 bits (:146-149);
//   * attn_out = (i32) trunc(weighted sum) (:196); the next input is clamp(attn_out / 256.0) (:207-213);
//   * the FFN activation (i8)(silu(gate/65536) * (up/65536) * 127) has no clamp (:258-265): the f32->i8
//     cast is taken as truncation to i32 followed by narrowing modulo 256 (what the x86 code does);
//   * residual updates x += (f32)acc / 65536.0 (:227, :275).
// f32 sums run sequentially in index order, as the scalar loops of the lowering do.
// Parity unpinned: the reference holds no known-answer test for this model (its host,
// bench_llama32_1b_int8.cpp, only times it).
// ---------------------------------------------------------------------------
struct SimpOracleLlamaI8 {
  int64_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, max_seq_len, head_dim;
  const float *rms_att_w, *rms_ffn_w, *rms_final_w, *wcls;
  const int8_t *wq_t, *wk_t, *wv_t, *wo_t, *w1_t, *w2_t, *w3_t;
  int8_t *k_cache, *v_cache;  // [n_layers, max_seq_len, kv_dim], caller-owned
};

namespace {
// tensor_matmul_nt with M = 1: out[j] = sum_p (i32)x[p] * (i32)Wt[j*K + p]
void matvec_nt_i8(const int8_t* x, const int8_t* Wt, int32_t* out, int64_t N, int64_t K, int nt) {
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t j = 0; j < N; ++j) {
    int32_t acc = 0;
    const int8_t* w = Wt + j * K;
    for (int64_t p = 0; p < K; ++p) acc += int32_t(x[p]) * int32_t(w[p]);
    out[j] = acc;
  }
}
inline int8_t quant_clamped(float v) {
  if (v > 127.0f) v = 127.0f;
  if (v < -128.0f) v = -128.0f;
  return int8_t(int32_t(v));
}
}  // namespace

ORACLE_API void simp_oracle_llama_i8_forward(const SimpOracleLlamaI8* mp, const int8_t* x_i8, int64_t pos,
                                             float* logits, int threads) {
  const SimpOracleLlamaI8& m = *mp;
  const int nt = clamp_threads(threads);
  const int64_t dim = m.dim, hd = m.hidden_dim, hs = m.head_dim;
  const int64_t kv_dim = m.n_kv_heads * hs, n_rep = m.n_heads / m.n_kv_heads, seq_len = pos + 1;
  std::vector<float> x(dim), xb(dim), att_scores(m.n_heads * m.max_seq_len), att_probs(m.n_heads * m.max_seq_len);
  std::vector<int8_t> xb_i8(dim), ffn_hb(hd);
  std::vector<int32_t> Q(dim), K(kv_dim), V(kv_dim), attn_out(dim), Wo(dim), Gate(hd), Up(hd), Down(dim);
  for (int64_t i = 0; i < dim; ++i) x[i] = float(x_i8[i]) * 1.0f;
  for (int64_t layer = 0; layer < m.n_layers; ++layer) {
    simp_oracle_rmsnorm(x.data(), m.rms_att_w, xb.data(), dim, 0.00001f, layer * dim);
    for (int64_t i = 0; i < dim; ++i) xb_i8[i] = quant_clamped(xb[i] * 127.0f);
    matvec_nt_i8(xb_i8.data(), m.wq_t + layer * dim * dim, Q.data(), dim, dim, nt);
    matvec_nt_i8(xb_i8.data(), m.wk_t + layer * kv_dim * dim, K.data(), kv_dim, dim, nt);
    matvec_nt_i8(xb_i8.data(), m.wv_t + layer * kv_dim * dim, V.data(), kv_dim, dim, nt);
    const int64_t cache_offset = layer * m.max_seq_len * kv_dim + pos * kv_dim;
    for (int64_t i = 0; i < kv_dim; ++i) {
      m.k_cache[cache_offset + i] = int8_t(uint8_t(uint32_t(K[i] / 256) & 0xffu));
      m.v_cache[cache_offset + i] = int8_t(uint8_t(uint32_t(V[i] / 256) & 0xffu));
    }
    for (int64_t i = 0; i < dim; ++i) attn_out[i] = 0;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t h = 0; h < m.n_heads; ++h) {
      const int64_t q_offset = h * hs, kv_head_offset = (h / n_rep) * hs, att_offset = h * m.max_seq_len;
      for (int64_t t = 0; t < seq_len; ++t) {
        float score = 0.0f;
        const int64_t k_pos = layer * m.max_seq_len * kv_dim + t * kv_dim + kv_head_offset;
        for (int64_t d = 0; d < hs; ++d) score = score + float(Q[q_offset + d]) * float(m.k_cache[k_pos + d]);
        att_scores[att_offset + t] = score / 8.0f;
      }
      simp_oracle_softmax(att_scores.data(), att_probs.data(), seq_len, att_offset, att_offset);
      for (int64_t d = 0; d < hs; ++d) {
        float val = 0.0f;
        for (int64_t t = 0; t < seq_len; ++t) {
          const int64_t v_pos = layer * m.max_seq_len * kv_dim + t * kv_dim + kv_head_offset;
          val = val + att_probs[att_offset + t] * float(m.v_cache[v_pos + d]);
        }
        attn_out[q_offset + d] = int32_t(val);
      }
    }
    for (int64_t i = 0; i < dim; ++i) xb_i8[i] = quant_clamped(float(attn_out[i]) / 256.0f);
    matvec_nt_i8(xb_i8.data(), m.wo_t + layer * dim * dim, Wo.data(), dim, dim, nt);
    for (int64_t i = 0; i < dim; ++i) x[i] = x[i] + float(Wo[i]) / 65536.0f;
    simp_oracle_rmsnorm(x.data(), m.rms_ffn_w, xb.data(), dim, 0.00001f, layer * dim);
    for (int64_t i = 0; i < dim; ++i) xb_i8[i] = quant_clamped(xb[i] * 127.0f);
    matvec_nt_i8(xb_i8.data(), m.w1_t + layer * hd * dim, Gate.data(), hd, dim, nt);
    matvec_nt_i8(xb_i8.data(), m.w3_t + layer * hd * dim, Up.data(), hd, dim, nt);
    for (int64_t i = 0; i < hd; ++i) {
      const float gate_f = float(Gate[i]) / 65536.0f;
      const float silu = gate_f / (1.0f + std::exp(0.0f - gate_f));
      const float up_f = float(Up[i]) / 65536.0f;
      float hb_val = silu * up_f * 127.0f;
      if (hb_val < -2147483648.0f) hb_val = -2147483648.0f;  // keep the conversion defined
      if (hb_val > 2147483520.0f) hb_val = 2147483520.0f;
      ffn_hb[i] = int8_t(uint8_t(uint32_t(int32_t(hb_val)) & 0xffu));
    }
    matvec_nt_i8(ffn_hb.data(), m.w2_t + layer * dim * hd, Down.data(), dim, hd, nt);
    for (int64_t i = 0; i < dim; ++i) x[i] = x[i] + float(Down[i]) / 65536.0f;
  }
  simp_oracle_rmsnorm(x.data(), m.rms_final_w, xb.data(), dim, 0.00001f, 0);
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < m.vocab_size; ++i) {
    float sum = 0.0f;
    const float* w = m.wcls + i * dim;
    for (int64_t j = 0; j < dim; ++j) sum = sum + w[j] * xb[j];
    logits[i] = sum;
  }
}

// ---------------------------------------------------------------------------
// Prefill of the same int8 model over seq_len tokens at once
// (examples/llama2/llama32_1b_int8_prefill.sl:11-232; the six exported variants differ only in the
// compile-time seq_len 8 ... 256).  Differences from the single-token text, all kept:
//   * rmsnorm is x * (1 / sqrt(mean(x^2) + 1e-5)) * w (reciprocal, left to right), computed inline (:33-51);
//   * no quantisation step clamps (:48, :148, :183, :209): f32 -> i8 is taken as truncation to i32 followed by
//     narrowing modulo 256, as for the FFN activation of the single-token model;
//   * causal attention with the softmax written out (:81-141); the cache of a layer is [seq_len, kv_dim] (:69);
//   * there is no final norm or classifier: the result is the residual stream x_fp32 [seq_len, dim] (:231).
// Parity unpinned (no known-answer test in the reference).
// ---------------------------------------------------------------------------
namespace {
inline int8_t narrow_f32_to_i8(float v) {
  if (v < -2147483648.0f) v = -2147483648.0f;  // keep the conversion defined
  if (v > 2147483520.0f) v = 2147483520.0f;
  return int8_t(uint8_t(uint32_t(int32_t(v)) & 0xffu));
}
// tensor_matmul_nt: C[t, j] = sum_p A[t, p] * Wt[j, p]
void matmul_nt_i8(const int8_t* A, const int8_t* Wt, int32_t* C, int64_t M, int64_t N, int64_t K, int nt) {
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t j = 0; j < N; ++j) {
    const int8_t* w = Wt + j * K;
    for (int64_t t = 0; t < M; ++t) {
      const int8_t* a = A + t * K;
      int32_t acc = 0;
      for (int64_t p = 0; p < K; ++p) acc += int32_t(a[p]) * int32_t(w[p]);
      C[t * N + j] = acc;
    }
  }
}
}  // namespace

ORACLE_API void simp_oracle_llama_i8_prefill(const SimpOracleLlamaI8* mp, const int8_t* x_i8, int64_t seq_len,
                                             float* x_fp32, int8_t* k_cache, int8_t* v_cache, int threads) {
  const SimpOracleLlamaI8& m = *mp;
  const int nt = clamp_threads(threads);
  const int64_t dim = m.dim, hd = m.hidden_dim, hs = m.head_dim, S = seq_len;
  const int64_t kv_dim = m.n_kv_heads * hs, n_rep = m.n_heads / m.n_kv_heads;
  std::vector<float> xb(S * dim), att_scores(m.n_heads * S * S), att_probs(m.n_heads * S * S);
  std::vector<int8_t> xb_i8(S * dim), ffn_hb(S * hd);
  std::vector<int32_t> Q(S * dim), K(S * kv_dim), V(S * kv_dim), attn_out(S * dim), Wo(S * dim), Gate(S * hd), Up(S * hd), Down(S * dim);
  for (int64_t i = 0; i < S * dim; ++i) x_fp32[i] = float(x_i8[i]) * 1.0f;
  auto norm_quant = [&](const float* w) {
    for (int64_t t = 0; t < S; ++t) {
      const int64_t o = t * dim;
      float ss = 0.0f;
      for (int64_t i = 0; i < dim; ++i) ss = ss + x_fp32[o + i] * x_fp32[o + i];
      ss = 1.0f / std::sqrt(ss / (float(dim) * 1.0f) + 0.00001f);
      for (int64_t i = 0; i < dim; ++i) {
        xb[o + i] = x_fp32[o + i] * ss * w[i];
        xb_i8[o + i] = narrow_f32_to_i8(xb[o + i] * 127.0f);
      }
    }
  };
  for (int64_t layer = 0; layer < m.n_layers; ++layer) {
    norm_quant(m.rms_att_w + layer * dim);
    matmul_nt_i8(xb_i8.data(), m.wq_t + layer * dim * dim, Q.data(), S, dim, dim, nt);
    matmul_nt_i8(xb_i8.data(), m.wk_t + layer * kv_dim * dim, K.data(), S, kv_dim, dim, nt);
    matmul_nt_i8(xb_i8.data(), m.wv_t + layer * kv_dim * dim, V.data(), S, kv_dim, dim, nt);
    const int64_t cl = layer * S * kv_dim;
    for (int64_t i = 0; i < S * kv_dim; ++i) {
      k_cache[cl + i] = int8_t(uint8_t(uint32_t(K[i] / 256) & 0xffu));
      v_cache[cl + i] = int8_t(uint8_t(uint32_t(V[i] / 256) & 0xffu));
    }
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
    for (int64_t h = 0; h < m.n_heads; ++h) {
      const int64_t qo = h * hs, ko = (h / n_rep) * hs;
      for (int64_t q_pos = 0; q_pos < S; ++q_pos) {
        const int64_t ao = h * S * S + q_pos * S;
        for (int64_t k_pos = 0; k_pos <= q_pos; ++k_pos) {
          float score = 0.0f;
          for (int64_t d = 0; d < hs; ++d)
            score = score + float(Q[q_pos * dim + qo + d]) * 1.0f * float(k_cache[cl + k_pos * kv_dim + ko + d]) * 1.0f;
          att_scores[ao + k_pos] = score / 8.0f;
        }
        float max_val = att_scores[ao];
        for (int64_t ki = 1; ki <= q_pos; ++ki)
          if (att_scores[ao + ki] > max_val) max_val = att_scores[ao + ki];
        float sum_exp = 0.0f;
        for (int64_t ki = 0; ki <= q_pos; ++ki) {
          const float e = std::exp(att_scores[ao + ki] - max_val);
          att_probs[ao + ki] = e;
          sum_exp = sum_exp + e;
        }
        for (int64_t ki = 0; ki <= q_pos; ++ki) att_probs[ao + ki] = att_probs[ao + ki] / sum_exp;
        for (int64_t d = 0; d < hs; ++d) {
          float val = 0.0f;
          for (int64_t vi = 0; vi <= q_pos; ++vi)
            val = val + att_probs[ao + vi] * float(v_cache[cl + vi * kv_dim + ko + d]) * 1.0f;
          attn_out[q_pos * dim + qo + d] = int32_t(val);
        }
      }
    }
    for (int64_t i = 0; i < S * dim; ++i) xb_i8[i] = narrow_f32_to_i8(float(attn_out[i]) * 1.0f / 256.0f);
    matmul_nt_i8(xb_i8.data(), m.wo_t + layer * dim * dim, Wo.data(), S, dim, dim, nt);
    for (int64_t i = 0; i < S * dim; ++i) x_fp32[i] = x_fp32[i] + float(Wo[i]) * 1.0f / 65536.0f;
    norm_quant(m.rms_ffn_w + layer * dim);
    matmul_nt_i8(xb_i8.data(), m.w1_t + layer * hd * dim, Gate.data(), S, hd, dim, nt);
    matmul_nt_i8(xb_i8.data(), m.w3_t + layer * hd * dim, Up.data(), S, hd, dim, nt);
    for (int64_t i = 0; i < S * hd; ++i) {
      const float gate_f = float(Gate[i]) * 1.0f / 65536.0f;
      const float silu = gate_f / (1.0f + std::exp(0.0f - gate_f));
      const float up_f = float(Up[i]) * 1.0f / 65536.0f;
      ffn_hb[i] = narrow_f32_to_i8(silu * up_f * 127.0f);
    }
    matmul_nt_i8(ffn_hb.data(), m.w2_t + layer * dim * hd, Down.data(), S, dim, hd, nt);
    for (int64_t i = 0; i < S * dim; ++i) x_fp32[i] = x_fp32[i] + float(Down[i]) * 1.0f / 65536.0f;
  }
}

// ---------------------------------------------------------------------------
// tensor_matmul on packed i4 (TensorMatMulOpLowering, packed-i4 branch,
// src/mlir/lowering/ConvertSimpToMemRef.cpp:2953-3133): operands hold two signed 4-bit values per byte along
// their LAST dimension (low nibble = even index; A is [M, K/2] bytes, B is [K, N/2] bytes); both are unpacked
// with sign extension, C[i, j] = (i16) trunc( sum_k (i32) a[i,k] * b[k,j] ), a fresh [M, N] i16 result.
// Pinned by the reference's runner: scalar_matmul_int4<N> / packed_matmul_int4<N> checksums on the
// ((i*N+j)%15)-7 fill (simptensor/benchmarks/bench_int4_matmul_runner.cpp:34-148; the .sl kernels being timed are
// simptensor/benchmarks/bench_int4_matmul.sl:16-47).
// ---------------------------------------------------------------------------
namespace {
inline int32_t nibble_s4(uint8_t byte, int64_t idx) {
  const int32_t n = (idx & 1) ? (byte >> 4) & 15 : byte & 15;
  return n >= 8 ? n - 16 : n;
}
}  // namespace
ORACLE_API void simp_oracle_tensor_matmul_i4(const uint8_t* A, const uint8_t* B, int16_t* C, int64_t M,
                                             int64_t K, int64_t N, int threads) {
  const int nt = clamp_threads(threads);
  const int64_t ak = (K + 1) / 2, bn = (N + 1) / 2;
#pragma omp parallel for num_threads(nt) schedule(static) if (nt > 1)
  for (int64_t i = 0; i < M; ++i)
    for (int64_t j = 0; j < N; ++j) {
      int32_t acc = 0;
      for (int64_t k = 0; k < K; ++k) acc += nibble_s4(A[i * ak + (k >> 1)], k) * nibble_s4(B[k * bn + (j >> 1)], j);
      C[i * N + j] = int16_t(uint16_t(uint32_t(acc) & 0xffffu));
    }
}

// ---------------------------------------------------------------------------
// tensor_gather (TensorGatherOpLowering, src/mlir/lowering/ConvertSimpToMemRef.cpp:2625-2776):
//   result[..., n, ...] = source[..., indices[n], ...] along `axis`; indices are i64; every other dimension is
//   copied whole.  With the source viewed as [outer, axis_dim, inner] this is dst[o, n, :] = src[o, indices[n], :].
// Elements are opaque (elem_size bytes).  Pinned by simptensor/tests/test_scatter_gather.sl:8-147 (eight known
// answers, expected values in test_scatter_gather_host.cpp:61-68).
// ---------------------------------------------------------------------------
ORACLE_API int simp_oracle_tensor_gather(const uint8_t* src, const int64_t* indices, uint8_t* dst, int64_t outer,
                                         int64_t axis_dim, int64_t inner, int64_t n_idx, int64_t elem_size) {
  const int64_t row = inner * elem_size;
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t n = 0; n < n_idx; ++n) {
      const int64_t s = indices[n];
      if (s < 0 || s >= axis_dim) return -1;   // the reference leaves this undefined
      std::memcpy(dst + (o * n_idx + n) * row, src + (o * axis_dim + s) * row, size_t(row));
    }
  return 0;
}

// ---------------------------------------------------------------------------
// conv2d (Conv2DOpLowering, src/mlir/lowering/ConvertSimpToMemRef.cpp:1924-2150): NHWC input, weights
// [OC, KH, KW, IC], bias [OC], NHWC output; out_h = (in_h + 2*pad_h - kh) / stride_h + 1 (same for w);
// acc = bias[oc]; for kh, kw, ic in that order: taps outside the input are skipped (zero padding);
// acc = acc + input * weight (separate multiply and add).
// Pinned by tests/mlir/integration/test_conv2d_host.cpp:28-44: a 4x4 ramp 0..15 under a 3x3 kernel of ones, bias 0 --
// the top-left unpadded window sums to 45.0 (with the pad 1 of test_conv2d_fp32_only.sl:17-18 the same window is
// the output at (1, 1)).
// ---------------------------------------------------------------------------
ORACLE_API void simp_oracle_conv2d_f32(const float* input, const float* weights, const float* bias, float* output,
                                       int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t out_c,
                                       int64_t kh, int64_t kw, int64_t stride_h, int64_t stride_w, int64_t pad_h,
                                       int64_t pad_w, int threads) {
  const int nt = clamp_threads(threads);
  const int64_t out_h = (in_h + 2 * pad_h - kh) / stride_h + 1, out_w = (in_w + 2 * pad_w - kw) / stride_w + 1;
#pragma omp parallel for num_threads(nt) schedule(static) collapse(2) if (nt > 1)
  for (int64_t b = 0; b < batch; ++b)
    for (int64_t oh = 0; oh < out_h; ++oh)
      for (int64_t ow = 0; ow < out_w; ++ow)
        for (int64_t oc = 0; oc < out_c; ++oc) {
          volatile float acc = bias[oc];   // volatile: keeps the multiply and the add separate (no contraction)
          for (int64_t y = 0; y < kh; ++y)
            for (int64_t x = 0; x < kw; ++x)
              for (int64_t ic = 0; ic < in_c; ++ic) {
                const int64_t ih = oh * stride_h + y - pad_h, iw = ow * stride_w + x - pad_w;
                if (ih < 0 || ih >= in_h || iw < 0 || iw >= in_w) continue;
                volatile float prod = input[((b * in_h + ih) * in_w + iw) * in_c + ic] * weights[((oc * kh + y) * kw + x) * in_c + ic];
                acc = acc + prod;
              }
          output[((b * out_h + oh) * out_w + ow) * out_c + oc] = acc;
        }
}
