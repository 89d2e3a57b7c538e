// rowops.cu -- rmsnorm, softmax, silu, int8 quantise/dequantise, W4 range dequantise.
//
// All of these are HBM-bound: each kernel reads its input once into registers,
// reduces with warp shuffles (+ one shared-memory hop per block), and writes once.
// Arithmetic follows the reference lowering term by term (IEEE division, expf; no
// fast-math), only the summation order differs (tree instead of sequential):
//   rmsnorm  src/mlir/lowering/ConvertSimpToMemRef.cpp:2192-2230
//   softmax  src/mlir/lowering/ConvertSimpToMemRef.cpp:2264-2316
//   silu     src/mlir/lowering/ConvertSimpToMemRef.cpp:2345-2354
#include "common.cuh"

namespace simp {

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------------- rmsnorm
// One block per row; thread t owns float4 slots t, t+T, ... (VPT of them) held in registers.
template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(float* __restrict__ x, const float* __restrict__ w,
                                                          float* __restrict__ y, int n4, float nf, float eps,
                                                          int64_t row_stride, const float* __restrict__ residual) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  float4* xr = reinterpret_cast<float4*>(x + row * row_stride);
  const float4* rr = residual ? reinterpret_cast<const float4*>(residual + row * row_stride) : nullptr;
  float4* yr = reinterpret_cast<float4*>(y + row * row_stride);
  const float4* wr = reinterpret_cast<const float4*>(w);
  float4 v[VPT];
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4) {
      v[i] = xr[idx];
      if (rr) {
        const float4 r = rr[idx];
        v[i].x += r.x; v[i].y += r.y; v[i].z += r.z; v[i].w += r.w;
        xr[idx] = v[i];
      }
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = block_sum(ss, red);
  const float r = sqrtf(ss / nf + eps);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4) {
      const float4 ww = __ldg(wr + idx);
      float4 o;
      o.x = (v[i].x / r) * ww.x; o.y = (v[i].y / r) * ww.y;
      o.z = (v[i].z / r) * ww.z; o.w = (v[i].w / r) * ww.w;
      yr[idx] = o;
    }
  }
}

// Any n / alignment: two passes over the row (the second one hits L1/L2).
__global__ void __launch_bounds__(256) rmsnorm_any_kernel(float* __restrict__ x, const float* __restrict__ w,
                                                          float* __restrict__ y, int64_t n, float nf, float eps,
                                                          int64_t row_stride, const float* __restrict__ residual) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  float* xr = x + row * row_stride;
  const float* rr = residual ? residual + row * row_stride : nullptr;
  float* yr = y + row * row_stride;
  float ss = 0.0f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float v = xr[i];
    if (rr) {
      v += rr[i];
      xr[i] = v;
    }
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float r = sqrtf(ss / nf + eps);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = (xr[i] / r) * w[i];
}

// ---------------------------------------------------------------------------------- softmax
template <int VPT>
__global__ void __launch_bounds__(256) softmax_vec_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          int n4, int64_t row_stride) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + row * row_stride);
  float4* yr = reinterpret_cast<float4*>(y + row * row_stride);
  float4 v[VPT];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4) {
      v[i] = xr[idx];
      m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    }
  }
  m = block_max(m, red);
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4) {
      v[i].x = expf(v[i].x - m); v[i].y = expf(v[i].y - m);
      v[i].z = expf(v[i].z - m); v[i].w = expf(v[i].w - m);
      s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    }
  }
  s = block_sum(s, red);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    if (idx < n4) {
      float4 o;
      o.x = v[i].x / s; o.y = v[i].y / s; o.z = v[i].z / s; o.w = v[i].w / s;
      yr[idx] = o;
    }
  }
}

// Any n / alignment.  The exponentials are parked in y (as the reference does) and rescaled.
__global__ void __launch_bounds__(256) softmax_any_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                          int64_t n, int64_t row_stride) {
  __shared__ float red[33];
  const int64_t row = blockIdx.x;
  const float* xr = x + row * row_stride;
  float* yr = y + row * row_stride;
  float m = -INFINITY;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, xr[i]);
  m = block_max(m, red);
  float s = 0.0f;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const float e = expf(xr[i] - m);
    yr[i] = e;
    s += e;
  }
  s = block_sum(s, red);
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) yr[i] = yr[i] / s;
}

// ---------------------------------------------------------------------------------- silu
__device__ __forceinline__ float silu1(float v) { return v / (1.0f + expf(-v)); }

__global__ void __launch_bounds__(256) silu_kernel(const float* __restrict__ x, const float* __restrict__ mul,
                                                   float* __restrict__ y, int64_t n, int vec_ok) {
  const int64_t tid = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int64_t nthreads = int64_t(gridDim.x) * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* m4 = reinterpret_cast<const float4*>(mul);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (int64_t i = tid; i < n4; i += nthreads) {
      const float4 v = x4[i];
      float4 o;
      o.x = silu1(v.x); o.y = silu1(v.y); o.z = silu1(v.z); o.w = silu1(v.w);
      if (mul) {
        const float4 g = m4[i];
        o.x *= g.x; o.y *= g.y; o.z *= g.z; o.w *= g.w;
      }
      y4[i] = o;
    }
    done = n4 << 2;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) {
    const float s = silu1(x[i]);
    y[i] = mul ? s * mul[i] : s;
  }
}

// ---------------------------------------------------------------------------------- int8 quantise / dequantise
__device__ __forceinline__ int8_t quant1(float x, float scale, int clamp) {
  float v = x * scale;
  if (clamp) {
    v = fminf(fmaxf(v, -128.0f), 127.0f);
    return (int8_t)__float2int_rz(v);
  }
  return (int8_t)(uint8_t)(((uint32_t)__float2int_rz(v)) & 0xffu);  // cvt.rzi.s32 saturates, then narrow mod 256
}

__global__ void __launch_bounds__(256) quantize_i8_kernel(const float* __restrict__ x, int8_t* __restrict__ y,
                                                          int64_t n, float scale, int clamp, int vec_ok) {
  const int64_t tid = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int64_t nthreads = int64_t(gridDim.x) * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    char4* y4 = reinterpret_cast<char4*>(y);
    for (int64_t i = tid; i < n4; i += nthreads) {
      const float4 v = x4[i];
      char4 o;
      o.x = quant1(v.x, scale, clamp); o.y = quant1(v.y, scale, clamp);
      o.z = quant1(v.z, scale, clamp); o.w = quant1(v.w, scale, clamp);
      y4[i] = o;
    }
    done = n4 << 2;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) y[i] = quant1(x[i], scale, clamp);
}

__global__ void __launch_bounds__(256) dequantize_i32_kernel(const int32_t* __restrict__ a, float* __restrict__ y,
                                                             int64_t n, float divisor, int vec_ok) {
  const int64_t tid = blockIdx.x * int64_t(blockDim.x) + threadIdx.x;
  const int64_t nthreads = int64_t(gridDim.x) * blockDim.x;
  int64_t done = 0;
  if (vec_ok) {
    const int64_t n4 = n >> 2;
    const int4* a4 = reinterpret_cast<const int4*>(a);
    float4* y4 = reinterpret_cast<float4*>(y);
    for (int64_t i = tid; i < n4; i += nthreads) {
      const int4 v = a4[i];
      float4 o;
      o.x = float(v.x) / divisor; o.y = float(v.y) / divisor;
      o.z = float(v.z) / divisor; o.w = float(v.w) / divisor;
      y4[i] = o;
    }
    done = n4 << 2;
  }
  for (int64_t i = done + tid; i < n; i += nthreads) y[i] = float(a[i]) / divisor;
}

// ---------------------------------------------------------------------------------- W4 range dequantise
// w = q*scale + zero with separate multiply and add, as DequantW4OpLowering emits them
// (ConvertSimpToMemRef.cpp:2419-2424).
__global__ void __launch_bounds__(256) dequant_w4_kernel(const uint8_t* __restrict__ qw, const float* __restrict__ sc,
                                                         const float* __restrict__ zr, int64_t idx0, int64_t count,
                                                         int64_t gs, float* __restrict__ out) {
  const int64_t nthreads = int64_t(gridDim.x) * blockDim.x;
  for (int64_t t = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; t < count; t += nthreads) {
    const int64_t idx = idx0 + t;
    const uint32_t b = qw[idx >> 1];
    const uint32_t q = (idx & 1) ? (b >> 4) : (b & 15u);
    const float s = sc[idx / gs];
    const float z = zr ? zr[idx / gs] : __fmul_rn(-8.0f, s);
    out[t] = __fadd_rn(__fmul_rn(float(q), s), z);
  }
}

static inline int ew_grid(int64_t work_items) {
  const int64_t cap = int64_t(ctx().sm_count) * 8;  // 8 resident 256-thread blocks per SM
  int64_t g = cdiv(work_items, 256);
  if (g < 1) g = 1;
  return int(g < cap ? g : cap);
}

}  // namespace simp

using namespace simp;

SIMP_API int simp_gpu_rmsnorm_f32(float* x, const float* w, float* y, int64_t rows, int64_t n, float eps,
                                  int64_t woff, int64_t row_stride, const float* residual) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(rows >= 0 && n >= 0 && woff >= 0, SIMP_ERR_ARG, "rmsnorm: negative size");
  if (rows == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && w && y, SIMP_ERR_ARG, "rmsnorm: null pointer");
  SIMP_REQUIRE(rows <= 0x7fffffff, SIMP_ERR_SHAPE, "rmsnorm: too many rows");
  if (row_stride == 0) row_stride = n;
  SIMP_REQUIRE(row_stride >= n || rows == 1, SIMP_ERR_ARG, "rmsnorm: row_stride < n");
  cudaStream_t st = ctx().stream;
  const float* wp = w + woff;
  const bool vec = (n % 4 == 0) && (row_stride % 4 == 0) && aligned16(x) && aligned16(y) && aligned16(wp) &&
                   (!residual || aligned16(residual)) && n <= 8192;
  if (vec) {
    const int n4 = int(n / 4);
    int vpt = 1;
    while (vpt < 8 && n4 > 256 * vpt) vpt *= 2;
    int threads = int(cdiv(cdiv(n4, vpt), 32) * 32);
    if (threads > 256) threads = 256;
    const float invn = float(n);
    switch (vpt) {
      case 1: rmsnorm_vec_kernel<1><<<int(rows), threads, 0, st>>>(x, wp, y, n4, invn, eps, row_stride, residual); break;
      case 2: rmsnorm_vec_kernel<2><<<int(rows), threads, 0, st>>>(x, wp, y, n4, invn, eps, row_stride, residual); break;
      case 4: rmsnorm_vec_kernel<4><<<int(rows), threads, 0, st>>>(x, wp, y, n4, invn, eps, row_stride, residual); break;
      default: rmsnorm_vec_kernel<8><<<int(rows), threads, 0, st>>>(x, wp, y, n4, invn, eps, row_stride, residual); break;
    }
  } else {
    const int threads = n >= 256 ? 256 : int(cdiv(n, 32) * 32);
    rmsnorm_any_kernel<<<int(rows), threads, 0, st>>>(x, wp, y, n, float(n), eps, row_stride, residual);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_gpu_softmax_f32(const float* x, float* y, int64_t rows, int64_t n, int64_t xoff, int64_t yoff,
                                  int64_t row_stride) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(rows >= 0 && n >= 0 && xoff >= 0 && yoff >= 0, SIMP_ERR_ARG, "softmax: negative size");
  if (rows == 0 || n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && y, SIMP_ERR_ARG, "softmax: null pointer");
  SIMP_REQUIRE(rows <= 0x7fffffff, SIMP_ERR_SHAPE, "softmax: too many rows");
  if (row_stride == 0) row_stride = n;
  cudaStream_t st = ctx().stream;
  const float* xp = x + xoff;
  float* yp = y + yoff;
  const bool vec = (n % 4 == 0) && (row_stride % 4 == 0) && aligned16(xp) && aligned16(yp) && n <= 8192;
  if (vec) {
    const int n4 = int(n / 4);
    int vpt = 1;
    while (vpt < 8 && n4 > 256 * vpt) vpt *= 2;
    int threads = int(cdiv(cdiv(n4, vpt), 32) * 32);
    if (threads > 256) threads = 256;
    switch (vpt) {
      case 1: softmax_vec_kernel<1><<<int(rows), threads, 0, st>>>(xp, yp, n4, row_stride); break;
      case 2: softmax_vec_kernel<2><<<int(rows), threads, 0, st>>>(xp, yp, n4, row_stride); break;
      case 4: softmax_vec_kernel<4><<<int(rows), threads, 0, st>>>(xp, yp, n4, row_stride); break;
      default: softmax_vec_kernel<8><<<int(rows), threads, 0, st>>>(xp, yp, n4, row_stride); break;
    }
  } else {
    const int threads = n >= 256 ? 256 : int(cdiv(n, 32) * 32);
    softmax_any_kernel<<<int(rows), threads, 0, st>>>(xp, yp, n, row_stride);
  }
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_gpu_silu_f32(const float* x, const float* mul, float* y, int64_t n) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(n >= 0, SIMP_ERR_ARG, "silu: negative size");
  if (n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && y, SIMP_ERR_ARG, "silu: null pointer");
  const int vec = aligned16(x) && aligned16(y) && (!mul || aligned16(mul));
  silu_kernel<<<ew_grid(cdiv(n, 4)), 256, 0, ctx().stream>>>(x, mul, y, n, vec);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_gpu_quantize_i8(const float* x, int8_t* y, int64_t n, float scale, int clamp) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(n >= 0, SIMP_ERR_ARG, "quantize_i8: negative size");
  if (n == 0) return SIMP_OK;
  SIMP_REQUIRE(x && y, SIMP_ERR_ARG, "quantize_i8: null pointer");
  const int vec = aligned16(x) && ((reinterpret_cast<uintptr_t>(y) & 3u) == 0);
  quantize_i8_kernel<<<ew_grid(cdiv(n, 4)), 256, 0, ctx().stream>>>(x, y, n, scale, clamp, vec);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_gpu_dequantize_i32(const int32_t* acc, float* y, int64_t n, float divisor) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(n >= 0, SIMP_ERR_ARG, "dequantize_i32: negative size");
  if (n == 0) return SIMP_OK;
  SIMP_REQUIRE(acc && y, SIMP_ERR_ARG, "dequantize_i32: null pointer");
  SIMP_REQUIRE(divisor != 0.0f, SIMP_ERR_ARG, "dequantize_i32: divisor is zero");
  const int vec = aligned16(acc) && aligned16(y);
  dequantize_i32_kernel<<<ew_grid(cdiv(n, 4)), 256, 0, ctx().stream>>>(acc, y, n, divisor, vec);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

SIMP_API int simp_gpu_dequant_w4(const uint8_t* qw, const float* sc, const float* zr, int64_t first_index,
                                 int64_t count, int64_t gs, float* out) {
  if (int rc = ensure_ready()) return rc;
  SIMP_REQUIRE(count >= 0 && first_index >= 0, SIMP_ERR_ARG, "dequant_w4: negative size");
  SIMP_REQUIRE(gs > 0, SIMP_ERR_ARG, "dequant_w4: group_size must be positive");
  if (count == 0) return SIMP_OK;
  SIMP_REQUIRE(qw && sc && out, SIMP_ERR_ARG, "dequant_w4: null pointer");
  dequant_w4_kernel<<<ew_grid(count), 256, 0, ctx().stream>>>(qw, sc, zr, first_index, count, gs, out);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

// ---- tensor_gather ------------------------------------------------------------------------------
// dst[o, n, :] = src[o, indices[n], :] over rows of `row_bytes` bytes (TensorGatherOpLowering,
// ConvertSimpToMemRef.cpp:2625-2776, with the source viewed as [outer, axis_dim, inner]).  One block per
// (o, n) row, 16-byte pieces when both rows are 16-byte aligned.  An index outside [0, axis_dim) -- undefined in
// the reference -- copies nothing and raises the device status word.
namespace simp {
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t* __restrict__ src, const int64_t* __restrict__ indices,
                                                          uint8_t* __restrict__ dst, int64_t axis_dim, int64_t n_idx,
                                                          int64_t row_bytes, int* status) {
  const int64_t o = blockIdx.y, n = blockIdx.x;
  const int64_t s = indices[n];
  if (s < 0 || s >= axis_dim) {
    if (threadIdx.x == 0 && atomicCAS(status, 0, 2) == 0) status[1] = int(n);
    return;
  }
  const uint8_t* from = src + (o * axis_dim + s) * row_bytes;
  uint8_t* to = dst + (o * n_idx + n) * row_bytes;
  if ((((reinterpret_cast<uintptr_t>(from) | reinterpret_cast<uintptr_t>(to)) | uintptr_t(row_bytes)) & 15u) == 0) {
    for (int64_t i = threadIdx.x; i < (row_bytes >> 4); i += blockDim.x)
      reinterpret_cast<uint4*>(to)[i] = reinterpret_cast<const uint4*>(from)[i];
  } else {
    for (int64_t i = threadIdx.x; i < row_bytes; i += blockDim.x) to[i] = from[i];
  }
}
}  // namespace simp

SIMP_API int simp_gpu_tensor_gather(const void* src_dev, const int64_t* indices_dev, void* dst_dev, int64_t outer,
                                    int64_t axis_dim, int64_t inner, int64_t n_idx, int64_t elem_size) {
  if (int rc = simp::ensure_ready()) return rc;
  SIMP_REQUIRE(outer >= 0 && axis_dim >= 0 && inner >= 0 && n_idx >= 0 && elem_size > 0, SIMP_ERR_ARG,
               "tensor_gather: negative size");
  if (outer == 0 || n_idx == 0 || inner == 0) return SIMP_OK;
  SIMP_REQUIRE(src_dev && indices_dev && dst_dev, SIMP_ERR_ARG, "tensor_gather: null pointer");
  SIMP_REQUIRE(outer <= 65535 && n_idx <= 0x7fffffff, SIMP_ERR_SHAPE, "tensor_gather: outer extent above 65535");
  simp::gather_rows_kernel<<<dim3(unsigned(n_idx), unsigned(outer)), 256, 0, simp::ctx().stream>>>(
      static_cast<const uint8_t*>(src_dev), indices_dev, static_cast<uint8_t*>(dst_dev), axis_dim, n_idx, inner * elem_size,
      simp::ctx().dev_status);
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}

// ---- conv2d ---------------------------------------------------------------------------------------
// Direct convolution as Conv2DOpLowering writes it (ConvertSimpToMemRef.cpp:1924-2150): NHWC input, weights
// [OC, KH, KW, IC], acc = bias[oc], taps in (kh, kw, ic) order, taps outside the input skipped, multiply and add
// kept separate (__fmul_rn / __fadd_rn, no contraction), so every output equals the CPU loop bit for bit.
// One thread per output element with oc fastest: neighbouring threads read the same input value (broadcast) and,
// through a [KH, KW, IC, OC] copy of the weights made per call, neighbouring weight values (coalesced).
namespace simp {
__global__ void conv2d_weights_to_hwio_kernel(const float* __restrict__ w, float* __restrict__ wt, int64_t oc, int64_t taps) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;   // over [OC, taps]
  if (idx >= oc * taps) return;
  const int64_t o = idx / taps, t = idx - o * taps;
  wt[t * oc + o] = w[idx];
}
__global__ void __launch_bounds__(256) conv2d_f32_kernel(const float* __restrict__ in, const float* __restrict__ wt,
                                                         const float* __restrict__ bias, float* __restrict__ out, int64_t total,
                                                         int in_h, int in_w, int in_c, int out_h, int out_w, int out_c, int kh,
                                                         int kw, int stride_h, int stride_w, int pad_h, int pad_w) {
  const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int oc = int(idx % out_c);
  int64_t r = idx / out_c;
  const int ow = int(r % out_w);
  r /= out_w;
  const int oh = int(r % out_h);
  const int64_t b = r / out_h;
  float acc = bias[oc];
  for (int y = 0; y < kh; ++y) {
    const int ih = oh * stride_h + y - pad_h;
    for (int x = 0; x < kw; ++x) {
      const int iw = ow * stride_w + x - pad_w;
      if (ih < 0 || ih >= in_h || iw < 0 || iw >= in_w) continue;
      const float* ip = in + ((b * in_h + ih) * in_w + iw) * int64_t(in_c);
      const float* wp = wt + (int64_t(y) * kw + x) * in_c * int64_t(out_c) + oc;
      for (int ic = 0; ic < in_c; ++ic) acc = __fadd_rn(acc, __fmul_rn(ip[ic], wp[int64_t(ic) * out_c]));
    }
  }
  out[idx] = acc;
}
}  // namespace simp

SIMP_API int simp_gpu_conv2d_f32(const float* input_dev, const float* weights_dev, const float* bias_dev, float* output_dev,
                                 int64_t batch, int64_t in_h, int64_t in_w, int64_t in_c, int64_t out_c, int64_t kernel_h,
                                 int64_t kernel_w, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w) {
  if (int rc = simp::ensure_ready()) return rc;
  SIMP_REQUIRE(batch >= 0 && in_h > 0 && in_w > 0 && in_c > 0 && out_c > 0 && kernel_h > 0 && kernel_w > 0 && stride_h > 0 &&
                   stride_w > 0 && pad_h >= 0 && pad_w >= 0,
               SIMP_ERR_ARG, "conv2d: non-positive dimension, stride or negative padding");
  SIMP_REQUIRE(in_h + 2 * pad_h >= kernel_h && in_w + 2 * pad_w >= kernel_w, SIMP_ERR_SHAPE, "conv2d: kernel larger than the padded input");
  if (batch == 0) return SIMP_OK;
  SIMP_REQUIRE(input_dev && weights_dev && bias_dev && output_dev, SIMP_ERR_ARG, "conv2d: null pointer");
  const int64_t out_h = (in_h + 2 * pad_h - kernel_h) / stride_h + 1, out_w = (in_w + 2 * pad_w - kernel_w) / stride_w + 1;
  const int64_t taps = kernel_h * kernel_w * in_c, total = batch * out_h * out_w * out_c;
  SIMP_REQUIRE(in_h < (1 << 30) && in_w < (1 << 30) && in_c < (1 << 30) && out_c < (1 << 30) && total / 256 < 0x7fffffff,
               SIMP_ERR_SHAPE, "conv2d: dimension too large");
  float* wt = static_cast<float*>(simp::scratch(size_t(taps) * out_c * 4, 11));
  if (!wt) return simp::scratch_failed("conv2d (weight copy)");
  cudaStream_t st = simp::ctx().stream;
  simp::conv2d_weights_to_hwio_kernel<<<unsigned((taps * out_c + 255) / 256), 256, 0, st>>>(weights_dev, wt, out_c, taps);
  simp::conv2d_f32_kernel<<<unsigned((total + 255) / 256), 256, 0, st>>>(input_dev, wt, bias_dev, output_dev, total, int(in_h),
                                                                         int(in_w), int(in_c), int(out_h), int(out_w), int(out_c),
                                                                         int(kernel_h), int(kernel_w), int(stride_h), int(stride_w),
                                                                         int(pad_h), int(pad_w));
  SIMP_LAUNCH_CHECK();
  return SIMP_OK;
}
