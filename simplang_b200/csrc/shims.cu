// shims.cu -- entry points with the argument expansion MLIR 14's std->LLVM lowering gives memref
// operands, so that a `call @simp_rt_*` emitted by a GPU lowering pattern links against this library
// with no glue code.
//
// A `!simp.array<T>` becomes memref<?xT> (src/mlir/lowering/ConvertSimpToMemRef.cpp:43-46), passed as
// five scalars (allocated pointer, aligned pointer, offset, size, stride); a ranked tensor becomes a
// static rank-2 memref, passed as seven (.., offset, size0, size1, stride0, stride1) -- the same
// expansion the reference hosts spell out by hand in their MEMREF_PARAMS macros
// (examples/llama2/generate_stories110M.cpp:12-22, simptensor/benchmarks/bench_prefill_matmul_runner.cpp:18-23).
// Element data is at aligned + offset.  Scalars are i64 / f32.  Each shim returns an i32 status and
// forwards to the host-pointer entry point of the same op; operands registered with
// simp_gpu_register_host stay resident on the device.
#include "common.cuh"

#define MEMREF1(T, name) T* name##_alloc, T* name, int64_t name##_off, int64_t name##_size, int64_t name##_stride
#define MEMREF2(T, name)                                                                              \
  T* name##_alloc, T* name, int64_t name##_off, int64_t name##_s0, int64_t name##_s1, int64_t name##_st0, \
      int64_t name##_st1

using namespace simp;

static inline int check_contig1(int64_t stride, const char* what) {
  SIMP_REQUIRE(stride == 1, SIMP_ERR_SHAPE, "%s: memref stride %lld (only contiguous arrays are supported)", what,
               (long long)stride);
  return SIMP_OK;
}
static inline int check_contig2(int64_t s1, int64_t st0, int64_t st1, const char* what) {
  SIMP_REQUIRE(st1 == 1 && st0 == s1, SIMP_ERR_SHAPE, "%s: tensor memref is not contiguous row-major", what);
  return SIMP_OK;
}

// simp.matmul(lhs, rhs, out, m, k, n, lhs_off, rhs_off, out_off): out += lhs . rhs
// (MatMulOpLowering, ConvertSimpToMemRef.cpp:1794-1920; call sites stories110M.sl:77-83)
SIMP_API int32_t simp_rt_matmul_f32(MEMREF1(float, lhs), MEMREF1(float, rhs), MEMREF1(float, out), int64_t m,
                                    int64_t k, int64_t n, int64_t lhs_offset, int64_t rhs_offset, int64_t out_offset) {
  (void)lhs_alloc; (void)rhs_alloc; (void)out_alloc; (void)lhs_size; (void)rhs_size; (void)out_size;
  if (int rc = check_contig1(lhs_stride, "matmul lhs")) return rc;
  if (int rc = check_contig1(rhs_stride, "matmul rhs")) return rc;
  if (int rc = check_contig1(out_stride, "matmul out")) return rc;
  return simp_host_matmul_f32(lhs + lhs_off, lhs_offset, rhs + rhs_off, rhs_offset, out + out_off, out_offset, m, k, n,
                              /*accumulate=*/1, /*b_transposed=*/0);
}

// simp.rmsnorm(x, w, y, n, eps, weight_offset)  (RMSNormOpLowering, ConvertSimpToMemRef.cpp:2157-2236)
SIMP_API int32_t simp_rt_rmsnorm_f32(MEMREF1(float, x), MEMREF1(float, w), MEMREF1(float, y), int64_t n, float eps,
                                     int64_t weight_offset) {
  (void)x_alloc; (void)w_alloc; (void)y_alloc; (void)x_size; (void)w_size; (void)y_size;
  if (int rc = check_contig1(x_stride, "rmsnorm x")) return rc;
  if (int rc = check_contig1(w_stride, "rmsnorm w")) return rc;
  if (int rc = check_contig1(y_stride, "rmsnorm y")) return rc;
  return simp_host_rmsnorm_f32(x + x_off, w + w_off, y + y_off, 1, n, eps, weight_offset);
}

// simp.softmax(x, y, n, x_offset, y_offset)  (SoftmaxOpLowering, ConvertSimpToMemRef.cpp:2239-2322)
SIMP_API int32_t simp_rt_softmax_f32(MEMREF1(float, x), MEMREF1(float, y), int64_t n, int64_t x_offset,
                                     int64_t y_offset) {
  (void)x_alloc; (void)y_alloc; (void)x_size; (void)y_size;
  if (int rc = check_contig1(x_stride, "softmax x")) return rc;
  if (int rc = check_contig1(y_stride, "softmax y")) return rc;
  return simp_host_softmax_f32(x + x_off, y + y_off, 1, n, x_offset, y_offset, n);
}

// simp.silu(x, y, n)  (SiLUOpLowering, ConvertSimpToMemRef.cpp:2325-2360)
SIMP_API int32_t simp_rt_silu_f32(MEMREF1(float, x), MEMREF1(float, y), int64_t n) {
  (void)x_alloc; (void)y_alloc; (void)x_size; (void)y_size;
  if (int rc = check_contig1(x_stride, "silu x")) return rc;
  if (int rc = check_contig1(y_stride, "silu y")) return rc;
  return simp_host_silu_f32(x + x_off, nullptr, y + y_off, n);
}

// simp.matmul_quant(qweights, scales, zeros, x, out, rows, cols, group_size, offset)
// (MatMulQuantOpLowering, ConvertSimpToMemRef.cpp:3853-4013): the op as written, i.e. scale_mode 0.
SIMP_API int32_t simp_rt_matmul_quant(MEMREF1(int8_t, qw), MEMREF1(float, sc), MEMREF1(float, zr), MEMREF1(float, x),
                                      MEMREF1(float, out), int64_t rows, int64_t cols, int64_t group_size,
                                      int64_t offset) {
  (void)qw_alloc; (void)sc_alloc; (void)zr_alloc; (void)x_alloc; (void)out_alloc;
  SIMP_REQUIRE(rows >= 0 && cols >= 0 && cols <= x_size && rows <= out_size, SIMP_ERR_SHAPE,
               "matmul_quant: rows %lld / cols %lld exceed the out (%lld) / x (%lld) arrays", (long long)rows,
               (long long)cols, (long long)out_size, (long long)x_size);
  if (int rc = check_contig1(qw_stride, "matmul_quant qweights")) return rc;
  if (int rc = check_contig1(sc_stride, "matmul_quant scales")) return rc;
  if (int rc = check_contig1(zr_stride, "matmul_quant zeros")) return rc;
  if (int rc = check_contig1(x_stride, "matmul_quant x")) return rc;
  if (int rc = check_contig1(out_stride, "matmul_quant out")) return rc;
  SIMP_REQUIRE(sc_size == zr_size, SIMP_ERR_SHAPE, "matmul_quant: scales and zeros differ in length");
  return simp_host_matmul_quant(reinterpret_cast<const uint8_t*>(qw + qw_off), size_t(qw_size), sc + sc_off,
                                zr + zr_off, size_t(sc_size), x + x_off, out + out_off, rows, cols, group_size, offset,
                                /*scale_mode=*/0);
}

// tensor_matmul / tensor_matmul_into on i8<M,K>, i8<K,N> -> i32<M,N>  (ConvertSimpToMemRef.cpp:3136-3279, 3490-3627)
SIMP_API int32_t simp_rt_tensor_matmul_i8(MEMREF2(int8_t, a), MEMREF2(int8_t, b), MEMREF2(int32_t, c)) {
  (void)a_alloc; (void)b_alloc; (void)c_alloc;
  if (int rc = check_contig2(a_s1, a_st0, a_st1, "tensor_matmul A")) return rc;
  if (int rc = check_contig2(b_s1, b_st0, b_st1, "tensor_matmul B")) return rc;
  if (int rc = check_contig2(c_s1, c_st0, c_st1, "tensor_matmul C")) return rc;
  SIMP_REQUIRE(a_s1 == b_s0 && c_s0 == a_s0 && c_s1 == b_s1, SIMP_ERR_SHAPE, "tensor_matmul: shapes do not agree");
  return simp_host_tensor_matmul_i8(a + a_off, b + b_off, c + c_off, a_s0, a_s1, b_s1, /*a_unsigned=*/0,
                                    /*b_transposed=*/0);
}

// tensor_matmul_nt on i8<M,K>, i8<N,K> -> i32<M,N>  (TensorMatMulNTOpLowering, ConvertSimpToMemRef.cpp:3373-3486)
SIMP_API int32_t simp_rt_tensor_matmul_nt_i8(MEMREF2(int8_t, a), MEMREF2(int8_t, bt), MEMREF2(int32_t, c)) {
  (void)a_alloc; (void)bt_alloc; (void)c_alloc;
  if (int rc = check_contig2(a_s1, a_st0, a_st1, "tensor_matmul_nt A")) return rc;
  if (int rc = check_contig2(bt_s1, bt_st0, bt_st1, "tensor_matmul_nt B")) return rc;
  if (int rc = check_contig2(c_s1, c_st0, c_st1, "tensor_matmul_nt C")) return rc;
  SIMP_REQUIRE(a_s1 == bt_s1 && c_s0 == a_s0 && c_s1 == bt_s0, SIMP_ERR_SHAPE, "tensor_matmul_nt: shapes do not agree");
  return simp_host_tensor_matmul_i8(a + a_off, bt + bt_off, c + c_off, a_s0, a_s1, bt_s0, /*a_unsigned=*/0,
                                    /*b_transposed=*/1);
}

// tensor_matmul on f32<M,K>, f32<K,N> -> f32<M,N>, fresh result  (ConvertSimpToMemRef.cpp:2884-2950, 3280-3291)
SIMP_API int32_t simp_rt_tensor_matmul_f32(MEMREF2(float, a), MEMREF2(float, b), MEMREF2(float, c)) {
  (void)a_alloc; (void)b_alloc; (void)c_alloc;
  if (int rc = check_contig2(a_s1, a_st0, a_st1, "tensor_matmul A")) return rc;
  if (int rc = check_contig2(b_s1, b_st0, b_st1, "tensor_matmul B")) return rc;
  if (int rc = check_contig2(c_s1, c_st0, c_st1, "tensor_matmul C")) return rc;
  SIMP_REQUIRE(a_s1 == b_s0 && c_s0 == a_s0 && c_s1 == b_s1, SIMP_ERR_SHAPE, "tensor_matmul: shapes do not agree");
  return simp_host_matmul_f32(a + a_off, 0, b + b_off, 0, c + c_off, 0, a_s0, a_s1, b_s1, /*accumulate=*/0,
                              /*b_transposed=*/0);
}
