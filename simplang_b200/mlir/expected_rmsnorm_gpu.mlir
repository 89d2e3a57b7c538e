// What `simplang kernels/test_rmsnorm.sl --emit-mlir --target gpu` is expected to contain after
// ConvertSimpToMemRef with the GPU patterns (hand-written expectation in the style of
// tests/mlir/integration/*.mlir of the reference; it cannot be produced here, the image has no MLIR 14).
//
// Before (simp dialect):
//   %y = simp.rmsnorm %x, %w, %out, %n, %eps, %woff
//          : (!simp.array<f32>, !simp.array<f32>, !simp.array<f32>, i64, f32, i64) -> !simp.array<f32>
// After:
module {
  func private @simp_rt_rmsnorm_f32(memref<?xf32>, memref<?xf32>, memref<?xf32>, i64, f32, i64) -> i32
  func @kernel_main(%x: memref<?xf32>, %w: memref<?xf32>, %out: memref<?xf32>) -> f32 {
    %n = arith.constant 4 : i64
    %woff = arith.constant 0 : i64
    %eps = arith.constant 1.000000e-05 : f32
    %st = call @simp_rt_rmsnorm_f32(%x, %w, %out, %n, %eps, %woff)
            : (memref<?xf32>, memref<?xf32>, memref<?xf32>, i64, f32, i64) -> i32
    %c0 = arith.constant 0 : index
    %r = memref.load %out[%c0] : memref<?xf32>
    return %r : f32
  }
}
// After std->LLVM each memref<?xf32> operand becomes (ptr, ptr, i64, i64, i64): the 5-scalar groups of
// SIMP_MEMREF1 in include/simp_gpu.h.
