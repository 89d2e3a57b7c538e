//===- ConvertSimpToGpuRuntime.cpp - simp hot-path ops -> libsimp_gpu calls ----------------===//
//
// Source for the SimpLang compiler tree (MLIR/LLVM 14), to live beside
// src/mlir/lowering/ConvertSimpToMemRef.cpp.  It is NOT built in this repository: the build image
// has no LLVM/MLIR 14.  tests/ and bench.py exercise the library these calls bind to.
//
// With `--target gpu` (a new flag of src/main.cpp beside --emit-mlir) these patterns are added to the pattern set of
// ConvertSimpToMemRefPass (ConvertSimpToMemRef.cpp:4078-4129) with a higher benefit than the loop
// expansions they replace.  Each one rewrites a `simp` op whose operands have already been converted
// to memrefs by the pass's type converter (ConvertSimpToMemRef.cpp:36-96) into
//
//     %st = call @simp_rt_<op>(memref operands..., scalar operands...) : (...) -> i32
//
// MLIR's std->LLVM lowering then expands every memref operand into (allocated, aligned, offset,
// sizes..., strides...), which is exactly the parameter list of the simp_rt_* shims in
// include/simp_gpu.h.  The status is ignored in generated code (the reference ops cannot fail either,
// include/mlir/Dialects/Simp/SimpOps.td:712); a host can read simp_gpu_last_error().
//
//===----------------------------------------------------------------------------------------===//

#include "mlir/Dialects/Simp/SimpDialect.h"
#include "mlir/Dialects/Simp/SimpOps.h"

#include "mlir/Dialect/Arithmetic/IR/Arithmetic.h"
#include "mlir/Dialect/MemRef/IR/MemRef.h"
#include "mlir/Dialect/StandardOps/IR/Ops.h"
#include "mlir/IR/BuiltinOps.h"
#include "mlir/Transforms/DialectConversion.h"

using namespace mlir;

namespace {

/// Declares `func private @name(argTypes...) -> i32` at module scope once and returns its symbol.
static FlatSymbolRefAttr getOrInsertRuntimeFn(ConversionPatternRewriter &rewriter, Operation *anchor,
                                              StringRef name, TypeRange argTypes) {
  auto module = anchor->getParentOfType<ModuleOp>();
  auto *ctx = module.getContext();
  if (!module.lookupSymbol<FuncOp>(name)) {
    OpBuilder::InsertionGuard guard(rewriter);
    rewriter.setInsertionPointToStart(module.getBody());
    auto fnType = FunctionType::get(ctx, argTypes, {IntegerType::get(ctx, 32)});
    auto fn = rewriter.create<FuncOp>(module.getLoc(), name, fnType);
    fn.setPrivate();
  }
  return SymbolRefAttr::get(ctx, name);
}

/// Emits the call and returns the op (result #0 is the i32 status).
static CallOp emitRuntimeCall(ConversionPatternRewriter &rewriter, Operation *op, StringRef name,
                              ValueRange args) {
  SmallVector<Type, 12> argTypes;
  for (Value v : args) argTypes.push_back(v.getType());
  auto callee = getOrInsertRuntimeFn(rewriter, op, name, argTypes);
  return rewriter.create<CallOp>(op->getLoc(), callee, TypeRange{rewriter.getI32Type()}, args);
}

static Value castToF32(ConversionPatternRewriter &rewriter, Location loc, Value v) {
  auto f32 = rewriter.getF32Type();
  if (v.getType() == f32) return v;
  if (v.getType().cast<FloatType>().getWidth() > 32) return rewriter.create<arith::TruncFOp>(loc, f32, v);
  return rewriter.create<arith::ExtFOp>(loc, f32, v);
}

static bool isF32MemRef(Value v) {
  auto t = v.getType().dyn_cast<MemRefType>();
  return t && t.getElementType().isF32();
}

// simp.rmsnorm(input, weight, output, size, epsilon, weight_offset)   [CPU form: :2157-2236]
struct RMSNormToGpu : public OpConversionPattern<simp::RMSNormOp> {
  using OpConversionPattern::OpConversionPattern;
  LogicalResult matchAndRewrite(simp::RMSNormOp op, OpAdaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    if (!isF32MemRef(adaptor.input())) return failure();  // f64 stays on the CPU expansion
    Value eps = castToF32(rewriter, op.getLoc(), adaptor.epsilon());
    emitRuntimeCall(rewriter, op, "simp_rt_rmsnorm_f32",
                    {adaptor.input(), adaptor.weight(), adaptor.output(), adaptor.size(), eps,
                     adaptor.weight_offset()});
    rewriter.replaceOp(op, adaptor.output());
    return success();
  }
};

// simp.softmax(input, output, size, input_offset, output_offset)     [CPU form: :2239-2322]
struct SoftmaxToGpu : public OpConversionPattern<simp::SoftmaxOp> {
  using OpConversionPattern::OpConversionPattern;
  LogicalResult matchAndRewrite(simp::SoftmaxOp op, OpAdaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    if (!isF32MemRef(adaptor.input())) return failure();
    emitRuntimeCall(rewriter, op, "simp_rt_softmax_f32",
                    {adaptor.input(), adaptor.output(), adaptor.size(), adaptor.input_offset(),
                     adaptor.output_offset()});
    rewriter.replaceOp(op, adaptor.output());
    return success();
  }
};

// simp.silu(input, output, size)                                      [CPU form: :2325-2360]
struct SiLUToGpu : public OpConversionPattern<simp::SiLUOp> {
  using OpConversionPattern::OpConversionPattern;
  LogicalResult matchAndRewrite(simp::SiLUOp op, OpAdaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    if (!isF32MemRef(adaptor.input())) return failure();
    emitRuntimeCall(rewriter, op, "simp_rt_silu_f32", {adaptor.input(), adaptor.output(), adaptor.size()});
    rewriter.replaceOp(op, adaptor.output());
    return success();
  }
};

// simp.matmul(lhs, rhs, output, m, k, n, lhs_offset, rhs_offset, output_offset)   [CPU form: :1794-1920]
// Operand order as in MatMulOpLowering: getOperands()[0..8].
struct MatMulToGpu : public OpConversionPattern<simp::MatMulOp> {
  using OpConversionPattern::OpConversionPattern;
  LogicalResult matchAndRewrite(simp::MatMulOp op, OpAdaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    auto operands = adaptor.getOperands();
    if (operands.size() != 9 || !isF32MemRef(operands[0])) return failure();
    emitRuntimeCall(rewriter, op, "simp_rt_matmul_f32", operands);
    rewriter.replaceOp(op, operands[2]);
    return success();
  }
};

// simp.matmul_quant(qweights, scales, zeros, input, output, rows, cols, group_size, offset)   [:3853-4013]
struct MatMulQuantToGpu : public OpConversionPattern<simp::MatMulQuantOp> {
  using OpConversionPattern::OpConversionPattern;
  LogicalResult matchAndRewrite(simp::MatMulQuantOp op, OpAdaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    emitRuntimeCall(rewriter, op, "simp_rt_matmul_quant",
                    {adaptor.qweights(), adaptor.scales(), adaptor.zeros(), adaptor.input(), adaptor.output(),
                     adaptor.rows(), adaptor.cols(), adaptor.group_size(), adaptor.offset()});
    rewriter.replaceOp(op, adaptor.output());
    return success();
  }
};

/// Shared by tensor_matmul / tensor_matmul_nt on static rank-2 i8 or f32 tensors: allocates the result
/// memref exactly as the CPU lowering does (:2926-2933) and calls the runtime into it.
template <typename OpT>
struct TensorMatMulToGpu : public OpConversionPattern<OpT> {
  TensorMatMulToGpu(TypeConverter &tc, MLIRContext *ctx, bool nt)
      : OpConversionPattern<OpT>(tc, ctx, /*benefit=*/2), nt(nt) {}
  LogicalResult matchAndRewrite(OpT op, typename OpT::Adaptor adaptor,
                                ConversionPatternRewriter &rewriter) const override {
    auto lhsT = adaptor.lhs().getType().template dyn_cast<MemRefType>();
    auto rhsT = adaptor.rhs().getType().template dyn_cast<MemRefType>();
    auto resT = this->getTypeConverter()->convertType(op.getResult().getType()).template dyn_cast<MemRefType>();
    if (!lhsT || !rhsT || !resT || lhsT.getRank() != 2 || rhsT.getRank() != 2 || !lhsT.hasStaticShape() ||
        !rhsT.hasStaticShape())
      return failure();  // batched / dynamic shapes keep the CPU expansion
    StringRef callee;
    if (lhsT.getElementType().isInteger(8) && resT.getElementType().isInteger(32))
      callee = nt ? "simp_rt_tensor_matmul_nt_i8" : "simp_rt_tensor_matmul_i8";
    else if (lhsT.getElementType().isF32() && !nt)
      callee = "simp_rt_tensor_matmul_f32";
    else
      return failure();
    Value result = rewriter.create<memref::AllocOp>(op.getLoc(), resT);
    emitRuntimeCall(rewriter, op, callee, {adaptor.lhs(), adaptor.rhs(), result});
    rewriter.replaceOp(op, result);
    return success();
  }
  bool nt;
};

}  // namespace

namespace mlir {
namespace simp {

/// Called from ConvertSimpToMemRefPass::runOnOperation() right after its own patterns.add<...>() when the
/// compiler runs with --target gpu.  Benefit 2 makes these win over the loop expansions (benefit 1);
/// a pattern that returns failure() (f64, dynamic shapes) falls back to the CPU expansion.
void populateSimpToGpuRuntimePatterns(TypeConverter &typeConverter, RewritePatternSet &patterns) {
  MLIRContext *ctx = patterns.getContext();
  patterns.add<RMSNormToGpu, SoftmaxToGpu, SiLUToGpu, MatMulToGpu, MatMulQuantToGpu>(typeConverter, ctx,
                                                                                    /*benefit=*/2);
  patterns.add<TensorMatMulToGpu<simp::TensorMatMulOp>>(typeConverter, ctx, /*nt=*/false);
  patterns.add<TensorMatMulToGpu<simp::TensorMatMulNTOp>>(typeConverter, ctx, /*nt=*/true);
}

}  // namespace simp
}  // namespace mlir
