//===- TensorAlgebraToB200.cpp - ta.mul / ta.elews_mul -> libcomet_b200 ------------------===//
//
// NOT COMPILED IN THIS REPOSITORY.  This file belongs in a COMET checkout at
// lib/Conversion/TensorAlgebraToB200/ and is written against the APIs that tree uses elsewhere; it
// needs COMET's headers and the LLVM/MLIR COMET is built with, neither of which exists here.
//
// What it does.  COMET lowers ta.mul / ta.elews_mul to the index-tree dialect and from there to
// SCF loops.  For a sparse transpose it does something else: it emits a call into its runtime
// library (lib/Conversion/TensorAlgebraToSCF/TensorAlgebraToSCF.cpp:253-404 ->
// transpose_2D_f64_i64).  The two passes below do the same for the multiplications that
// libcomet_b200 implements on the GPU, so that `comet-opt --convert-ta-to-b200 ...` produces a
// program whose hot loops are calls into that library while every other op keeps its lowering.
//
// Two stages are needed because of where the information lives in COMET's pipeline
// (frontends/comet_dsl/comet.cpp):
//   * ta.mul only exists BEFORE createLowerTensorAlgebraToIndexTreePass (:447) -- after it the op is
//     an index tree;
//   * the arrays of a sparse tensor only exist AFTER the tensor-declaration lowering passes
//     (:483-488), which run later and which classify a declaration as input or output by looking
//     at its users (lib/Dialect/TensorAlgebra/Transforms/TensorDeclLowering.cpp:720-823).
// Stage 1 (ConvertTensorAlgebraToB200) therefore replaces a matched ta.mul (+ its ta.set_op) by a
// func.call to a private function @b200.<op> that still takes and returns TENSORS.  The declaration
// lowering treats a func.call user as a plain read (TensorDeclLowering.cpp:785-788), so sparse
// inputs are read from file as always.  Stage 2 (FinalizeB200Calls) runs where the sparse
// transpose is lowered today, finds the @b200.* calls, takes the operands apart with
// ta.SpTensorGetDimPos/Crd/..., bufferization.to_memref and memref.cast exactly as the transpose
// lowering does, declares the runtime function once (hasFuncDeclaration) and emits the call.
//
// Operand order of every emitted call is the one include/comet_b200.h declares
// (COMET_B200_SPARSE2D): per sparse operand 4 format constants, then per dimension pos, crd,
// tile_pos, tile_crd, then vals, then the dims memref -- the order transpose_2D_f64_i64 receives
// (lib/ExecutionEngine/TransposeUtils.cpp:1439-1451).  Dense operands are one unranked memref.
// Scalars trail.  Symbol suffix _f64_i64 / _f64_i32 follows the tensor type's index width like
// read_input_2D_f64_i64 / _i32 (TensorDeclLowering.cpp:1038).
//
//===----------------------------------------------------------------------===//

#include "comet/Conversion/TensorAlgebraToB200/TensorAlgebraToB200.h"
#include "comet/Dialect/TensorAlgebra/IR/TADialect.h"
#include "comet/Dialect/Utils/Utils.h"

#include "mlir/Dialect/Arith/IR/Arith.h"
#include "mlir/Dialect/Bufferization/IR/Bufferization.h"
#include "mlir/Dialect/Func/IR/FuncOps.h"
#include "mlir/Dialect/MemRef/IR/MemRef.h"
#include "mlir/Dialect/Tensor/IR/Tensor.h"
#include "mlir/IR/AffineMap.h"
#include "mlir/IR/BuiltinTypes.h"
#include "mlir/IR/PatternMatch.h"
#include "mlir/Pass/Pass.h"
#include "llvm/ADT/SmallVector.h"
#include "llvm/ADT/StringSwitch.h"

#include <string>
#include <vector>

using namespace mlir;
using namespace mlir::arith;
using namespace mlir::bufferization;
using namespace mlir::tensorAlgebra;

namespace mlir
{
  namespace comet
  {
#define GEN_PASS_DEF_CONVERTTENSORALGEBRATOB200
#define GEN_PASS_DEF_FINALIZEB200CALLS
#include "comet/Conversion/Passes.h.inc"
  }
}

namespace
{
  //===--------------------------------------------------------------------===//
  // Shared vocabulary of the two stages
  //===--------------------------------------------------------------------===//

  /// Names of the tensor-level callees stage 1 emits and stage 2 consumes.
  constexpr llvm::StringLiteral kSpmv("b200.spmv");                 // (A sparse, x, y)          -> y'
  constexpr llvm::StringLiteral kSpmm("b200.spmm");                 // (A sparse, B, C)          -> C'
  constexpr llvm::StringLiteral kDenseSparse("b200.dense_sparse");  // (A dense, B sparse, C)    -> C'
  constexpr llvm::StringLiteral kSpgemm("b200.spgemm");             // (A, B [, M]) all CSR      -> C sparse
  constexpr llvm::StringLiteral kElewsSD("b200.elews_sparse_dense");// (A sparse, B dense)       -> C sparse (A's pattern)
  constexpr llvm::StringLiteral kElewsSS("b200.elews_sparse_sparse");// (A, B) CSR               -> C sparse
  constexpr llvm::StringLiteral kSddmm("b200.sddmm");               // (S sparse, X, D)          -> O sparse (S's pattern)
  constexpr llvm::StringLiteral kMaskedCount("b200.masked_count");  // (A, B, M) CSR             -> f64

  /// Attributes carried by the tensor-level call.
  constexpr llvm::StringLiteral kSemiringAttr("b200.semiring");     // i32: COMET_B200_PLUS_TIMES ...
  constexpr llvm::StringLiteral kAccumulateAttr("b200.accumulate"); // i32: 0 = output was just filled with 0.0
  constexpr llvm::StringLiteral kMaskedAttr("b200.masked");         // unit: a push mask is the last operand

  /// Semiring codes of include/comet_b200.h; -1 = not handled by the library.
  int semiringCode(llvm::StringRef s)
  {
    return llvm::StringSwitch<int>(s)
        .Case("plusxy_times", 0)
        .Case("plusxy_pairxy", 1)
        .Case("plusxy_first", 2)
        .Case("plusxy_second", 3)
        .Case("minxy_plusxy", 4)
        .Case("minxy_first", 5)
        .Case("minxy_second", 6)
        .Case("any_pairxy", 7)
        .Default(-1);
  }

  enum class Fmt { Dense, CSR, DCSR, COO, Other };

  /// Storage format of a rank-2 tensor value, from its type (CSR = [D, CU], DCSR = [CU, CU],
  /// COO = [CN, S]; lib/Dialect/Utils/Utils.cpp:997-1010).
  Fmt formatOf(Value v)
  {
    Type t = v.getType();
    if (isa<TensorType>(t))
      return Fmt::Dense;
    auto sp = dyn_cast<SparseTensorType>(t);
    if (!sp || sp.getRank() != 2)
      return Fmt::Other;
    std::string f(getTensorFormatString(t));
    if (f == "CSR")
      return Fmt::CSR;
    if (f == "DCSR")
      return Fmt::DCSR;
    if (f == "COO")
      return Fmt::COO;
    return Fmt::Other;
  }

  bool isSparse2D(Fmt f) { return f == Fmt::CSR || f == Fmt::DCSR || f == Fmt::COO; }

  int64_t rankOf(Value v)
  {
    if (auto t = dyn_cast<TensorType>(v.getType()))
      return t.getRank();
    if (auto s = dyn_cast<SparseTensorType>(v.getType()))
      return s.getRank();
    return -1;
  }

  bool isF64(Value v)
  {
    if (auto t = dyn_cast<TensorType>(v.getType()))
      return t.getElementType().isF64();
    if (auto s = dyn_cast<SparseTensorType>(v.getType()))
      return s.getElementType().isF64();
    return false;
  }

  /// The three indexing maps of ta.mul as lists of dimension positions: rhs1, rhs2, lhs.
  bool mapsAre(ArrayAttr maps, ArrayRef<ArrayRef<unsigned>> want)
  {
    if (maps.size() != want.size())
      return false;
    for (unsigned i = 0; i < want.size(); i++)
    {
      AffineMap m = cast<AffineMapAttr>(maps[i]).getValue();
      if (m.getNumResults() != want[i].size())
        return false;
      for (unsigned j = 0; j < want[i].size(); j++)
      {
        auto d = dyn_cast<AffineDimExpr>(m.getResult(j));
        if (!d || d.getPosition() != want[i][j])
          return false;
      }
    }
    return true;
  }

  /// The ta.set_op that stores `produced` (ta.mul results are always stored through one,
  /// frontends/comet_dsl/mlir/MLIRGen.cpp) and the tensor it stores into.
  TensorSetOp storeOf(Value produced, Value &dest)
  {
    for (Operation *u : produced.getUsers())
      if (auto set = dyn_cast<TensorSetOp>(u))
        if (set->getOperand(0) == produced)
        {
          dest = set->getOperand(1);
          return set;
        }
    return nullptr;
  }

  /// 0 when `dest` (a dense tensor declaration) is filled with the constant 0.0 and nothing else
  /// writes it before `before`; 1 otherwise.  COMET's loops read-modify-write the output
  /// (lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:1266-1278), so 1 is always correct and 0 only
  /// saves the upload of the old contents.
  int accumulateFlag(Value dest, Operation *before)
  {
    TensorFillOp fill;
    for (Operation *u : dest.getUsers())
    {
      if (u == before || !u->isBeforeInBlock(before))
        continue;
      if (auto f = dyn_cast<TensorFillOp>(u))
      {
        if (fill)
          return 1;
        fill = f;
        continue;
      }
      if (isa<PrintOp, TensorDimOp>(u))
        continue;
      return 1; // some other op touched it first
    }
    if (!fill)
      return 1;
    if (auto v = dyn_cast<FloatAttr>(fill.getValue()))
      return v.getValueAsDouble() == 0.0 ? 0 : 1;
    return 1;
  }

  func::FuncOp declare(ModuleOp module, Location loc, StringRef name, FunctionType type)
  {
    if (auto f = module.lookupSymbol<func::FuncOp>(name))
      return f;
    auto f = func::FuncOp::create(loc, name, type, ArrayRef<NamedAttribute>{});
    f.setPrivate();
    module.push_back(f);
    return f;
  }

  /// Replaces every use of `dest` that comes after `after` in its block by `value`: the effect
  /// ta.set_op has when it is lowered (ConvertSetOp, TensorAlgebraToSCF.cpp:613-630).
  void forwardStore(PatternRewriter &rewriter, Value dest, Value value, Operation *after)
  {
    rewriter.replaceUsesWithIf(dest, value, [&](OpOperand &use) {
      Operation *anc = after->getBlock()->findAncestorOpInBlock(*use.getOwner());
      return anc && after->isBeforeInBlock(anc);
    });
  }

  //===--------------------------------------------------------------------===//
  // Stage 1: ta.mul / ta.elews_mul / ta.reduce  ->  func.call @b200.<op> on tensors
  //===--------------------------------------------------------------------===//

  /// Emits `%r = func.call @name(operands) {attrs} : (...) -> resultType` and the declaration.
  Value emitTensorCall(PatternRewriter &rewriter, Operation *at, StringRef name, ValueRange operands,
                       Type resultType, ArrayRef<NamedAttribute> attrs)
  {
    auto module = at->getParentOfType<ModuleOp>();
    // one declaration per distinct signature: the name carries the operand formats
    std::string sym(name);
    for (Value v : operands)
    {
      sym += ".";
      sym += isa<TensorType>(v.getType()) ? ("d" + std::to_string(rankOf(v))) : std::string(getTensorFormatString(v.getType()));
    }
    SmallVector<Type> in(operands.getTypes());
    declare(module, at->getLoc(), sym, FunctionType::get(at->getContext(), in, {resultType}));
    auto call = rewriter.create<func::CallOp>(at->getLoc(), sym, TypeRange{resultType}, operands);
    for (auto a : attrs)
      call->setAttr(a.getName(), a.getValue());
    return call.getResult(0);
  }

  struct MulToB200 : public OpRewritePattern<TensorMultOp>
  {
    using OpRewritePattern<TensorMultOp>::OpRewritePattern;

    LogicalResult matchAndRewrite(TensorMultOp op, PatternRewriter &rewriter) const final
    {
      Value a = op.getRhs1(), b = op.getRhs2();
      if (!isF64(a) || !isF64(b))
        return failure(); // f32 symbols exist in the library; the pattern is kept to the tested type
      const int sr = semiringCode(op.getSemiring());
      if (sr < 0)
        return failure();
      Value dest;
      TensorSetOp set = storeOf(op.getResult(), dest);
      if (!set)
        return failure();
      const Fmt fa = formatOf(a), fb = formatOf(b), fc = formatOf(dest);
      ArrayAttr maps = op.getIndexingMaps();
      const bool masked = op.getMask() != nullptr;
      if (masked && (!op.getMaskType() || *op.getMaskType() != "push"))
        return failure(); // pull / auto masks stay on the index-tree path

      auto i32 = [&](int v) { return rewriter.getI32IntegerAttr(v); };
      rewriter.setInsertionPoint(set);
      Value result;

      // ---- sparse x dense vector / matrix -> dense (SpMV, SpMM) --------------------------------
      if (isSparse2D(fa) && fb == Fmt::Dense && fc == Fmt::Dense && !masked && sr <= 1)
      {
        const bool vec = rankOf(b) == 1 && mapsAre(maps, {{0, 1}, {1}, {0}});
        const bool mat = rankOf(b) == 2 && mapsAre(maps, {{0, 1}, {1, 2}, {0, 2}});
        if (!vec && !mat)
          return failure();
        result = emitTensorCall(rewriter, set, vec ? kSpmv : kSpmm, {a, b, dest}, dest.getType(),
                                {rewriter.getNamedAttr(kSemiringAttr, i32(sr)),
                                 rewriter.getNamedAttr(kAccumulateAttr, i32(accumulateFlag(dest, set)))});
      }
      // ---- dense vector / matrix x sparse -> dense ----------------------------------------------
      else if (fa == Fmt::Dense && isSparse2D(fb) && fc == Fmt::Dense && !masked && sr <= 1)
      {
        const bool vec = rankOf(a) == 1 && mapsAre(maps, {{0}, {0, 1}, {1}});
        const bool mat = rankOf(a) == 2 && mapsAre(maps, {{0, 1}, {1, 2}, {0, 2}});
        if (!vec && !mat)
          return failure();
        result = emitTensorCall(rewriter, set, kDenseSparse, {a, b, dest}, dest.getType(),
                                {rewriter.getNamedAttr(kSemiringAttr, i32(sr)),
                                 rewriter.getNamedAttr(kAccumulateAttr, i32(accumulateFlag(dest, set)))});
      }
      // ---- CSR x CSR -> CSR, optional push mask (Gustavson SpGEMM) -------------------------------
      else if (fa == Fmt::CSR && fb == Fmt::CSR && fc == Fmt::CSR && mapsAre(maps, {{0, 1}, {1, 2}, {0, 2}}))
      {
        if (masked && formatOf(op.getMask()) != Fmt::CSR)
          return failure();
        SmallVector<Value> operands{a, b};
        SmallVector<NamedAttribute> attrs{rewriter.getNamedAttr(kSemiringAttr, i32(sr))};
        if (masked)
        {
          operands.push_back(op.getMask());
          attrs.push_back(rewriter.getNamedAttr(kMaskedAttr, rewriter.getUnitAttr()));
        }
        result = emitTensorCall(rewriter, set, kSpgemm, operands, dest.getType(), attrs);
        // The output declaration has no other role than naming the result: once nothing refers to
        // it any more the declaration lowering never sees it (it would otherwise take it for an input).
      }
      else
        return failure();

      forwardStore(rewriter, dest, result, set);
      rewriter.eraseOp(set);
      rewriter.eraseOp(op);
      if (dest.use_empty() && isa<SparseTensorType>(dest.getType()))
        if (Operation *decl = dest.getDefiningOp())
          rewriter.eraseOp(decl);
      return success();
    }
  };

  struct ElewsToB200 : public OpRewritePattern<TensorElewsMultOp>
  {
    using OpRewritePattern<TensorElewsMultOp>::OpRewritePattern;

    LogicalResult matchAndRewrite(TensorElewsMultOp op, PatternRewriter &rewriter) const final
    {
      Value a = op.getRhs1(), b = op.getRhs2();
      if (!isF64(a) || !isF64(b) || op.getSemiring() != "noop_times")
        return failure();
      Value dest;
      TensorSetOp set = storeOf(op.getResult(), dest);
      if (!set)
        return failure();
      if (!mapsAre(op.getIndexingMaps(), {{0, 1}, {0, 1}, {0, 1}}))
        return failure();
      Fmt fa = formatOf(a), fb = formatOf(b);
      const Fmt fc = formatOf(dest);
      rewriter.setInsertionPoint(set);
      Value result;

      // ---- SDDMM: S .* (X * D), the pair --opt-fusion fuses (test/integration/kernels/sddmm.ta) ----
      auto denseProduct = [&](Value v) -> TensorMultOp {
        // v is the tensor a dense x dense ta.mul was stored into, and that ta.mul has no other reader
        for (Operation *u : v.getUsers())
          if (auto s = dyn_cast<TensorSetOp>(u))
            if (s->getOperand(1) == v)
              if (auto m = s->getOperand(0).getDefiningOp<TensorMultOp>())
                if (formatOf(m.getRhs1()) == Fmt::Dense && formatOf(m.getRhs2()) == Fmt::Dense &&
                    m.getSemiring() == "plusxy_times" && !m.getMask() &&
                    mapsAre(m.getIndexingMaps(), {{0, 1}, {1, 2}, {0, 2}}))
                  return m;
        return nullptr;
      };
      if (fa == Fmt::CSR && fb == Fmt::Dense && fc == Fmt::CSR)
        if (TensorMultOp prod = denseProduct(b))
        {
          result = emitTensorCall(rewriter, set, kSddmm, {a, prod.getRhs1(), prod.getRhs2()}, dest.getType(), {});
          forwardStore(rewriter, dest, result, set);
          rewriter.eraseOp(set);
          rewriter.eraseOp(op);
          // the dense product itself is dead now if S .* T was its only reader; DCE removes it
          return success();
        }

      if (fa == Fmt::Dense && isSparse2D(fb))
      { // the product commutes: put the sparse operand first
        std::swap(a, b);
        std::swap(fa, fb);
      }
      if ((fa == Fmt::CSR || fa == Fmt::COO) && fb == Fmt::Dense && fc == fa)
        result = emitTensorCall(rewriter, set, kElewsSD, {a, b}, dest.getType(), {});
      else if (fa == Fmt::CSR && fb == Fmt::CSR && fc == Fmt::CSR)
        result = emitTensorCall(rewriter, set, kElewsSS, {a, b}, dest.getType(), {});
      else
        return failure();

      forwardStore(rewriter, dest, result, set);
      rewriter.eraseOp(set);
      rewriter.eraseOp(op);
      if (dest.use_empty())
        if (Operation *decl = dest.getDefiningOp())
          rewriter.eraseOp(decl);
      return success();
    }
  };

  /// SUM(C<M,push> = A * B) under plus-pair where C is only summed: the triangle-count idiom
  /// (test/integration/kernels/triangleCount_SandiaLL_wMasking.ta).  Runs after MulToB200, so the
  /// product is already a @b200.spgemm call; if ta.reduce is its only reader the pair collapses into
  /// one counting call and C is never stored.
  struct ReduceOfMaskedPairToB200 : public OpRewritePattern<ReduceOp>
  {
    using OpRewritePattern<ReduceOp>::OpRewritePattern;

    LogicalResult matchAndRewrite(ReduceOp op, PatternRewriter &rewriter) const final
    {
      auto call = op.getRhs().getDefiningOp<func::CallOp>();
      if (!call || !call.getCallee().starts_with(kSpgemm) || !call->hasAttr(kMaskedAttr))
        return failure();
      if (cast<IntegerAttr>(call->getAttr(kSemiringAttr)).getInt() != 1 /* plus-pair */)
        return failure();
      if (!call.getResult(0).hasOneUse() || !op.getResult().getType().isF64())
        return failure();
      rewriter.setInsertionPoint(op);
      Value count = emitTensorCall(rewriter, op, kMaskedCount, call.getOperands(), rewriter.getF64Type(), {});
      rewriter.replaceOp(op, count);
      rewriter.eraseOp(call);
      return success();
    }
  };

  struct ConvertTensorAlgebraToB200Pass
      : public mlir::comet::impl::ConvertTensorAlgebraToB200Base<ConvertTensorAlgebraToB200Pass>
  {
    void runOnOperation() override
    {
      RewritePatternSet patterns(&getContext());
      // elementwise first: the SDDMM pattern has to see the dense ta.mul before MulToB200 could
      // touch it (it never matches dense x dense, but the order keeps the intent visible)
      patterns.add<ElewsToB200>(&getContext(), /*benefit=*/3);
      patterns.add<MulToB200>(&getContext(), /*benefit=*/2);
      patterns.add<ReduceOfMaskedPairToB200>(&getContext(), /*benefit=*/1);
      if (failed(applyPatternsAndFoldGreedily(getOperation(), std::move(patterns))))
        signalPassFailure();
    }
  };

  //===--------------------------------------------------------------------===//
  // Stage 2: func.call @b200.<op> on tensors  ->  func.call @comet_b200_<op>_f64_i{64,32} on memrefs
  //===--------------------------------------------------------------------===//

  struct Lowering
  {
    PatternRewriter &rewriter;
    Location loc;
    ModuleOp module;
    MLIRContext *ctx;
    IntegerType i32, i64;
    IndexType index;

    Lowering(PatternRewriter &r, Operation *at)
        : rewriter(r), loc(at->getLoc()), module(at->getParentOfType<ModuleOp>()), ctx(at->getContext()),
          i32(IntegerType::get(ctx, 32)), i64(IntegerType::get(ctx, 64)), index(IndexType::get(ctx)) {}

    Value cI32(int v) { return rewriter.create<ConstantOp>(loc, i32, rewriter.getI32IntegerAttr(v)); }
    Value cIdx(int64_t v) { return rewriter.create<ConstantIndexOp>(loc, v); }

    /// One sparse operand in the order of COMET_B200_SPARSE2D: the same sequence of ops the sparse
    /// transpose lowering builds (TensorAlgebraToSCF.cpp:296-338).
    void sparseArgs(Value tensor, SmallVectorImpl<Value> &args, SmallVectorImpl<Type> &types)
    {
      auto sp = cast<SparseTensorType>(tensor.getType());
      Type idxMem = UnrankedMemRefType::get(sp.getIndicesType(), 0);
      Type valMem = UnrankedMemRefType::get(sp.getElementType(), 0);
      Type dimMem = UnrankedMemRefType::get(index, 0);
      std::string formats(getTensorFormatString(tensor.getType()));
      for (Value f : getFormatsValueInt(formats, 2, rewriter, loc, i32)) // A1format, A1tile, A2format, A2tile
      {
        args.push_back(f);
        types.push_back(i32);
      }
      auto pushIndexArray = [&](Value t) {
        auto shaped = cast<ShapedType>(t.getType());
        Value m = rewriter.create<ToMemrefOp>(loc, MemRefType::get(shaped.getShape(), shaped.getElementType()), t);
        args.push_back(rewriter.create<memref::CastOp>(loc, idxMem, m));
        types.push_back(idxMem);
      };
      for (int d = 0; d < 2; d++)
      {
        auto dim = rewriter.getI32IntegerAttr(d);
        pushIndexArray(rewriter.create<SpTensorGetDimPos>(loc, tensor, dim));
        pushIndexArray(rewriter.create<SpTensorGetDimCrd>(loc, tensor, dim));
        pushIndexArray(rewriter.create<SpTensorGetDimBlockPos>(loc, tensor, dim));
        pushIndexArray(rewriter.create<SpTensorGetDimBlockCrd>(loc, tensor, dim));
      }
      Value vals = rewriter.create<SpTensorGetVals>(loc, tensor);
      Value valsMem = rewriter.create<ToMemrefOp>(loc, MemRefType::get({ShapedType::kDynamic}, sp.getElementType()), vals);
      args.push_back(rewriter.create<memref::CastOp>(loc, valMem, valsMem));
      types.push_back(valMem);
      // {rows, cols}: the dims tensor of the construct op, as the transpose lowering passes it
      Value dims = cast<SparseTensorConstructOp>(tensor.getDefiningOp()).getDims();
      auto dimsT = cast<ShapedType>(dims.getType());
      Value dimsMem = rewriter.create<ToMemrefOp>(loc, MemRefType::get(dimsT.getShape(), dimsT.getElementType()), dims);
      args.push_back(rewriter.create<memref::CastOp>(loc, dimMem, dimsMem));
      types.push_back(dimMem);
    }

    /// A dense operand as one unranked memref; returns the ranked memref too (results are re-wrapped).
    Value denseArg(Value tensor, SmallVectorImpl<Value> &args, SmallVectorImpl<Type> &types)
    {
      auto t = cast<TensorType>(tensor.getType());
      Value m = rewriter.create<ToMemrefOp>(loc, MemRefType::get(t.getShape(), t.getElementType()), tensor);
      Type um = UnrankedMemRefType::get(t.getElementType(), 0);
      args.push_back(rewriter.create<memref::CastOp>(loc, um, m));
      types.push_back(um);
      return m;
    }

    void i32Arg(int v, SmallVectorImpl<Value> &args, SmallVectorImpl<Type> &types)
    {
      args.push_back(cI32(v));
      types.push_back(i32);
    }

    std::string symbol(StringRef op, Value sparseOperand)
    {
      auto sp = cast<SparseTensorType>(sparseOperand.getType());
      return ("comet_b200_" + op + "_f64_i" + std::to_string(sp.getIndicesType().getWidth())).str();
    }

    func::CallOp call(StringRef name, ArrayRef<Value> args, ArrayRef<Type> types, TypeRange results = {})
    {
      declare(module, loc, name, FunctionType::get(ctx, types, results));
      return rewriter.create<func::CallOp>(loc, name, results, args);
    }

    /// The CSR result of a two-call operation: C2pos[rows + 1] and the 11-entry sizes array are
    /// allocated, the symbolic call fills them and returns a handle, C2crd / Cval are allocated from
    /// sizes[8] (nnz, the slot read_input_sizes_2D_f64 uses: SparseUtils.cpp:1672-1687), the numeric
    /// call fills them, and the arrays are wrapped in ta.spTensor_construct exactly like the arrays a
    /// file reader call has filled (TensorDeclLowering.cpp:985-1128).
    Value sparseResult(StringRef symbolicName, SmallVectorImpl<Value> &args, SmallVectorImpl<Type> &types,
                       Value rowsFrom, Value colsFrom, int colsDim, SparseTensorType resultType)
    {
      IntegerType idxTy = resultType.getIndicesType();
      Type idxMem = UnrankedMemRefType::get(idxTy, 0);
      Type i64Mem = UnrankedMemRefType::get(i64, 0);
      Type valMem = UnrankedMemRefType::get(resultType.getElementType(), 0);
      auto dynIdx = MemRefType::get({ShapedType::kDynamic}, idxTy);
      auto dynVal = MemRefType::get({ShapedType::kDynamic}, resultType.getElementType());

      Value rows = rewriter.create<SpTensorGetDimSize>(loc, rowsFrom, rewriter.getI32IntegerAttr(0));
      Value cols = rewriter.create<SpTensorGetDimSize>(loc, colsFrom, rewriter.getI32IntegerAttr(colsDim));
      Value rowsPlus1 = rewriter.create<AddIOp>(loc, rows, cIdx(1));
      Value pos = insertAllocAndInitialize(loc, dynIdx, ValueRange{rowsPlus1}, rewriter);
      Value sizes = rewriter.create<memref::AllocOp>(loc, MemRefType::get({11}, i64));
      args.push_back(rewriter.create<memref::CastOp>(loc, idxMem, pos));
      types.push_back(idxMem);
      args.push_back(rewriter.create<memref::CastOp>(loc, i64Mem, sizes));
      types.push_back(i64Mem);
      Value handle = call(symbolicName, args, types, TypeRange{i64}).getResult(0);

      Value nnz64 = rewriter.create<memref::LoadOp>(loc, sizes, ValueRange{cIdx(8)});
      Value nnz = rewriter.create<IndexCastOp>(loc, index, nnz64);
      Value crd = insertAllocAndInitialize(loc, dynIdx, ValueRange{nnz}, rewriter);
      Value val = insertAllocAndInitialize(loc, dynVal, ValueRange{nnz}, rewriter);
      std::string numeric = "comet_b200_spgemm_numeric_f64_i" + std::to_string(idxTy.getWidth());
      SmallVector<Value> nargs{handle, rewriter.create<memref::CastOp>(loc, idxMem, crd),
                               rewriter.create<memref::CastOp>(loc, valMem, val)};
      SmallVector<Type> ntypes{i64, idxMem, valMem};
      call(numeric, nargs, ntypes);

      // A1pos = {rows}, A1crd and the tile arrays empty, like every CSR tensor COMET builds
      // (lib/Conversion/IndexTreeToSCF/SymbolicDomainConversion.cpp:262-271)
      Value a1pos = insertAllocAndInitialize(loc, dynIdx, ValueRange{cIdx(1)}, rewriter);
      Value rowsCast = idxTy.isIndex() ? rows : rewriter.create<IndexCastOp>(loc, idxTy, rows).getResult();
      rewriter.create<memref::StoreOp>(loc, rowsCast, a1pos, ValueRange{cIdx(0)});
      Value empty = insertAllocAndInitialize(loc, dynIdx, ValueRange{cIdx(0)}, rewriter);
      auto asTensor = [&](Value m) -> Value {
        return rewriter.create<ToTensorOp>(loc, m, rewriter.getUnitAttr(), rewriter.getUnitAttr());
      };
      Value dims = rewriter.create<tensor::FromElementsOp>(loc, ValueRange{rows, cols});
      auto formats = getFormats("CSR", 2, ctx);
      SmallVector<Attribute> formatAttrs;
      for (auto f : formats)
        formatAttrs.push_back(TensorFormatEnumAttr::get(ctx, f));
      return rewriter.create<SparseTensorConstructOp>(
          loc, resultType, dims, ValueRange{asTensor(a1pos), asTensor(pos)}, ValueRange{asTensor(empty), asTensor(crd)},
          ValueRange{asTensor(empty), asTensor(empty)}, ValueRange{asTensor(empty), asTensor(empty)}, asTensor(val), 2,
          rewriter.getArrayAttr(formatAttrs));
    }

    /// A sparse result that shares an operand's pattern (sparse .* dense, SDDMM): the operand's index
    /// arrays are reused as they are -- what COMET does for this case
    /// (SymbolicDomainConversion.cpp:277-297) -- and only a value array is allocated.
    Value samePatternResult(Value like, Value &valsMemOut)
    {
      auto sp = cast<SparseTensorType>(like.getType());
      auto construct = cast<SparseTensorConstructOp>(like.getDefiningOp());
      Value oldVals = rewriter.create<SpTensorGetVals>(loc, like);
      Value n = rewriter.create<tensor::DimOp>(loc, oldVals, 0);
      valsMemOut = insertAllocAndInitialize(loc, MemRefType::get({ShapedType::kDynamic}, sp.getElementType()),
                                            ValueRange{n}, rewriter);
      Value vals = rewriter.create<ToTensorOp>(loc, valsMemOut, rewriter.getUnitAttr(), rewriter.getUnitAttr());
      return rewriter.create<SparseTensorConstructOp>(loc, sp, construct.getDims(), construct.getPosIndices(),
                                                      construct.getCrdIndices(), construct.getBlockPosIndices(),
                                                      construct.getBlockCrdIndices(), vals, 2,
                                                      construct.getDimensionFormats());
    }
  };

  struct FinalizeCall : public OpRewritePattern<func::CallOp>
  {
    using OpRewritePattern<func::CallOp>::OpRewritePattern;

    LogicalResult matchAndRewrite(func::CallOp op, PatternRewriter &rewriter) const final
    {
      StringRef callee = op.getCallee();
      if (!callee.starts_with("b200."))
        return failure();
      // operands must have been lowered: sparse ones to ta.spTensor_construct, dense ones to tensors
      // backed by an allocation (the declaration lowering passes have run)
      for (Value v : op.getOperands())
        if (isa<SparseTensorType>(v.getType()) && !v.getDefiningOp<SparseTensorConstructOp>())
          return failure();

      Lowering L(rewriter, op);
      rewriter.setInsertionPoint(op);
      SmallVector<Value> args;
      SmallVector<Type> types;
      auto intAttr = [&](StringRef name, int dflt) {
        auto a = op->getAttrOfType<IntegerAttr>(name);
        return a ? (int)a.getInt() : dflt;
      };
      const int semiring = intAttr(kSemiringAttr, 0);
      const int accumulate = intAttr(kAccumulateAttr, 1);

      if (callee.starts_with(kSpmv) || callee.starts_with(kSpmm))
      {
        // comet_b200_sp{mv,mm}_f64_iNN(A..., x|B, y|C, semiring, accumulate)
        L.sparseArgs(op.getOperand(0), args, types);
        L.denseArg(op.getOperand(1), args, types);
        Value out = L.denseArg(op.getOperand(2), args, types);
        L.i32Arg(semiring, args, types);
        L.i32Arg(accumulate, args, types);
        L.call(L.symbol(callee.starts_with(kSpmv) ? "spmv" : "spmm", op.getOperand(0)), args, types);
        // the runtime wrote into the output's own buffer: the result is that buffer seen as a tensor again
        Value res = rewriter.create<ToTensorOp>(L.loc, out, rewriter.getUnitAttr(), rewriter.getUnitAttr());
        rewriter.replaceOp(op, res);
        return success();
      }
      if (callee.starts_with(kDenseSparse))
      {
        // comet_b200_dense_times_sparse_f64_iNN(A, B..., C, semiring, accumulate)
        L.denseArg(op.getOperand(0), args, types);
        L.sparseArgs(op.getOperand(1), args, types);
        Value out = L.denseArg(op.getOperand(2), args, types);
        L.i32Arg(semiring, args, types);
        L.i32Arg(accumulate, args, types);
        L.call(L.symbol("dense_times_sparse", op.getOperand(1)), args, types);
        rewriter.replaceOp(op, rewriter.create<ToTensorOp>(L.loc, out, rewriter.getUnitAttr(), rewriter.getUnitAttr()));
        return success();
      }
      if (callee.starts_with(kSpgemm))
      {
        // comet_b200_spgemm_symbolic_f64_iNN(A..., B..., M..., mask_type, semiring, C2pos, sizes) -> handle
        const bool masked = op->hasAttr(kMaskedAttr);
        L.sparseArgs(op.getOperand(0), args, types);
        L.sparseArgs(op.getOperand(1), args, types);
        L.sparseArgs(masked ? op.getOperand(2) : op.getOperand(0), args, types); // ignored when mask_type = 0
        L.i32Arg(masked ? 1 : 0, args, types);
        L.i32Arg(semiring, args, types);
        Value C = L.sparseResult(L.symbol("spgemm_symbolic", op.getOperand(0)), args, types, op.getOperand(0),
                                 op.getOperand(1), 1, cast<SparseTensorType>(op.getResult(0).getType()));
        rewriter.replaceOp(op, C);
        return success();
      }
      if (callee.starts_with(kElewsSS))
      {
        L.sparseArgs(op.getOperand(0), args, types);
        L.sparseArgs(op.getOperand(1), args, types);
        Value C = L.sparseResult(L.symbol("elews_mul_sparse_sparse_symbolic", op.getOperand(0)), args, types,
                                 op.getOperand(0), op.getOperand(0), 1, cast<SparseTensorType>(op.getResult(0).getType()));
        rewriter.replaceOp(op, C);
        return success();
      }
      if (callee.starts_with(kElewsSD) || callee.starts_with(kSddmm))
      {
        // comet_b200_elews_mul_sparse_dense_f64_iNN(A..., B, C...) / comet_b200_sddmm_f64_iNN(S..., X, D, O...)
        Value valsMem;
        Value C = L.samePatternResult(op.getOperand(0), valsMem);
        L.sparseArgs(op.getOperand(0), args, types);
        L.denseArg(op.getOperand(1), args, types);
        if (callee.starts_with(kSddmm))
          L.denseArg(op.getOperand(2), args, types);
        L.sparseArgs(C, args, types);
        L.call(L.symbol(callee.starts_with(kSddmm) ? "sddmm" : "elews_mul_sparse_dense", op.getOperand(0)), args, types);
        rewriter.replaceOp(op, C);
        return success();
      }
      if (callee.starts_with(kMaskedCount))
      {
        // comet_b200_masked_spgemm_count_f64_iNN(A..., B..., M..., push, plus-pair, out) ; out[0] is an i64 count
        L.sparseArgs(op.getOperand(0), args, types);
        L.sparseArgs(op.getOperand(1), args, types);
        L.sparseArgs(op.getOperand(2), args, types);
        L.i32Arg(1, args, types);
        L.i32Arg(1, args, types);
        Value out = rewriter.create<memref::AllocOp>(L.loc, MemRefType::get({1}, L.i64));
        Type um = UnrankedMemRefType::get(L.i64, 0);
        args.push_back(rewriter.create<memref::CastOp>(L.loc, um, out));
        types.push_back(um);
        L.call(L.symbol("masked_spgemm_count", op.getOperand(0)), args, types);
        Value n = rewriter.create<memref::LoadOp>(L.loc, out, ValueRange{L.cIdx(0)});
        rewriter.replaceOp(op, rewriter.create<SIToFPOp>(L.loc, rewriter.getF64Type(), n).getResult());
        return success();
      }
      return failure();
    }
  };

  struct FinalizeB200CallsPass : public mlir::comet::impl::FinalizeB200CallsBase<FinalizeB200CallsPass>
  {
    void runOnOperation() override
    {
      func::FuncOp function = getOperation();
      RewritePatternSet patterns(&getContext());
      patterns.add<FinalizeCall>(&getContext());
      if (failed(applyPatternsAndFoldGreedily(function, std::move(patterns))))
        return signalPassFailure();
      // the tensor-level declarations are dead now
      auto module = function->getParentOfType<ModuleOp>();
      SmallVector<func::FuncOp> dead;
      for (auto f : module.getOps<func::FuncOp>())
        if (f.isPrivate() && f.getName().starts_with("b200.") && f.symbolKnownUseEmpty(module))
          dead.push_back(f);
      for (auto f : dead)
        f.erase();
    }
  };
} // end anonymous namespace

std::unique_ptr<Pass> mlir::comet::createConvertTensorAlgebraToB200Pass()
{
  return std::make_unique<ConvertTensorAlgebraToB200Pass>();
}

std::unique_ptr<Pass> mlir::comet::createFinalizeB200CallsPass()
{
  return std::make_unique<FinalizeB200CallsPass>();
}
