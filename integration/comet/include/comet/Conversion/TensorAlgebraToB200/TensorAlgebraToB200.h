//===- TensorAlgebraToB200.h - ta.mul / ta.elews_mul -> libcomet_b200 calls -*- C++ -*-===//
//
// NOT COMPILED IN THIS REPOSITORY: it needs the COMET source tree and the LLVM/MLIR it is built
// against.  Copy the three directories under integration/comet/ over a COMET checkout (same relative
// paths) and apply frontends/comet_dsl/comet.cpp.diff.
//
//===----------------------------------------------------------------------===//

#ifndef COMET_CONVERSION_TENSORALGEBRATOB200_H
#define COMET_CONVERSION_TENSORALGEBRATOB200_H

#include "mlir/Support/LLVM.h"
#include <memory>

namespace mlir
{
  class Pass;

  namespace comet
  {
#define GEN_PASS_DECL_CONVERTTENSORALGEBRATOB200
#define GEN_PASS_DECL_FINALIZEB200CALLS
#include "comet/Conversion/Passes.h.inc"

    /// Stage 1, before createLowerTensorAlgebraToIndexTreePass(): every ta.mul / ta.elews_mul (with
    /// the ta.set_op that stores its result) whose operand formats, indexing maps and semiring
    /// libcomet_b200 implements is replaced by a TENSOR-LEVEL func.call to a private declaration
    /// named @b200.<op>; everything else is left for the index-tree path.
    std::unique_ptr<Pass> createConvertTensorAlgebraToB200Pass();

    /// Stage 2, after the tensor-declaration lowering passes (where ta.transpose of a sparse tensor is
    /// lowered to its runtime call today): each @b200.<op> call becomes the real call(s) into
    /// libcomet_b200 on unranked memrefs, sparse results are allocated with the two-call protocol
    /// and wrapped in ta.spTensor_construct.
    std::unique_ptr<Pass> createFinalizeB200CallsPass();
  }
} // namespace mlir

#endif // COMET_CONVERSION_TENSORALGEBRATOB200_H
