/*
 * libcomet_b200 -- C ABI of the B200 execution path for COMET's sparse
 * tensor-algebra operations (ta.mul / ta.elews_mul on CSR, DCSR and COO
 * operands, semirings plus-times and plus-pair, f64 values, i64 indices).
 *
 * Two layers, both plain C (pointers, sizes, no C++ or torch types):
 *
 *  1. comet_b200_<op>_f64_i64(...)      HOST memref descriptors.  These are the
 *     symbols a COMET lowering emits func.call's to, next to read_input_2D_f64_i64
 *     and comet_sort64.  Argument conventions follow COMET's existing runtime
 *     calls (paths below are relative to the COMET source tree):
 *       - a memref<?xT> crosses the boundary as (int64 rank, void *desc) where
 *         desc points to {T *allocated; T *aligned; int64 offset; int64 sizes[rank];
 *         int64 strides[rank]}   (lib/ExecutionEngine/SparseUtils.cpp:1829-1837,
 *         :2622-2626; frontends/numpy-scipy/cometpy/MLIRGen/utils.py:5-21);
 *       - a sparse tensor is passed as four format integers followed by, per
 *         dimension, pos, crd, tile_pos, tile_crd, and finally vals, exactly as
 *         transpose_2D_f64_i64 receives its operands
 *         (lib/Conversion/TensorAlgebraToSCF/TensorAlgebraToSCF.cpp:303-400,
 *          lib/ExecutionEngine/TransposeUtils.cpp:1439-1451), then a
 *         memref<2xindex> holding {rows, cols} (same file :339-343);
 *       - format integers use the runtime encoding Dense=0, Compressed_unique=1,
 *         Compressed_nonunique=2, singleton=3, unknown=-1
 *         (include/comet/ExecutionEngine/RunnerUtils.h:71-77): CSR = (0,1),
 *         DCSR = (1,1), COO = (2,3);
 *       - the caller allocates every output; functions return void and results
 *         are complete in host memory on return, so comet_print_memref_* and
 *         ta.reduce code that follows keeps working;
 *       - symbol names follow <op>_f<valbits>_i<idxbits>
 *         (TensorAlgebraToSCF.cpp:360, TensorDeclLowering.cpp:1038).
 *     Tile arrays are accepted and ignored (always empty for CSR/DCSR/COO).
 *
 *  2. comet_b200_dev_<op>_f64_i64(...)  DEVICE pointers + sizes + a CUDA stream,
 *     asynchronous, returning 0 or an error status.  Layer 1 is a thin wrapper
 *     that stages host memrefs into device memory and calls layer 2.
 *
 * There is no CPU fallback: every entry point needs a CUDA device and fails
 * (message on stderr, then exit(1), like COMET's runtime; or a retrievable
 * error with COMET_B200_ON_ERROR=return) when none is usable.
 */
#ifndef COMET_B200_H
#define COMET_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define COMET_B200_EXPORT __attribute__((visibility("default")))
#else
#define COMET_B200_EXPORT
#endif

/* semiring of ta.mul: "plusxy_times" / "plusxy_pairxy"
   (frontends/comet_dsl/mlir/MLIRGen.cpp:102-145; arithmetic in
   lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:198-361) */
#define COMET_B200_PLUS_TIMES 0
#define COMET_B200_PLUS_PAIR 1
/* further semirings, taken by the sparse x sparse product only (the ones COMET tests on
   CSR x CSR: test/integration/semiring/mm_Semiring*_CSRxCSR_oCSR.ta) */
#define COMET_B200_PLUS_FIRST 2
#define COMET_B200_PLUS_SECOND 3
#define COMET_B200_MIN_PLUS 4
#define COMET_B200_MIN_FIRST 5
#define COMET_B200_MIN_SECOND 6
#define COMET_B200_ANY_PAIR 7

/* MaskType of ta.mul (include/comet/Dialect/TensorAlgebra/IR/TAOps.td:348-433) */
#define COMET_B200_MASK_NONE 0
#define COMET_B200_MASK_PUSH 1

/* runtime format codes (include/comet/ExecutionEngine/RunnerUtils.h:71-77) */
#define COMET_B200_FMT_DENSE 0
#define COMET_B200_FMT_CU 1
#define COMET_B200_FMT_CN 2
#define COMET_B200_FMT_S 3

/* StridedMemRefType<T,1> and <T,2> of MLIR's C runner ABI, restated. */
typedef struct {
    void *allocated;
    void *aligned;
    int64_t offset;
    int64_t sizes[1];
    int64_t strides[1];
} comet_b200_memref1d;

typedef struct {
    void *allocated;
    void *aligned;
    int64_t offset;
    int64_t sizes[2];
    int64_t strides[2];
} comet_b200_memref2d;

/* One sparse 2-D operand, in the order COMET passes it to its runtime. */
#define COMET_B200_SPARSE2D(P)                                                          \
    int32_t P##1format, int32_t P##1tile_format, int32_t P##2format, int32_t P##2tile_format, \
        int64_t P##1pos_rank, void *P##1pos_ptr, int64_t P##1crd_rank, void *P##1crd_ptr,     \
        int64_t P##1tile_pos_rank, void *P##1tile_pos_ptr, int64_t P##1tile_crd_rank,         \
        void *P##1tile_crd_ptr, int64_t P##2pos_rank, void *P##2pos_ptr, int64_t P##2crd_rank, \
        void *P##2crd_ptr, int64_t P##2tile_pos_rank, void *P##2tile_pos_ptr,                 \
        int64_t P##2tile_crd_rank, void *P##2tile_crd_ptr, int64_t P##val_rank, void *P##val_ptr, \
        int64_t P##dims_rank, void *P##dims_ptr

/* ------------------------------------------------------------------------- */
/* Layer 1: host memref descriptors                                           */
/* ------------------------------------------------------------------------- */

/* `accumulate` (spmv, spmm): 1 = the dense output holds values the products are
   added to, which is what COMET's loops do (they read-modify-write the output,
   IndexTreeToSCF.cpp:1266-1278); 0 = the lowering has seen the ta.fill 0.0 that
   precedes the multiply (every reference test has one), so the old contents are
   neither uploaded nor read. */

/* y[a] = y[a] (+) sum_b A[a,b] (x) x[b].  Replaces the loop nest COMET generates
   for ta.mul with a CSR/DCSR/COO lhs and a dense vector
   (lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:476-489, 667-783, 1247-1284;
   test/integration/ops/mult_spmv_{CSR,DCSR,COO}xDense.ta). */
COMET_B200_EXPORT void comet_b200_spmv_f64_i64(COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr,
                                               int64_t y_rank, void *y_ptr, int32_t semiring,
                                               int32_t accumulate);

/* C[a,c] = C[a,c] (+) sum_b A[a,b] (x) B[b,c], B and C row-major 2-D memrefs.
   Replaces the a->b->c loop nest of ta.mul sparse x dense
   (TensorAlgebraToIndexTree.cpp:276-323; test/integration/ops/mult_spmm_*xDense.ta). */
COMET_B200_EXPORT void comet_b200_spmm_f64_i64(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                               int64_t C_rank, void *C_ptr, int32_t semiring,
                                               int32_t accumulate);

/* C[a,c] = C[a,c] (+) sum_b A[a,b] (x) B[b,c] with dense A and C (both rank-1 vectors or both
   row-major rank-2 matrices) and sparse B (CSR, DCSR or COO): the dense x sparse forms of ta.mul
   (test/integration/ops/mult_Dense{Mat,Vec}x{CSR,DCSR,COO}.ta; loops a -> b -> c,
   lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:476-489, 667-783). */
COMET_B200_EXPORT void comet_b200_dense_times_sparse_f64_i64(int64_t A_rank, void *A_ptr,
                                                             COMET_B200_SPARSE2D(B), int64_t C_rank,
                                                             void *C_ptr, int32_t semiring,
                                                             int32_t accumulate);

/* O = S .* (X * D): O takes S's pos/crd, O.val[p] = S.val[p] * sum_k X[i,k] * D[k,j].
   X is a row-major [rows, K] memref; D is a 2-D memref of sizes {K, cols} whose
   strides select the layout: {ld, 1} is the D[k,j] operand of
   test/integration/kernels/sddmm.ta, {1, ld} is a row-major [cols, K] matrix
   viewed transposed.  Replaces the ta.mul + ta.elews_mul pair that COMET fuses
   with --opt-fusion (lib/Dialect/IndexTree/Transforms/KernelFusion.cpp:127-144). */
COMET_B200_EXPORT void comet_b200_sddmm_f64_i64(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                int64_t D_rank, void *D_ptr,
                                                COMET_B200_SPARSE2D(O));

/* C = A .* B with sparse A (CSR or COO) and dense row-major B; C takes A's
   pos/crd (lib/Conversion/IndexTreeToSCF/SymbolicDomainConversion.cpp:277-297;
   test/integration/ops/eltwise_mult_{CSR,COO}xDense_o{CSR,COO}.ta). */
COMET_B200_EXPORT void comet_b200_elews_mul_sparse_dense_f64_i64(COMET_B200_SPARSE2D(A),
                                                                 int64_t B_rank, void *B_ptr,
                                                                 COMET_B200_SPARSE2D(C));

/* C = A .* B with sparse A (CSR, DCSR or COO), dense row-major B and a DENSE row-major C: the
   products are assigned at A's stored positions, every other element of C keeps its value
   (test/integration/ops/eltwise_mult_{CSR,DCSR}xDense_oDense.ta, eltwise_mult_DensexCSR_oDense.ta;
   the multiplication commutes, so dense .* sparse is the same call). */
COMET_B200_EXPORT void comet_b200_elews_mul_sparse_dense_to_dense_f64_i64(COMET_B200_SPARSE2D(A),
                                                                          int64_t B_rank, void *B_ptr,
                                                                          int64_t C_rank, void *C_ptr);

/* The MatrixMarket reader with its sort on the device: same argument lists as read_input_sizes_2D_f64 and
   read_input_2D_f64_{i64,i32} (lib/ExecutionEngine/SparseUtils.cpp:2427-2450, 2562-2568; memref ranks as
   int64_t).  The file is named by the environment variable SPARSE_FILE_NAME<fileID> (SPARSE_FILE_NAME for
   fileID 9999).  The sizes call fills the 11-entry array {A1pos, A1crd, A1tile_pos, A1tile_crd, A2pos, A2crd,
   A2tile_pos, A2tile_crd, nnz, rows, cols}; the caller allocates and the second call fills.  readMode:
   1 all entries, 2 strictly lower triangle, 3 lower, 4 strictly upper, 5 upper (CSR and COO; DCSR keeps all). */
COMET_B200_EXPORT void comet_b200_read_input_sizes_2D_f64(int32_t fileID, int32_t A1format, int32_t A1tile_format,
                                                          int32_t A2format, int32_t A2tile_format,
                                                          int64_t sizes_rank, void *sizes_ptr, int32_t readMode);
COMET_B200_EXPORT void comet_b200_read_input_2D_f64_i64(
    int32_t fileID, int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format,
    int64_t A1pos_rank, void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank,
    void *A1tile_pos_ptr, int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr,
    int64_t A2crd_rank, void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr, int64_t A2tile_crd_rank,
    void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t readMode);
COMET_B200_EXPORT void comet_b200_read_input_2D_f64_i32(
    int32_t fileID, int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format,
    int64_t A1pos_rank, void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank,
    void *A1tile_pos_ptr, int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr,
    int64_t A2crd_rank, void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr, int64_t A2tile_crd_rank,
    void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t readMode);

/* B = transpose(A) for a sparse matrix: replaces transpose_2D_f64_i64 of the reference runtime
   (lib/ExecutionEngine/TransposeUtils.cpp:1439-1466) with the same argument list (memref ranks as int64_t):
   the four format codes and the eight index memrefs of A, A's values, the same for B, and the `sizes` memref
   whose first two entries are {rows, cols} of A and are swapped on return.  CSR -> CSR and COO -> COO, the
   two pairs the reference handles; the caller has allocated B's arrays (B2pos of cols+1 entries for CSR). */
COMET_B200_EXPORT void comet_b200_transpose_2D_f64_i64(
    int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format, int64_t A1pos_rank,
    void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank, void *A1tile_pos_ptr,
    int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr, int64_t A2crd_rank,
    void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr, int64_t A2tile_crd_rank,
    void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t B1format, int32_t B1tile_format,
    int32_t B2format, int32_t B2tile_format, int64_t B1pos_rank, void *B1pos_ptr, int64_t B1crd_rank,
    void *B1crd_ptr, int64_t B1tile_pos_rank, void *B1tile_pos_ptr, int64_t B1tile_crd_rank,
    void *B1tile_crd_ptr, int64_t B2pos_rank, void *B2pos_ptr, int64_t B2crd_rank, void *B2crd_ptr,
    int64_t B2tile_pos_rank, void *B2tile_pos_ptr, int64_t B2tile_crd_rank, void *B2tile_crd_ptr,
    int64_t Bval_rank, void *Bval_ptr, int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT void comet_b200_transpose_2D_f64_i32(
    int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format, int64_t A1pos_rank,
    void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank, void *A1tile_pos_ptr,
    int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr, int64_t A2crd_rank,
    void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr, int64_t A2tile_crd_rank,
    void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t B1format, int32_t B1tile_format,
    int32_t B2format, int32_t B2tile_format, int64_t B1pos_rank, void *B1pos_ptr, int64_t B1crd_rank,
    void *B1crd_ptr, int64_t B1tile_pos_rank, void *B1tile_pos_ptr, int64_t B1tile_crd_rank,
    void *B1tile_crd_ptr, int64_t B2pos_rank, void *B2pos_ptr, int64_t B2crd_rank, void *B2crd_ptr,
    int64_t B2tile_pos_rank, void *B2tile_pos_ptr, int64_t B2tile_crd_rank, void *B2tile_crd_ptr,
    int64_t Bval_rank, void *Bval_ptr, int64_t sizes_rank, void *sizes_ptr);

/* Sparse-output operations use the two-call protocol COMET already uses for
   file input (read_input_sizes_2D_f64 then read_input_2D_f64_i64,
   lib/Dialect/TensorAlgebra/Transforms/TensorDeclLowering.cpp:937-1052): the
   symbolic call fills C2pos[rows+1] and an 11-entry sizes array laid out like
   read_input_sizes_2D's (SparseUtils.cpp:1672-1687) and returns a handle; the
   caller allocates C2crd[nnz], Cval[nnz]; the numeric call fills them and
   releases the handle.  Output A1pos = {rows}, A1crd unused
   (SymbolicDomainConversion.cpp:262-271). */

/* C = A*B or C<M,push> = A*B, all CSR, Gustavson row by row.  Restates the
   workspace transformation and its symbolic phase
   (lib/Dialect/IndexTree/Transforms/WorkspaceTransforms.cpp:97-276,
    lib/Conversion/IndexTreeToSCF/SymbolicDomainConversion.cpp:81-340,
    lib/Conversion/TensorAlgebraToSCF/SparseTensorConversionPass.cpp:982-1159);
   output crd sorted per row like comet_sort64 leaves it.  Pass mask_type
   COMET_B200_MASK_NONE and any (ignored) M block when there is no mask.  The
   mask's crd must be ascending within a row. */
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_f64_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);

COMET_B200_EXPORT void comet_b200_spgemm_numeric_f64_i64(int64_t handle, int64_t C2crd_rank,
                                                         void *C2crd_ptr, int64_t Cval_rank,
                                                         void *Cval_ptr);

/* C = A .* B, both CSR: per-row intersection
   (lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:854-1073;
   test/integration/ops/eltwise_mult_CSRxCSR_oCSR.ta).  Same protocol; finish
   with comet_b200_spgemm_numeric_f64_i64. */
COMET_B200_EXPORT int64_t comet_b200_elews_mul_sparse_sparse_symbolic_f64_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), int64_t C2pos_rank, void *C2pos_ptr,
    int64_t sizes_rank, void *sizes_ptr);

/* Drops a handle without running the numeric phase. */
COMET_B200_EXPORT void comet_b200_handle_destroy(int64_t handle);

/* out[0] = SUM(C<M,push> = A*B) under plus-pair, as an exact int64, without
   storing C: the fused form of the masked ta.mul + ta.reduce of
   test/integration/kernels/triangleCount_SandiaLL_wMasking.ta
   (mask: lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:1075-1162, 1327-1448;
    reduce: lib/Conversion/TensorAlgebraToSCF/TensorAlgebraToSCF.cpp:417-529).
   With A = B = M = L (strict lower triangle) this is the triangle count. */
COMET_B200_EXPORT void comet_b200_masked_spgemm_count_f64_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t out_rank, void *out_ptr);

/* ------------------------------------------------------------------------- */
/* The same entry points for 32-bit index arrays (pos / crd memrefs of i32;    */
/* dims, sizes and the count stay 64-bit).  COMET picks the index width per    */
/* tensor type: i64 on its CPU target (frontends/comet_dsl/comet.cpp:817-823), */
/* and cometpy keeps scipy's int32 index arrays, which instantiates the _i32   */
/* runtime symbols (frontends/numpy-scipy/cometpy/comet.py:198-218; compare    */
/* read_input_2D_f64_i32, lib/ExecutionEngine/SparseUtils.cpp:2396).  Indices  */
/* are widened on the device; a sparse result with 2^31-1 or more entries is   */
/* refused.  A handle must be finished by the numeric call of the same width.  */
/* ------------------------------------------------------------------------- */
COMET_B200_EXPORT void comet_b200_spmv_f64_i32(COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr,
                                               int64_t y_rank, void *y_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_spmm_f64_i32(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                               int64_t C_rank, void *C_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_dense_times_sparse_f64_i32(int64_t A_rank, void *A_ptr,
                                                             COMET_B200_SPARSE2D(B), int64_t C_rank,
                                                             void *C_ptr, int32_t semiring,
                                                             int32_t accumulate);
COMET_B200_EXPORT void comet_b200_sddmm_f64_i32(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                int64_t D_rank, void *D_ptr,
                                                COMET_B200_SPARSE2D(O));
COMET_B200_EXPORT void comet_b200_elews_mul_sparse_dense_f64_i32(COMET_B200_SPARSE2D(A),
                                                                 int64_t B_rank, void *B_ptr,
                                                                 COMET_B200_SPARSE2D(C));
COMET_B200_EXPORT void comet_b200_elews_mul_sparse_dense_to_dense_f64_i32(COMET_B200_SPARSE2D(A),
                                                                          int64_t B_rank, void *B_ptr,
                                                                          int64_t C_rank, void *C_ptr);
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_f64_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT void comet_b200_spgemm_numeric_f64_i32(int64_t handle, int64_t C2crd_rank,
                                                         void *C2crd_ptr, int64_t Cval_rank,
                                                         void *Cval_ptr);
COMET_B200_EXPORT int64_t comet_b200_elews_mul_sparse_sparse_symbolic_f64_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), int64_t C2pos_rank, void *C2pos_ptr,
    int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT void comet_b200_masked_spgemm_count_f64_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t out_rank, void *out_ptr);

/* ------------------------------------------------------------------------- */
/* float values: COMET instantiates its runtime symbols for f32 as well        */
/* (read_input_2D_f32_i32 / _f32_i64, lib/ExecutionEngine/SparseUtils.cpp      */
/* :2354-2400).  Same argument lists; value memrefs (vals, x, y, B, C, X, D)   */
/* hold float.  Values are widened to double on the device after the upload    */
/* and results rounded to float once before the download, so a result equals   */
/* the double-precision result rounded to float.                               */
/* ------------------------------------------------------------------------- */
COMET_B200_EXPORT void comet_b200_spmv_f32_i64(COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr,
                                               int64_t y_rank, void *y_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_spmv_f32_i32(COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr,
                                               int64_t y_rank, void *y_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_spmm_f32_i64(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                               int64_t C_rank, void *C_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_spmm_f32_i32(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                               int64_t C_rank, void *C_ptr, int32_t semiring,
                                               int32_t accumulate);
COMET_B200_EXPORT void comet_b200_sddmm_f32_i64(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O));
COMET_B200_EXPORT void comet_b200_sddmm_f32_i32(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O));
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_f32_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_f32_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT void comet_b200_spgemm_numeric_f32_i64(int64_t handle, int64_t C2crd_rank, void *C2crd_ptr,
                                                         int64_t Cval_rank, void *Cval_ptr);
COMET_B200_EXPORT void comet_b200_spgemm_numeric_f32_i32(int64_t handle, int64_t C2crd_rank, void *C2crd_ptr,
                                                         int64_t Cval_rank, void *Cval_ptr);

/* ------------------------------------------------------------------------- */
/* Several GPUs: one process per GPU, one row block of the left operand per    */
/* rank.  COMET itself has no collective and no multi-device runtime (its      */
/* generated code calls the runtime from one host thread,                      */
/* lib/Dialect/TensorAlgebra/Transforms/TensorDeclLowering.cpp:937-1052), so   */
/* these entry points have no counterpart there; they are how a COMET program  */
/* started once per GPU (mpirun, torchrun) spreads one operation over a node.  */
/*                                                                             */
/* Set-up: rank 0 calls comet_b200_comm_unique_id, the host program hands the  */
/* 128 bytes to every rank (MPI_Bcast, a file, a socket), and every rank calls */
/* comet_b200_comm_init with its CUDA device current.  NCCL is loaded with     */
/* dlopen at that moment; single-GPU programs never touch it.                  */
/*                                                                             */
/* The *_sharded_* entry points take the same argument lists as the plain ones */
/* with this meaning: the LEFT sparse operand (A, S), the mask M, the dense X  */
/* of SDDMM and every OUTPUT are this rank's contiguous row block (row pointer */
/* starting at 0); the RIGHT operand (B, D = Y, B of the sparse product) is    */
/* the whole matrix and must hold the same contents on every rank.  Each rank  */
/* uploads one N-th of the right operand over its own PCIe link, the slices    */
/* are exchanged between the GPUs (ncclAllGather into each GPU's own memory),  */
/* and the single-GPU kernels run on local memory.  The calls are collective:  */
/* every rank makes the same call in the same order; a rank whose operands     */
/* are refused makes all ranks return with an error instead of leaving the     */
/* others waiting.                                                             */
/* ------------------------------------------------------------------------- */
COMET_B200_EXPORT int32_t comet_b200_comm_unique_id(void *id_out, int64_t id_bytes);   /* id_bytes >= 128 */
COMET_B200_EXPORT int32_t comet_b200_comm_init(int32_t nranks, int32_t rank, const void *id);
COMET_B200_EXPORT int32_t comet_b200_comm_nranks(void);   /* 0 without a communicator */
COMET_B200_EXPORT int32_t comet_b200_comm_rank(void);     /* -1 without a communicator */
COMET_B200_EXPORT int32_t comet_b200_comm_destroy(void);
/* bytes of one slice when `total_bytes` of a replicated array are exchanged between `nranks` ranks:
   ceil(total / nranks) rounded up to 256 (a pure function; needs no device) */
COMET_B200_EXPORT int64_t comet_b200_comm_slice_bytes(int64_t total_bytes, int32_t nranks);

COMET_B200_EXPORT void comet_b200_spmm_sharded_f64_i64(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                                       int64_t C_rank, void *C_ptr, int32_t semiring,
                                                       int32_t accumulate);
COMET_B200_EXPORT void comet_b200_sddmm_sharded_f64_i64(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                        int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O));
/* sizes: as in the plain call for this rank's block; when the memref holds 13 entries or more,
   sizes[11] = entries held by the blocks of the lower ranks (this block's offset in the whole C2crd / Cval)
   and sizes[12] = entries of all blocks together (one ncclAllGather of the per-rank counts).  Finish
   with comet_b200_spgemm_numeric_f64_i64 on the block's own arrays. */
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_sharded_f64_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);
/* out[0] = the count over the blocks of ALL ranks (ncclAllReduce on the stream of the counting kernels) */
COMET_B200_EXPORT void comet_b200_masked_spgemm_count_sharded_f64_i64(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t out_rank, void *out_ptr);
COMET_B200_EXPORT void comet_b200_spmm_sharded_f64_i32(COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                                                       int64_t C_rank, void *C_ptr, int32_t semiring,
                                                       int32_t accumulate);
COMET_B200_EXPORT void comet_b200_sddmm_sharded_f64_i32(COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr,
                                                        int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O));
COMET_B200_EXPORT int64_t comet_b200_spgemm_symbolic_sharded_f64_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr);
COMET_B200_EXPORT void comet_b200_masked_spgemm_count_sharded_f64_i32(
    COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type,
    int32_t semiring, int64_t out_rank, void *out_ptr);

/* Collectives of the device layer on the communicator of the current device, asynchronous on `stream`:
   sum of n int64 in place; all[r] = rank r's *one; completion of a buffer of nranks slices of slice_bytes
   of which this rank has filled slice number rank. */
COMET_B200_EXPORT int32_t comet_b200_dev_allreduce_sum_i64(int64_t *buf, int64_t n, void *stream);
COMET_B200_EXPORT int32_t comet_b200_dev_allgather_i64(const int64_t *one, int64_t *all, void *stream);
COMET_B200_EXPORT int32_t comet_b200_dev_allgather_slices(void *buf, int64_t slice_bytes, void *stream);

/* ------------------------------------------------------------------------- */
/* The same operations in the shape cometpy calls its kernels with.            */
/* cometpy emits each kernel with llvm.emit_c_interface and calls              */
/* _mlir_ciface_<kernel> through ctypes                                        */
/* (frontends/numpy-scipy/cometpy/MLIRGen/ops.py:548-553, lowering.py:212-460):*/
/* results first, one POINTER per shaped result (a memref struct for a dense   */
/* result; for a CSR result the struct {dims, insert_1, A1pos, insert_2, A2pos,*/
/* A2crd, Aval} of MLIRGen/utils.py:26-27), filled by the callee with malloc'ed*/
/* arrays that cometpy wraps without copying (lowering.py:433-448); then the   */
/* inputs, a dense array as one memref POINTER, a scipy CSR matrix as seven    */
/* arguments: dims*, insert_pos_1 (by value), A1pos*, insert_pos_2 (by value), */
/* A2pos*, A2crd*, Aval* (lowering.py:298-321).  A scalar result is returned.  */
/* `C` / `O` point to the CSR result struct.  The insert positions are         */
/* ignored.  Release result arrays with comet_b200_ciface_free (= free).       */
/* ------------------------------------------------------------------------- */
#define COMET_B200_CIFACE_CSR(P)                                                                      \
    comet_b200_memref1d *P##dims, int64_t P##insert_1, comet_b200_memref1d *P##1pos, int64_t P##insert_2, \
        comet_b200_memref1d *P##2pos, comet_b200_memref1d *P##2crd, comet_b200_memref1d *P##val

COMET_B200_EXPORT void _mlir_ciface_comet_b200_spmv_csr_f64_i64(comet_b200_memref1d *y, COMET_B200_CIFACE_CSR(A),
                                                                comet_b200_memref1d *x);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spmm_csr_f64_i64(comet_b200_memref2d *C, COMET_B200_CIFACE_CSR(A),
                                                                comet_b200_memref2d *B);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spgemm_csr_f64_i64(void *C, COMET_B200_CIFACE_CSR(A),
                                                                  COMET_B200_CIFACE_CSR(B), int64_t semiring);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spgemm_masked_csr_f64_i64(void *C, COMET_B200_CIFACE_CSR(A),
                                                                         COMET_B200_CIFACE_CSR(B),
                                                                         COMET_B200_CIFACE_CSR(M), int64_t semiring);
COMET_B200_EXPORT double _mlir_ciface_comet_b200_masked_count_csr_f64_i64(COMET_B200_CIFACE_CSR(A),
                                                                          COMET_B200_CIFACE_CSR(B),
                                                                          COMET_B200_CIFACE_CSR(M));
/* Y is the row-major [cols, K] operand */
COMET_B200_EXPORT void _mlir_ciface_comet_b200_sddmm_csr_f64_i64(void *O, COMET_B200_CIFACE_CSR(S),
                                                                 comet_b200_memref2d *X, comet_b200_memref2d *Y);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spmv_csr_f64_i32(comet_b200_memref1d *y, COMET_B200_CIFACE_CSR(A),
                                                                comet_b200_memref1d *x);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spmm_csr_f64_i32(comet_b200_memref2d *C, COMET_B200_CIFACE_CSR(A),
                                                                comet_b200_memref2d *B);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spgemm_csr_f64_i32(void *C, COMET_B200_CIFACE_CSR(A),
                                                                  COMET_B200_CIFACE_CSR(B), int64_t semiring);
COMET_B200_EXPORT void _mlir_ciface_comet_b200_spgemm_masked_csr_f64_i32(void *C, COMET_B200_CIFACE_CSR(A),
                                                                         COMET_B200_CIFACE_CSR(B),
                                                                         COMET_B200_CIFACE_CSR(M), int64_t semiring);
COMET_B200_EXPORT double _mlir_ciface_comet_b200_masked_count_csr_f64_i32(COMET_B200_CIFACE_CSR(A),
                                                                          COMET_B200_CIFACE_CSR(B),
                                                                          COMET_B200_CIFACE_CSR(M));
COMET_B200_EXPORT void _mlir_ciface_comet_b200_sddmm_csr_f64_i32(void *O, COMET_B200_CIFACE_CSR(S),
                                                                 comet_b200_memref2d *X, comet_b200_memref2d *Y);
COMET_B200_EXPORT void comet_b200_ciface_free(void *p);

/* ------------------------------------------------------------------------- */
/* Error reporting (COMET's runtime has none beyond stderr + exit; see         */
/* SparseUtils.cpp:158-168).                                                   */
/* ------------------------------------------------------------------------- */
COMET_B200_EXPORT const char *comet_b200_last_error(void);   /* "" when the last call succeeded */
COMET_B200_EXPORT void comet_b200_set_error_mode(int32_t return_instead_of_exit);
COMET_B200_EXPORT int32_t comet_b200_version(void);

/* ------------------------------------------------------------------------- */
/* Layer 2: device pointers.  All arrays live in the current device's memory; */
/* `stream` is a cudaStream_t (NULL = default stream).  row_ids, when not      */
/* NULL, maps stored row r to its coordinate (the A1crd array of DCSR) and     */
/* nrows is then the number of stored rows.  Returns 0 on success.             */
/*                                                                             */
/* Preconditions the device layer does not check (layer 1 checks them before   */
/* it calls down): nnz equals pos[nrows] -- work lists are sized from it, and  */
/* with a smaller value long rows would be left out --, pos starts at 0 and    */
/* never decreases, every coordinate lies inside the matrix.                   */
/*                                                                             */
/* Concurrency: the entry points of this layer keep their work lists, counters */
/* and narrowed index copies in ONE scratch area per device, which is reused   */
/* (and grown, with a device synchronisation) from call to call.  Calls on the */
/* same device must therefore not overlap: issue them from one host thread at  */
/* a time and onto one stream at a time (or order the streams with events).    */
/* Different devices are independent.                                          */
/* ------------------------------------------------------------------------- */
COMET_B200_EXPORT int32_t comet_b200_dev_spmv_f64_i64(int64_t nrows, int64_t nnz,
                                                      const int64_t *row_ids,
                                                      const int64_t *pos, const int64_t *crd,
                                                      const double *val, const double *x, double *y,
                                                      int32_t semiring, int32_t accumulate,
                                                      void *stream);

/* variant: 0 = automatic.  Bits 24-25 pick the kernel family: 0 = by shape (the entry-stream kernel
   from 64 columns and 65536 stored entries on, for plus-times; the row-panel kernels otherwise),
   1 = entry stream whenever the shape allows it (K even, at most 256; worth asking for with
   narrow B and a power-law A, where it is several times faster than the panels),
   2 = row panels, 3 = the entry stream with the rows of B staged by TMA bulk copies
   (cp.async.bulk completing on an mbarrier) instead of per-lane cp.async; with bit 26 set as well, one
   cp.async.bulk.tensor ... tile::gather4 copy per stage of four rows (a tensor map of B is built per call).  For the row panels the low bits are (panel width in columns) |
   (lanes per row << 16): the number of B columns handled per pass over A and the lane-group
   size, for tuning. */
COMET_B200_EXPORT int32_t comet_b200_dev_spmm_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz,
                                                      int64_t k,
                                                      const int64_t *row_ids, const int64_t *pos,
                                                      const int64_t *crd, const double *val,
                                                      const double *b, int64_t ldb, double *c,
                                                      int64_t ldc, int32_t semiring,
                                                      int32_t accumulate, int32_t variant,
                                                      void *stream);

/* SpMM that allocates nothing (this entry point has no counterpart in the
   reference; it exists for hosts of this library that cannot call cudaMalloc
   inside an operation: programs running under a fixed device-memory budget,
   latency-critical loops where an allocation could stall the device, runtimes
   that own the whole heap).  Same operation and arguments as
   comet_b200_dev_spmm_f64_i64 without the tuning knob; the long-row work list
   lives in a 4 MiB array inside the library image (held by every GPU that loads
   the library until the process exits) instead of growable scratch memory.
   Limits: nnz up to about 67 million (the list's capacity), k <= 256 and even,
   ldb/ldc even, b and c 16-byte aligned; anything beyond is refused with an
   error, never truncated.  The first call on a device looks up the array's
   device address; make that call before starting any stream capture.  All
   calls on a device share the array, so calls that can overlap on the GPU
   (different streams) race on it and must be serialised by the caller. */
COMET_B200_EXPORT int32_t comet_b200_dev_spmm_noalloc_f64_i64(
    int64_t nrows, int64_t nnz, int64_t k, const int64_t *row_ids, const int64_t *pos,
    const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
    int32_t semiring, int32_t accumulate, void *stream);

/* c[m, ncols] (+)= a[m, rows(B)] * B for the nstored rows B holds (row_ids as above).  With 32 or more rows
   of a and B in plain CSR (row_ids null) the product is formed transposed, C^T = B^T A^T, through the SpMM
   kernels (B is transposed on the device first; temporaries of the size of a, c and B come from the stream's
   memory pool); otherwise one f64 atomic per product and row of a. */
COMET_B200_EXPORT int32_t comet_b200_dev_dense_times_sparse_f64_i64(
    int64_t m, int64_t ncols, int64_t nstored, int64_t nnz, const int64_t *row_ids, const int64_t *pos,
    const int64_t *crd, const double *val, const double *a, int64_t lda, double *c, int64_t ldc,
    int32_t semiring, int32_t accumulate, void *stream);

/* y is row-major [ncols, k] with leading dimension ldy. */
COMET_B200_EXPORT int32_t comet_b200_dev_sddmm_f64_i64(int64_t nrows, int64_t nnz, int64_t k,
                                                       const int64_t *pos,
                                                       const int64_t *crd, const double *sval,
                                                       const double *x, int64_t ldx, const double *y,
                                                       int64_t ldy, double *out, void *stream);

/* Entries sorted by (major, minor); entries with equal coordinates keep their input order, as the
   std::stable_sort of the reference reader does (lib/ExecutionEngine/SparseUtils.cpp:360-367; duplicates
   are kept, not summed).  major_out / minor_out / vals_out may be NULL.  nmajor * nminor must fit 63 bits.
   Synchronises the stream (it reports coordinates outside nmajor x nminor). */
COMET_B200_EXPORT int32_t comet_b200_dev_sort_coo_f64_i64(int64_t n, int64_t nmajor, int64_t nminor,
                                                          const int64_t *major, const int64_t *minor,
                                                          const double *vals, int64_t *major_out,
                                                          int64_t *minor_out, double *vals_out, void *stream);

/* Coordinate entries in any order -> CSR arrays (pos[nrows+1], crd[nnz], val[nnz]) in the order the reference
   reader builds them (CooMatrix sort + CsrMatrix::Init, lib/ExecutionEngine/SparseUtils.cpp:360-533). */
COMET_B200_EXPORT int32_t comet_b200_dev_coo_to_csr_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz,
                                                            const int64_t *rows, const int64_t *cols,
                                                            const double *vals, int64_t *pos, int64_t *crd,
                                                            double *val, void *stream);

/* CSR of the transposed matrix: tpos[ncols+1], tcrd[nnz] (row indices of the input, ascending inside a
   column), tval[nnz].  The CSR -> CSR branch of transpose_2D (lib/ExecutionEngine/TransposeUtils.cpp:738-812). */
COMET_B200_EXPORT int32_t comet_b200_dev_csr_transpose_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz,
                                                               const int64_t *pos, const int64_t *crd,
                                                               const double *val, int64_t *tpos, int64_t *tcrd,
                                                               double *tval, void *stream);

/* dst[j, i] = src[i, j] for a row-major [rows, cols] src (used to bring a D[k,j]
   operand into the [cols, K] layout the SDDMM kernel gathers from). */
COMET_B200_EXPORT int32_t comet_b200_dev_transpose_f64(int64_t rows, int64_t cols, const double *src,
                                                       int64_t lds, double *dst, int64_t ldd,
                                                       void *stream);

/* rows == NULL: CSR (pos given); rows != NULL: COO (row coordinate per entry). */
COMET_B200_EXPORT int32_t comet_b200_dev_elews_mul_sparse_dense_f64_i64(
    int64_t nrows, int64_t nnz, const int64_t *pos, const int64_t *rows, const int64_t *crd,
    const double *val, const double *b, int64_t ldb, double *out, void *stream);

/* Dense-output form: c[row, col] = val * b[row, col] at the stored positions (pos/row_ids for CSR/DCSR
   with nstored rows, or rows != NULL for COO). */
COMET_B200_EXPORT int32_t comet_b200_dev_elews_mul_sparse_dense_to_dense_f64_i64(
    int64_t nstored, int64_t nnz, const int64_t *row_ids, const int64_t *pos, const int64_t *rows,
    const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
    void *stream);

/* Sparse-output operations on device arrays.  *handle_out receives a handle,
   cpos[nrows+1] is filled, *nnz_host (host memory) receives nnz(C) after an
   internal stream synchronisation (the caller has to size crd/val). */
COMET_B200_EXPORT int32_t comet_b200_dev_spgemm_symbolic_f64_i64(
    int64_t nrows, int64_t ncols_b, int64_t nnz_b, const int64_t *apos, const int64_t *acrd,
    const double *aval, const int64_t *bpos, const int64_t *bcrd, const double *bval,
    const int64_t *mpos, const int64_t *mcrd, int32_t semiring, int64_t *cpos, int64_t *nnz_host,
    int64_t *handle_out, void *stream);

COMET_B200_EXPORT int32_t comet_b200_dev_elews_mul_sparse_sparse_symbolic_f64_i64(
    int64_t nrows, const int64_t *apos, const int64_t *acrd, const double *aval,
    const int64_t *bpos, const int64_t *bcrd, const double *bval, int64_t *cpos, int64_t *nnz_host,
    int64_t *handle_out, void *stream);

/* The operand arrays given to the symbolic call must still be valid.  keep != 0
   leaves the handle alive so the numeric phase can be repeated (benchmarks). */
COMET_B200_EXPORT int32_t comet_b200_dev_spgemm_numeric_f64_i64(int64_t handle, int64_t *ccrd,
                                                                double *cval, int32_t keep,
                                                                void *stream);

/* *count_dev (device memory, int64) receives the number of products A[i,k]*B[k,j]
   with (i,j) stored in M, over rows [row_lo, row_hi) of A and M.  A duplicate
   coordinate in M counts once (a mask bit), one in A or B counts per occurrence,
   as in the reference's loops.  Rows of A and B need no ordering; a row of M must
   hold its coordinates in ascending order (equal ones adjacent), which is how
   COMET's reader leaves them (lib/ExecutionEngine/SparseUtils.cpp:360-367). */
COMET_B200_EXPORT int32_t comet_b200_dev_masked_spgemm_count_f64_i64(
    int64_t row_lo, int64_t row_hi, int64_t ncols, int64_t nnz_a, int64_t nnz_b, int64_t nnz_m,
    const int64_t *apos, const int64_t *acrd, const int64_t *bpos, const int64_t *bcrd,
    const int64_t *mpos, const int64_t *mcrd, int64_t *count_dev, void *stream);

/* Measurement aid (no counterpart in the reference): the bare gather SpMM / SDDMM are built around.  For
   each of the nnz column indices the k-double row b[crd[p], :] is read and folded into a sum; out
   (device, at least 8 * ctas_per_sm * SM-count doubles) receives one partial sum per warp.  fold_rows > 0
   maps every index into the first fold_rows rows (a working set that fits L2).  Timing it over a
   benchmark's column stream gives the rate a gather-per-entry kernel is bounded by on that stream. */
COMET_B200_EXPORT int32_t comet_b200_dev_gather_probe_f64_i64(int64_t nnz, const int64_t *crd, const double *b,
                                                              int64_t ldb, int64_t k, int64_t fold_rows,
                                                              int32_t ctas_per_sm, double *out, int64_t out_len,
                                                              void *stream);

/* Measurement aid: launches an empty kernel on `stream` (the launch floor of back-to-back small calls). */
COMET_B200_EXPORT int32_t comet_b200_dev_noop(void *stream);

/* Frees the library's scratch memory on the current device. */
COMET_B200_EXPORT void comet_b200_release_scratch(void);

#ifdef __cplusplus
}
#endif
#endif /* COMET_B200_H */
