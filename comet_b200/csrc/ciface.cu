// The entry points in the shape cometpy calls kernels with.
//
// cometpy (COMET's numpy / scipy front end) compiles every kernel as a func.func with the
// llvm.emit_c_interface attribute and calls the symbol _mlir_ciface_<kernel> through ctypes
// (frontends/numpy-scipy/cometpy/MLIRGen/ops.py:548-553, lowering.py:373-427).  That convention is:
//   * results first: one POINTER per shaped result -- a memref struct for a dense result, one struct
//     holding the per-dimension memrefs for a sparse result (MLIRGen/utils.py:23-48: for CSR
//     {dims, insert_1, A1pos, insert_2, A2pos, A2crd, Aval}); the callee allocates the arrays with
//     malloc and fills in the descriptors, and cometpy wraps them WITHOUT a copy
//     (np.ctypeslib.as_array, lowering.py:433-448); a scalar result is the C return value;
//   * then the inputs, flattened: a dense ndarray is one POINTER to its memref struct; a scipy CSR
//     matrix is seven arguments -- dims*, insert_pos_1 (by value), A1pos*, insert_pos_2 (by value),
//     A2pos*, A2crd*, Aval* (lowering.py:298-321).
// The functions below have exactly that shape for CSR operands, so a kernel cometpy would generate
// for `A @ x`, `A @ B`, `A @ B` (sparse), `einsum(..., mask=M, semiring='+,pair').sum()` and the
// sampled product can be replaced by one of them symbol for symbol.  They forward to the host-memref
// entry points of layer 1.  Result arrays are malloc'ed; whoever wraps them owns them
// (comet_b200_ciface_free = free).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

using namespace cb200;

namespace {

typedef comet_b200_memref1d M1;
typedef comet_b200_memref2d M2;

// the sparse result struct of MLIRGen/utils.py:26-27 (identical for i32 indices: every member is a memref descriptor)
struct OutCsr {
    M1 dims;
    int64_t insert_1;
    M1 a1pos;
    int64_t insert_2;
    M1 a2pos;
    M1 a2crd;
    M1 aval;
};

struct Csr {   // one flattened CSR input
    M1 *dims, *a1pos, *a2pos, *a2crd, *aval;
};

void set1d(M1 *m, void *data, int64_t n)
{
    m->allocated = m->aligned = data;
    m->offset = 0;
    m->sizes[0] = n;
    m->strides[0] = 1;
}

void *zalloc(size_t bytes)
{
    void *p = calloc(bytes ? bytes : 8, 1);     // zeroed: an output's row pointer is read as "no entries yet" by layer 1
    if (!p) {
        fail("ciface: out of host memory (%zu bytes)", bytes);
        return nullptr;
    }
    return p;
}

M1 g_empty = {nullptr, nullptr, 0, {0}, {1}};

// the 24 arguments of COMET_B200_SPARSE2D for a CSR operand held as cometpy holds it
#define CSR_ARGS(c) 0, -1, 1, -1, 1, (void *)(c).a1pos, 1, (void *)&g_empty, 1, (void *)&g_empty, 1, (void *)&g_empty, 1, \
                    (void *)(c).a2pos, 1, (void *)(c).a2crd, 1, (void *)&g_empty, 1, (void *)&g_empty, 1, (void *)(c).aval, 1, \
                    (void *)(c).dims

int64_t rows_of(const Csr &c) { return ((int64_t *)c.dims->aligned)[c.dims->offset]; }
int64_t cols_of(const Csr &c) { return ((int64_t *)c.dims->aligned)[c.dims->offset + 1]; }

template <int ISZ>
void spmv(M1 *out, const Csr &A, M1 *x)
{
    const int64_t n = rows_of(A);
    double *y = (double *)zalloc((size_t)n * 8);
    if (!y) return;
    set1d(out, y, n);
    if (ISZ == 8) comet_b200_spmv_f64_i64(CSR_ARGS(A), 1, x, 1, out, COMET_B200_PLUS_TIMES, 0);
    else comet_b200_spmv_f64_i32(CSR_ARGS(A), 1, x, 1, out, COMET_B200_PLUS_TIMES, 0);
}

template <int ISZ>
void spmm(M2 *out, const Csr &A, M2 *B)
{
    const int64_t n = rows_of(A), k = B->sizes[1];
    double *c = (double *)zalloc((size_t)n * k * 8);
    if (!c) return;
    out->allocated = out->aligned = c;
    out->offset = 0;
    out->sizes[0] = n; out->sizes[1] = k;
    out->strides[0] = k; out->strides[1] = 1;
    if (ISZ == 8) comet_b200_spmm_f64_i64(CSR_ARGS(A), 2, B, 2, out, COMET_B200_PLUS_TIMES, 0);
    else comet_b200_spmm_f64_i32(CSR_ARGS(A), 2, B, 2, out, COMET_B200_PLUS_TIMES, 0);
}

// fills the result struct with freshly allocated CSR arrays of `rows` rows; the caller sets a2crd / aval later
template <int ISZ>
bool out_csr_begin(OutCsr *out, int64_t rows, int64_t cols)
{
    memset(out, 0, sizeof(*out));
    int64_t *dims = (int64_t *)zalloc(16);
    void *a1pos = zalloc(ISZ), *a2pos = zalloc((size_t)(rows + 1) * ISZ);
    if (!dims || !a1pos || !a2pos) return false;
    dims[0] = rows; dims[1] = cols;
    if (ISZ == 8) *(int64_t *)a1pos = rows; else *(int32_t *)a1pos = (int32_t)rows;
    set1d(&out->dims, dims, 2);
    set1d(&out->a1pos, a1pos, 1);
    set1d(&out->a2pos, a2pos, rows + 1);
    set1d(&out->a2crd, nullptr, 0);
    set1d(&out->aval, nullptr, 0);
    return true;
}

template <int ISZ>
void out_csr_finish(OutCsr *out, int64_t handle, int64_t nnz)
{
    if (!handle) return;
    void *crd = zalloc((size_t)nnz * ISZ);
    double *val = (double *)zalloc((size_t)nnz * 8);
    if (!crd || !val) { comet_b200_handle_destroy(handle); return; }
    set1d(&out->a2crd, crd, nnz);
    set1d(&out->aval, val, nnz);
    if (ISZ == 8) comet_b200_spgemm_numeric_f64_i64(handle, 1, &out->a2crd, 1, &out->aval);
    else comet_b200_spgemm_numeric_f64_i32(handle, 1, &out->a2crd, 1, &out->aval);
}

template <int ISZ>
void spgemm(OutCsr *out, const Csr &A, const Csr &B, const Csr *M, int64_t semiring)
{
    if (!out_csr_begin<ISZ>(out, rows_of(A), cols_of(B))) return;
    int64_t sizes[11] = {0};
    M1 sz;
    set1d(&sz, sizes, 11);
    const Csr &Mm = M ? *M : A;
    int64_t h;
    if (ISZ == 8)
        h = comet_b200_spgemm_symbolic_f64_i64(CSR_ARGS(A), CSR_ARGS(B), CSR_ARGS(Mm), M ? COMET_B200_MASK_PUSH : COMET_B200_MASK_NONE,
                                               (int32_t)semiring, 1, &out->a2pos, 1, &sz);
    else
        h = comet_b200_spgemm_symbolic_f64_i32(CSR_ARGS(A), CSR_ARGS(B), CSR_ARGS(Mm), M ? COMET_B200_MASK_PUSH : COMET_B200_MASK_NONE,
                                               (int32_t)semiring, 1, &out->a2pos, 1, &sz);
    out_csr_finish<ISZ>(out, h, sizes[8]);
}

template <int ISZ>
double masked_count(const Csr &A, const Csr &B, const Csr &M)
{
    int64_t count = 0;
    M1 o;
    set1d(&o, &count, 1);
    if (ISZ == 8)
        comet_b200_masked_spgemm_count_f64_i64(CSR_ARGS(A), CSR_ARGS(B), CSR_ARGS(M), COMET_B200_MASK_PUSH, COMET_B200_PLUS_PAIR, 1, &o);
    else
        comet_b200_masked_spgemm_count_f64_i32(CSR_ARGS(A), CSR_ARGS(B), CSR_ARGS(M), COMET_B200_MASK_PUSH, COMET_B200_PLUS_PAIR, 1, &o);
    return (double)count;      // COMET sums f64 values; the count is exact below 2^53
}

// O = S .* (X * Y^T): the result shares S's pattern, so its index arrays are copies of S's
template <int ISZ>
void sddmm(OutCsr *out, const Csr &S, M2 *X, M2 *Y)
{
    const int64_t rows = rows_of(S);
    if (!out_csr_begin<ISZ>(out, rows, cols_of(S))) return;
    const int64_t nnz = S.aval->sizes[0];
    void *crd = zalloc((size_t)nnz * ISZ);
    double *val = (double *)zalloc((size_t)nnz * 8);
    if (!crd || !val) return;
    set1d(&out->a2crd, crd, nnz);
    set1d(&out->aval, val, nnz);
    // Y is row-major [cols, K]: presented as the {K, cols} operand with strides {1, ld}
    M2 d = *Y;
    d.sizes[0] = Y->sizes[1]; d.sizes[1] = Y->sizes[0];
    d.strides[0] = Y->strides[1]; d.strides[1] = Y->strides[0];
    Csr O = {&out->dims, &out->a1pos, &out->a2pos, &out->a2crd, &out->aval};
    if (ISZ == 8) comet_b200_sddmm_f64_i64(CSR_ARGS(S), 2, X, 2, &d, CSR_ARGS(O));
    else comet_b200_sddmm_f64_i32(CSR_ARGS(S), 2, X, 2, &d, CSR_ARGS(O));
}

}  // namespace

#define CSR_PARAMS(P) comet_b200_memref1d *P##dims, int64_t P##ins1, comet_b200_memref1d *P##1pos, int64_t P##ins2, \
                      comet_b200_memref1d *P##2pos, comet_b200_memref1d *P##2crd, comet_b200_memref1d *P##val
#define CSR_PACK(P) Csr{P##dims, P##1pos, P##2pos, P##2crd, P##val}
#define IGNORE_INS(P) (void)P##ins1; (void)P##ins2

extern "C" {

#define CIFACE_WIDTH(SUFFIX, ISZ)                                                                                       \
    void _mlir_ciface_comet_b200_spmv_csr_f64_##SUFFIX(comet_b200_memref1d *y, CSR_PARAMS(A), comet_b200_memref1d *x)   \
    {                                                                                                                   \
        IGNORE_INS(A); clear_error(); spmv<ISZ>(y, CSR_PACK(A), x);                                                      \
    }                                                                                                                   \
    void _mlir_ciface_comet_b200_spmm_csr_f64_##SUFFIX(comet_b200_memref2d *C, CSR_PARAMS(A), comet_b200_memref2d *B)   \
    {                                                                                                                   \
        IGNORE_INS(A); clear_error(); spmm<ISZ>(C, CSR_PACK(A), B);                                                      \
    }                                                                                                                   \
    void _mlir_ciface_comet_b200_spgemm_csr_f64_##SUFFIX(void *C, CSR_PARAMS(A), CSR_PARAMS(B), int64_t semiring)       \
    {                                                                                                                   \
        IGNORE_INS(A); IGNORE_INS(B); clear_error(); spgemm<ISZ>((OutCsr *)C, CSR_PACK(A), CSR_PACK(B), nullptr, semiring); \
    }                                                                                                                   \
    void _mlir_ciface_comet_b200_spgemm_masked_csr_f64_##SUFFIX(void *C, CSR_PARAMS(A), CSR_PARAMS(B), CSR_PARAMS(M),   \
                                                                int64_t semiring)                                       \
    {                                                                                                                   \
        IGNORE_INS(A); IGNORE_INS(B); IGNORE_INS(M); clear_error();                                                      \
        Csr m = CSR_PACK(M);                                                                                            \
        spgemm<ISZ>((OutCsr *)C, CSR_PACK(A), CSR_PACK(B), &m, semiring);                                                \
    }                                                                                                                   \
    double _mlir_ciface_comet_b200_masked_count_csr_f64_##SUFFIX(CSR_PARAMS(A), CSR_PARAMS(B), CSR_PARAMS(M))           \
    {                                                                                                                   \
        IGNORE_INS(A); IGNORE_INS(B); IGNORE_INS(M); clear_error();                                                      \
        return masked_count<ISZ>(CSR_PACK(A), CSR_PACK(B), CSR_PACK(M));                                                 \
    }                                                                                                                   \
    void _mlir_ciface_comet_b200_sddmm_csr_f64_##SUFFIX(void *O, CSR_PARAMS(S), comet_b200_memref2d *X,                 \
                                                        comet_b200_memref2d *Y)                                         \
    {                                                                                                                   \
        IGNORE_INS(S); clear_error(); sddmm<ISZ>((OutCsr *)O, CSR_PACK(S), X, Y);                                        \
    }

CIFACE_WIDTH(i64, 8)
CIFACE_WIDTH(i32, 4)

void comet_b200_ciface_free(void *p) { free(p); }

}
