/*
 * comet_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A CPU restatement, in plain C, of the loop nests that the COMET compiler
 * generates for ta.mul / ta.elews_mul on CSR / DCSR / COO operands, and of the
 * MatrixMarket reader of COMET's runtime.  It exists only so that the CUDA
 * path can be checked against it (tests, the smoke check, and the CPU
 * baseline leg of the benchmark).  Nothing in the shipped library may call it.
 *
 * Parity status: PINNED against the reference's own golden outputs (the
 * CHECK lines of its integration tests, stored under tests/golden/), because
 * the reference compiler cannot be built without LLVM/MLIR.  The golden
 * outputs carry six significant digits, so they pin semantics and structure;
 * large inputs are checked oracle-vs-GPU.
 *
 * Arithmetic rules restated from the reference (paths are relative to the
 * COMET source tree):
 *   - combine then reduce as two separate IEEE operations, never fused
 *     (lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:198-361, 1247-1284);
 *     compile this file with -ffp-contract=off.
 *   - "times" combine = a*b, "pairxy" combine = 1.0 (same file :290-293);
 *     "plusxy" reduce = old + v, "noop" reduce = v (:307-361).
 *   - dense outputs are read-modify-written: C = C_old + sum (:1266-1278).
 *   - index iteration order follows first appearance of the labels:
 *     a -> b -> c for C[a,c] = A[a,b] * B[b,c]
 *     (lib/Conversion/TensorAlgebraToIndexTree/TensorAlgebraToIndexTree.cpp:316-323).
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* Single-precision build (-DORACLE_F32 -> libcomet_oracle_f32.so): COMET generates the same loops for
   Tensor<float>, with f32 mulf / addf.  Every `double` from here on becomes float, so the arithmetic below
   is done in single precision in the same order; the system headers above keep their own double. */
#ifdef ORACLE_F32
#define double float
#endif

/* semiring codes shared with include/comet_b200.h */
enum { SEMIRING_PLUS_TIMES = 0, SEMIRING_PLUS_PAIR = 1, SEMIRING_PLUS_FIRST = 2, SEMIRING_PLUS_SECOND = 3,
       SEMIRING_MIN_PLUS = 4, SEMIRING_MIN_FIRST = 5, SEMIRING_MIN_SECOND = 6, SEMIRING_ANY_PAIR = 7 };

/* readMode values of comet_read(id, mode): lib/ExecutionEngine/SparseUtils.cpp:50-64 */
enum { READ_DEFAULT = 1, READ_LOWER_TRI_STRICT = 2, READ_LOWER_TRI = 3,
       READ_UPPER_TRI_STRICT = 4, READ_UPPER_TRI = 5 };

ORACLE_API int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oracle_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* MatrixMarket reader: SparseUtils.cpp:145-356 (CooMatrix::InitMarket)       */
/* ------------------------------------------------------------------------- */

typedef struct {
    int64_t nrows, ncols, nnz;
    int64_t nnz_lower, nnz_upper, nnz_lower_strict, nnz_upper_strict;
    int64_t *row, *col;
    double *val;
} coo_t;

static void coo_count(coo_t *m, int64_t r, int64_t c)
{
    /* triangle counters are updated for the entry as written in the file only,
       not for its mirrored twin (SparseUtils.cpp:315-330) */
    if (r > c) { m->nnz_lower_strict++; m->nnz_lower++; }
    else if (r < c) { m->nnz_upper_strict++; m->nnz_upper++; }
    else { m->nnz_lower++; m->nnz_upper++; }
}

static int coo_read_market(const char *path, coo_t *m)
{
    FILE *f = fopen(path, "r");
    if (!f) return -1;
    memset(m, 0, sizeof(*m));
    int array = 0, symmetric = 0, skew = 0, header_done = 0;
    int64_t cur = 0, cap = 0;
    char line[1024];
    while (fgets(line, sizeof(line), f)) {
        if (line[0] == '%') {
            if (line[1] == '%') {
                symmetric = strstr(line, "symmetric") != NULL;
                skew = strstr(line, "skew") != NULL;
                array = strstr(line, "array") != NULL;
            }
            continue;
        }
        if (!header_done) {
            long long a = 0, b = 0, c = 0;
            int n = sscanf(line, "%lld %lld %lld", &a, &b, &c);
            if (!array && n == 3) { m->nrows = a; m->ncols = b; cap = symmetric ? 2 * c : c; }
            else if (array && n == 2) { m->nrows = a; m->ncols = b; cap = a * b; }
            else { fclose(f); return -2; }
            m->row = (int64_t *)malloc(sizeof(int64_t) * (cap ? cap : 1));
            m->col = (int64_t *)malloc(sizeof(int64_t) * (cap ? cap : 1));
            m->val = (double *)malloc(sizeof(double) * (cap ? cap : 1));
            header_done = 1;
            continue;
        }
        /* a blank trailing line ends the stream for the reference too */
        {
            const char *s = line;
            while (*s == ' ' || *s == '\t' || *s == '\r' || *s == '\n') s++;
            if (*s == 0) continue;
        }
        if (cur >= cap) { fclose(f); return -3; }
        int64_t r, c;
        double v;
        if (array) {
            v = strtod(line, NULL);
            c = cur / m->nrows;
            r = cur - m->nrows * c;
        } else {
            char *l = line, *t = NULL;
            r = strtol(l, &t, 0); if (t == l) { fclose(f); return -4; } l = t;
            c = strtol(l, &t, 0); if (t == l) { fclose(f); return -4; } l = t;
            v = strtod(l, &t);
            if (t == l) v = 1.0;          /* pattern files: default value 1.0 */
            r -= 1; c -= 1;               /* 1-based -> 0-based */
        }
        m->row[cur] = r; m->col[cur] = c; m->val[cur] = v;
        coo_count(m, r, c);
        cur++;
        if (symmetric && r != c) {
            m->row[cur] = c; m->col[cur] = r; m->val[cur] = skew ? -v : v;
            cur++;
        }
    }
    fclose(f);
    m->nnz = cur;
    if (symmetric) {
        m->nnz_upper = m->nnz_lower;
        m->nnz_upper_strict = m->nnz_lower_strict;
    }
    return 0;
}

/* stable merge sort of a permutation by (row, col): the reference uses
   std::stable_sort with CooComparatorRow (SparseUtils.cpp:360-367, 424) so
   duplicate coordinates keep their file order and are NOT summed. */
static void sort_perm_row_col(int64_t n, const int64_t *row, const int64_t *col, int64_t *perm)
{
    int64_t *tmp = (int64_t *)malloc(sizeof(int64_t) * (n ? n : 1));
    for (int64_t i = 0; i < n; i++) perm[i] = i;
    for (int64_t w = 1; w < n; w *= 2) {
        for (int64_t lo = 0; lo < n; lo += 2 * w) {
            int64_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            int64_t i = lo, j = mid, k = lo;
            while (i < mid && j < hi) {
                int64_t a = perm[i], b = perm[j];
                int b_less = (row[b] < row[a]) || (row[b] == row[a] && col[b] < col[a]);
                tmp[k++] = b_less ? perm[j++] : perm[i++];
            }
            while (i < mid) tmp[k++] = perm[i++];
            while (j < hi) tmp[k++] = perm[j++];
        }
        memcpy(perm, tmp, sizeof(int64_t) * n);
    }
    free(tmp);
}

static int keep_entry(int mode, int64_t r, int64_t c)
{
    /* filters of CsrMatrix::Init (SparseUtils.cpp:462-520) and of the COO
       fill loop (:1859-1893) */
    switch (mode) {
    case READ_LOWER_TRI_STRICT: return r > c;
    case READ_LOWER_TRI: return r >= c;
    case READ_UPPER_TRI_STRICT: return r < c;
    case READ_UPPER_TRI: return r <= c;
    default: return 1;
    }
}

static int64_t mode_nnz(const coo_t *m, int mode)
{
    switch (mode) {   /* getNumNonZeros, SparseUtils.cpp:1606-1624 */
    case READ_LOWER_TRI_STRICT: return m->nnz_lower_strict;
    case READ_LOWER_TRI: return m->nnz_lower;
    case READ_UPPER_TRI_STRICT: return m->nnz_upper_strict;
    case READ_UPPER_TRI: return m->nnz_upper;
    default: return m->nnz;
    }
}

/* One reader handle = one parsed file, like the reference's cached
   FileReaderWrapper (SparseUtils.cpp:1434-1602). */
typedef struct { coo_t coo; int64_t *perm; } reader_t;

ORACLE_API void *oracle_reader_open(const char *path)
{
    reader_t *r = (reader_t *)calloc(1, sizeof(reader_t));
    if (coo_read_market(path, &r->coo) != 0) { free(r); return NULL; }
    r->perm = (int64_t *)malloc(sizeof(int64_t) * (r->coo.nnz ? r->coo.nnz : 1));
    sort_perm_row_col(r->coo.nnz, r->coo.row, r->coo.col, r->perm);
    return r;
}

ORACLE_API void oracle_reader_close(void *h)
{
    reader_t *r = (reader_t *)h;
    if (!r) return;
    free(r->coo.row); free(r->coo.col); free(r->coo.val); free(r->perm); free(r);
}

/* Format codes of the runtime (include/comet/ExecutionEngine/RunnerUtils.h:71-77):
   Dense=0, Compressed_unique=1, Compressed_nonunique=2, singleton=3.
   sizes[11] as read_input_sizes_2D fills it (SparseUtils.cpp:1643-1751):
   A1pos, A1crd, A1tile_pos, A1tile_crd, A2pos, A2crd, A2tile_pos, A2tile_crd,
   nnz, nrows, ncols. */
ORACLE_API int oracle_reader_sizes(void *h, int a1fmt, int a2fmt, int mode, int64_t *sizes)
{
    reader_t *r = (reader_t *)h;
    const coo_t *m = &r->coo;
    int64_t nnz = mode_nnz(m, mode);
    memset(sizes, 0, sizeof(int64_t) * 11);
    sizes[9] = m->nrows; sizes[10] = m->ncols;
    if (a1fmt == 2 && a2fmt == 3) {            /* COO */
        sizes[0] = 2; sizes[1] = nnz; sizes[4] = 1; sizes[5] = nnz; sizes[8] = nnz;
    } else if (a1fmt == 0 && a2fmt == 1) {     /* CSR */
        sizes[0] = 1; sizes[1] = 1; sizes[4] = m->nrows + 1; sizes[5] = nnz; sizes[8] = nnz;
    } else if (a1fmt == 1 && a2fmt == 1) {     /* DCSR: DcsrMatrix::Init :686-735 */
        int64_t nr = 0, prev = -1;
        for (int64_t i = 0; i < m->nnz; i++) {
            int64_t row = m->row[r->perm[i]];
            if (row != prev) { nr++; prev = row; }
        }
        sizes[0] = 2; sizes[1] = nr; sizes[4] = nr + 1; sizes[5] = m->nnz; sizes[8] = m->nnz;
    } else {
        return -1;
    }
    return 0;
}

/* Fill caller-allocated arrays like read_input_2D (SparseUtils.cpp:1813-2078). */
ORACLE_API int oracle_reader_fill(void *h, int a1fmt, int a2fmt, int mode,
                                  int64_t *a1pos, int64_t *a1crd, int64_t *a2pos, int64_t *a2crd,
                                  double *aval)
{
    reader_t *r = (reader_t *)h;
    const coo_t *m = &r->coo;
    a1pos[0] = -1; a1crd[0] = -1; a2pos[0] = -1;
    if (a1fmt == 2 && a2fmt == 3) {            /* COO :1853-1898 */
        int64_t n = 0;
        a1pos[0] = 0;
        for (int64_t i = 0; i < m->nnz; i++) {
            int64_t e = r->perm[i];
            if (!keep_entry(mode, m->row[e], m->col[e])) continue;
            a1crd[n] = m->row[e]; a2crd[n] = m->col[e]; aval[n] = m->val[e]; n++;
        }
        a1pos[1] = n;
    } else if (a1fmt == 0 && a2fmt == 1) {     /* CSR :404-533, :1900-1941 */
        int64_t total = mode_nnz(m, mode), cur = 0, prev_row = -1;
        for (int64_t i = 0; i < m->nnz; i++) {
            int64_t e = r->perm[i];
            int64_t row = m->row[e], col = m->col[e];
            if (!keep_entry(mode, row, col)) continue;
            for (int64_t q = prev_row + 1; q <= row; q++) a2pos[q] = cur;
            prev_row = row;
            a2crd[cur] = col; aval[cur] = m->val[e]; cur++;
        }
        for (int64_t q = prev_row + 1; q <= m->nrows; q++) a2pos[q] = total;
        a1pos[0] = m->nrows;
    } else if (a1fmt == 1 && a2fmt == 1) {     /* DCSR :686-735 */
        int64_t nr = 0, prev = -1;
        for (int64_t i = 0; i < m->nnz; i++) {
            int64_t e = r->perm[i];
            if (m->row[e] != prev) { a2pos[nr] = i; a1crd[nr] = m->row[e]; nr++; prev = m->row[e]; }
            a2crd[i] = m->col[e]; aval[i] = m->val[e];
        }
        a2pos[nr] = m->nnz;
        a1pos[0] = 0; a1pos[1] = nr;
    } else {
        return -1;
    }
    return 0;
}

/* ------------------------------------------------------------------------- */
/* Dense-output products.  Row loop parallel like scf.forall -> OpenMP        */
/* (TensorAlgebraToIndexTree.cpp:276-323, frontends/comet_dsl/comet.cpp:718); */
/* inner sparse loops sequential in position order (IndexTreeToSCF.cpp:667-700)*/
/* ------------------------------------------------------------------------- */

/* second operator of the semiring (getSemiringSecondVal, IndexTreeToSCF.cpp:198-305) */
static inline double combine(int semiring, double a, double b)
{
    switch (semiring) {
    case SEMIRING_PLUS_PAIR: case SEMIRING_ANY_PAIR: return 1.0;
    case SEMIRING_PLUS_FIRST: case SEMIRING_MIN_FIRST: return a;
    case SEMIRING_PLUS_SECOND: case SEMIRING_MIN_SECOND: return b;
    case SEMIRING_MIN_PLUS: return a + b;
    default: return a * b;
    }
}

/* first operator (getSemiringFirstVal, :307-361): plusxy adds, minxy is select(old < v, old, v),
   any takes the new value */
static inline double reduce(int semiring, double old, double v)
{
    switch (semiring) {
    case SEMIRING_MIN_PLUS: case SEMIRING_MIN_FIRST: case SEMIRING_MIN_SECOND: return old < v ? old : v;
    case SEMIRING_ANY_PAIR: return v;
    default: return old + v;
    }
}

ORACLE_API void oracle_spmv_csr(int64_t nrows, const int64_t *pos, const int64_t *crd,
                                const double *val, const double *x, double *y, int semiring)
{
#pragma omp parallel for schedule(static)
    for (int64_t a = 0; a < nrows; a++) {
        double acc = y[a];
        for (int64_t p = pos[a]; p < pos[a + 1]; p++) {
            double v = combine(semiring, val[p], x[crd[p]]);
            acc = acc + v;
        }
        y[a] = acc;
    }
}

/* DCSR: both dims compressed -> two sparse loops, sequential, only stored rows
   visited (IndexTreeToSCF.cpp:667-700). */
ORACLE_API void oracle_spmv_dcsr(const int64_t *a1pos, const int64_t *a1crd, const int64_t *a2pos,
                                 const int64_t *a2crd, const double *val, const double *x, double *y,
                                 int semiring)
{
    for (int64_t r = a1pos[0]; r < a1pos[1]; r++) {
        int64_t a = a1crd[r];
        for (int64_t p = a2pos[r]; p < a2pos[r + 1]; p++)
            y[a] = y[a] + combine(semiring, val[p], x[a2crd[p]]);
    }
}

/* COO: one loop over positions; dim 1 is a singleton sharing the position
   (IndexTreeToSCF.cpp:736-783). */
ORACLE_API void oracle_spmv_coo(const int64_t *a1pos, const int64_t *a1crd, const int64_t *a2crd,
                                const double *val, const double *x, double *y, int semiring)
{
    for (int64_t p = a1pos[0]; p < a1pos[1]; p++)
        y[a1crd[p]] = y[a1crd[p]] + combine(semiring, val[p], x[a2crd[p]]);
}

ORACLE_API void oracle_spmm_csr(int64_t nrows, int64_t k, const int64_t *pos, const int64_t *crd,
                                const double *val, const double *b, int64_t ldb, double *c,
                                int64_t ldc, int semiring)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t a = 0; a < nrows; a++) {
        double *crow = c + a * ldc;
        for (int64_t p = pos[a]; p < pos[a + 1]; p++) {
            const double *brow = b + crd[p] * ldb;
            double av = val[p];
            for (int64_t j = 0; j < k; j++)
                crow[j] = crow[j] + combine(semiring, av, brow[j]);
        }
    }
}

ORACLE_API void oracle_spmm_dcsr(int64_t k, const int64_t *a1pos, const int64_t *a1crd,
                                 const int64_t *a2pos, const int64_t *a2crd, const double *val,
                                 const double *b, int64_t ldb, double *c, int64_t ldc, int semiring)
{
    for (int64_t r = a1pos[0]; r < a1pos[1]; r++) {
        double *crow = c + a1crd[r] * ldc;
        for (int64_t p = a2pos[r]; p < a2pos[r + 1]; p++) {
            const double *brow = b + a2crd[p] * ldb;
            for (int64_t j = 0; j < k; j++)
                crow[j] = crow[j] + combine(semiring, val[p], brow[j]);
        }
    }
}

ORACLE_API void oracle_spmm_coo(int64_t k, const int64_t *a1pos, const int64_t *a1crd,
                                const int64_t *a2crd, const double *val, const double *b,
                                int64_t ldb, double *c, int64_t ldc, int semiring)
{
    for (int64_t p = a1pos[0]; p < a1pos[1]; p++) {
        double *crow = c + a1crd[p] * ldc;
        const double *brow = b + a2crd[p] * ldb;
        for (int64_t j = 0; j < k; j++)
            crow[j] = crow[j] + combine(semiring, val[p], brow[j]);
    }
}

/* Dense x sparse: C[a,c] = C[a,c] + A[a,b] * B[b,c] with A dense (m rows; m = 1 for a vector) and B
   sparse; loops a -> b -> c in label order, a parallel, b over the rows B stores, c over the row's
   entries (test/integration/ops/mult_Dense{Mat,Vec}x{CSR,DCSR,COO}.ta).  `rows` (DCSR row
   coordinates) may be NULL; for COO pass nstored = nnz, rows = row coordinates, pos = NULL. */
ORACLE_API void oracle_dense_times_sparse(int64_t m, int64_t nstored, const int64_t *rows,
                                          const int64_t *pos, const int64_t *crd, const double *val,
                                          const double *a, int64_t lda, double *c, int64_t ldc, int semiring)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; i++) {
        for (int64_t r = 0; r < nstored; r++) {
            int64_t b = rows ? rows[r] : r;
            int64_t s = pos ? pos[r] : r, e = pos ? pos[r + 1] : r + 1;
            double av = a[i * lda + b];
            for (int64_t p = s; p < e; p++)
                c[i * ldc + crd[p]] = c[i * ldc + crd[p]] + combine(semiring, av, val[p]);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* SDDMM: out.val[p] = S.val[p] * sum_k X[i,k] * Y[j,k], k ascending, the sum  */
/* starting from T = 0.0 (test/integration/kernels/sddmm.ta:24-30).  The       */
/* reference's fused loop computes the whole dense row T[i,:] first; only the  */
/* sampled entries are observable, and each of them is this same k-ordered sum */
/* so the O(nnz*K) form below gives identical values.  Y is addressed through  */
/* two strides so both D[k,j] (ys_k = ld, ys_j = 1) and row-major Y[j,k]       */
/* (ys_k = 1, ys_j = ld) are covered.                                          */
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_sddmm_csr(int64_t nrows, int64_t k, const int64_t *pos, const int64_t *crd,
                                 const double *sval, const double *x, int64_t ldx, const double *y,
                                 int64_t ys_k, int64_t ys_j, double *out)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t i = 0; i < nrows; i++) {
        const double *xr = x + i * ldx;
        for (int64_t p = pos[i]; p < pos[i + 1]; p++) {
            const double *yc = y + crd[p] * ys_j;
            double t = 0.0;
            for (int64_t kk = 0; kk < k; kk++) {
                double v = xr[kk] * yc[kk * ys_k];
                t = t + v;
            }
            out[p] = sval[p] * t;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Elementwise multiply (ta.elews_mul, semiring noop_times).                   */
/* sparse x dense -> sparse keeps the sparse operand's pos/crd                 */
/* (lib/Conversion/IndexTreeToSCF/SymbolicDomainConversion.cpp:277-297).       */
/* ------------------------------------------------------------------------- */
ORACLE_API void oracle_elews_csr_dense(int64_t nrows, const int64_t *pos, const int64_t *crd,
                                       const double *val, const double *b, int64_t ldb, double *out)
{
    for (int64_t a = 0; a < nrows; a++)
        for (int64_t p = pos[a]; p < pos[a + 1]; p++)
            out[p] = val[p] * b[a * ldb + crd[p]];
}

ORACLE_API void oracle_elews_coo_dense(int64_t nnz, const int64_t *rows, const int64_t *cols,
                                       const double *val, const double *b, int64_t ldb, double *out)
{
    for (int64_t p = 0; p < nnz; p++)
        out[p] = val[p] * b[rows[p] * ldb + cols[p]];
}

/* sparse .* sparse: two-pointer intersection of both rows
   (IndexTreeToSCF.cpp:854-1073); symbolic count first, then fill.
   Pass cpos only (ccrd = cval = NULL) for the symbolic phase. */
ORACLE_API int64_t oracle_elews_csr_csr(int64_t nrows, const int64_t *apos, const int64_t *acrd,
                                        const double *aval, const int64_t *bpos, const int64_t *bcrd,
                                        const double *bval, int64_t *cpos, int64_t *ccrd, double *cval)
{
    int64_t n = 0;
    cpos[0] = 0;
    for (int64_t i = 0; i < nrows; i++) {
        int64_t p = apos[i], q = bpos[i];
        while (p < apos[i + 1] && q < bpos[i + 1]) {
            int64_t ca = acrd[p], cb = bcrd[q];
            if (ca == cb) {
                if (ccrd) { ccrd[n] = ca; cval[n] = aval[p] * bval[q]; }
                n++;
            }
            /* advance whichever side holds the smaller (or equal) coordinate */
            if (ca <= cb) p++;
            if (cb <= ca) q++;
        }
        cpos[i + 1] = n;
    }
    return n;
}

/* ------------------------------------------------------------------------- */
/* Gustavson SpGEMM with workspace, optional push mask.                       */
/* symbolic: SymbolicDomainConversion.cpp:81-210 (mark[j] = row + 1)           */
/* numeric : lib/Conversion/TensorAlgebraToSCF/SparseTensorConversionPass.cpp  */
/*           :1029-1112 (first touch stores the product, later touches add),   */
/*           crd list sorted by comet_sort64 = std::sort                       */
/*           (IndexTreeToSCF.cpp:796-852, SparseUtils.cpp:2600-2626), then     */
/*           copied out in sorted order.                                       */
/* mask    : bits of M row i set before the row, tested for every product,     */
/*           cleared after (IndexTreeToSCF.cpp:1075-1162, 1327-1448).          */
/* ------------------------------------------------------------------------- */
static int cmp_i64(const void *a, const void *b)
{
    int64_t x = *(const int64_t *)a, y = *(const int64_t *)b;
    return (x > y) - (x < y);
}

ORACLE_API int64_t oracle_spgemm_symbolic(int64_t nrows, int64_t ncols, const int64_t *apos,
                                          const int64_t *acrd, const int64_t *bpos,
                                          const int64_t *bcrd, const int64_t *mpos,
                                          const int64_t *mcrd, int64_t *cpos)
{
    int64_t *mark = (int64_t *)calloc((size_t)(ncols ? ncols : 1), sizeof(int64_t));
    unsigned char *mask = mpos ? (unsigned char *)calloc((size_t)(ncols ? ncols : 1), 1) : NULL;
    int64_t nnz = 0;
    cpos[0] = 0;
    for (int64_t i = 0; i < nrows; i++) {
        if (mask) for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 1;
        for (int64_t p = apos[i]; p < apos[i + 1]; p++) {
            int64_t k = acrd[p];
            for (int64_t q = bpos[k]; q < bpos[k + 1]; q++) {
                int64_t j = bcrd[q];
                if (mask && !mask[j]) continue;
                if (mark[j] != i + 1) { mark[j] = i + 1; nnz++; }
            }
        }
        if (mask) for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 0;
        cpos[i + 1] = nnz;
    }
    free(mark); free(mask);
    return nnz;
}

ORACLE_API void oracle_spgemm_numeric(int64_t nrows, int64_t ncols, const int64_t *apos,
                                      const int64_t *acrd, const double *aval, const int64_t *bpos,
                                      const int64_t *bcrd, const double *bval, const int64_t *mpos,
                                      const int64_t *mcrd, int semiring, const int64_t *cpos,
                                      int64_t *ccrd, double *cval)
{
    size_t nc = (size_t)(ncols ? ncols : 1);
    double *ws = (double *)calloc(nc, sizeof(double));
    int32_t *mark = (int32_t *)calloc(nc, sizeof(int32_t));
    int64_t *list = (int64_t *)malloc(nc * sizeof(int64_t));
    unsigned char *mask = mpos ? (unsigned char *)calloc(nc, 1) : NULL;
    int32_t mark_value = 0;
    for (int64_t i = 0; i < nrows; i++) {
        int64_t num = 0;
        mark_value++;
        if (mask) for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 1;
        for (int64_t p = apos[i]; p < apos[i + 1]; p++) {
            int64_t k = acrd[p];
            double av = aval[p];
            for (int64_t q = bpos[k]; q < bpos[k + 1]; q++) {
                int64_t j = bcrd[q];
                if (mask && !mask[j]) continue;
                double v = combine(semiring, av, bval[q]);
                if (mark[j] == mark_value) ws[j] = reduce(semiring, ws[j], v);
                else { mark[j] = mark_value; list[num++] = j; ws[j] = v; }
            }
        }
        if (mask) for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 0;
        qsort(list, (size_t)num, sizeof(int64_t), cmp_i64);
        int64_t ins = cpos[i];
        for (int64_t t = 0; t < num; t++) { ccrd[ins] = list[t]; cval[ins] = ws[list[t]]; ins++; }
    }
    free(ws); free(mark); free(list); free(mask);
}

/* ta.reduce on a sparse tensor: sequential sum over vals
   (lib/Conversion/TensorAlgebraToSCF/TensorAlgebraToSCF.cpp:483-517). */
ORACLE_API double oracle_reduce_sum(int64_t n, const double *vals)
{
    double s = 0.0;
    for (int64_t i = 0; i < n; i++) s = s + vals[i];
    return s;
}

/* SUM(C<M,push> = A*B) under plus-pair for the row range [row_lo, row_hi),
   without storing C: every product that passes the mask contributes 1.0 to
   some stored value, and the final SUM adds all stored values, so the total
   is the number of passing products.  Exact in int64.  Used for triangle
   counting (test/integration/kernels/triangleCount_SandiaLL_wMasking.ta) and,
   over a row range, as the bounded CPU-baseline sample. */
ORACLE_API int64_t oracle_masked_pair_count(int64_t row_lo, int64_t row_hi, int64_t ncols,
                                            const int64_t *apos, const int64_t *acrd,
                                            const int64_t *bpos, const int64_t *bcrd,
                                            const int64_t *mpos, const int64_t *mcrd)
{
    unsigned char *mask = (unsigned char *)calloc((size_t)(ncols ? ncols : 1), 1);
    int64_t count = 0;
    for (int64_t i = row_lo; i < row_hi; i++) {
        for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 1;
        for (int64_t p = apos[i]; p < apos[i + 1]; p++) {
            int64_t k = acrd[p];
            for (int64_t q = bpos[k]; q < bpos[k + 1]; q++)
                count += mask[bcrd[q]];
        }
        for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 0;
    }
    free(mask);
    return count;
}

/* ------------------------------------------------------------------------- */
/* Row-parallel variants of the two sparse-output paths.  NOT COMET's          */
/* schedule: COMET emits sequential loops whenever the output is sparse        */
/* (lib/Conversion/TensorAlgebraToIndexTree/TensorAlgebraToIndexTree.cpp       */
/* :279-282), so its own CPU time is the single-thread functions above.  These */
/* exist only so that the benchmark can also print what the host's cores can   */
/* do with the same algorithm once rows are handed to threads, each with its   */
/* own workspace (two passes: counts, then prefix sum, then fill).  Results    */
/* are identical to the sequential functions.                                  */
/* ------------------------------------------------------------------------- */
ORACLE_API int64_t oracle_spgemm_rowparallel(int64_t nrows, int64_t ncols, const int64_t *apos,
                                             const int64_t *acrd, const double *aval,
                                             const int64_t *bpos, const int64_t *bcrd, const double *bval,
                                             int semiring, int64_t *cpos, int64_t *ccrd, double *cval)
{
    /* pass 1 (ccrd == NULL): per-row counts into cpos[i+1]; pass 2: fill, cpos already scanned */
    size_t nc = (size_t)(ncols ? ncols : 1);
#pragma omp parallel
    {
        int64_t *mark = (int64_t *)calloc(nc, sizeof(int64_t));
        double *ws = ccrd ? (double *)calloc(nc, sizeof(double)) : NULL;
        int64_t *list = ccrd ? (int64_t *)malloc(nc * sizeof(int64_t)) : NULL;
#pragma omp for schedule(dynamic, 16)
        for (int64_t i = 0; i < nrows; i++) {
            int64_t num = 0;
            for (int64_t p = apos[i]; p < apos[i + 1]; p++) {
                int64_t k = acrd[p];
                double av = aval[p];
                for (int64_t q = bpos[k]; q < bpos[k + 1]; q++) {
                    int64_t j = bcrd[q];
                    if (!ccrd) {
                        if (mark[j] != i + 1) { mark[j] = i + 1; num++; }
                    } else {
                        double v = combine(semiring, av, bval[q]);
                        if (mark[j] == i + 1) ws[j] = reduce(semiring, ws[j], v);
                        else { mark[j] = i + 1; list[num++] = j; ws[j] = v; }
                    }
                }
            }
            if (!ccrd) cpos[i + 1] = num;
            else {
                qsort(list, (size_t)num, sizeof(int64_t), cmp_i64);
                int64_t ins = cpos[i];
                for (int64_t t = 0; t < num; t++) { ccrd[ins] = list[t]; cval[ins] = ws[list[t]]; ins++; }
            }
        }
        free(mark); free(ws); free(list);
    }
    if (!ccrd) {
        cpos[0] = 0;
        for (int64_t i = 0; i < nrows; i++) cpos[i + 1] += cpos[i];
    }
    return cpos[nrows];
}

ORACLE_API int64_t oracle_masked_pair_count_rowparallel(int64_t row_lo, int64_t row_hi, int64_t ncols,
                                                        const int64_t *apos, const int64_t *acrd,
                                                        const int64_t *bpos, const int64_t *bcrd,
                                                        const int64_t *mpos, const int64_t *mcrd)
{
    int64_t count = 0;
#pragma omp parallel reduction(+ : count)
    {
        unsigned char *mask = (unsigned char *)calloc((size_t)(ncols ? ncols : 1), 1);
#pragma omp for schedule(dynamic, 64)
        for (int64_t i = row_lo; i < row_hi; i++) {
            for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 1;
            for (int64_t p = apos[i]; p < apos[i + 1]; p++) {
                int64_t k = acrd[p];
                for (int64_t q = bpos[k]; q < bpos[k + 1]; q++) count += mask[bcrd[q]];
            }
            for (int64_t t = mpos[i]; t < mpos[i + 1]; t++) mask[mcrd[t]] = 0;
        }
        free(mask);
    }
    return count;
}
