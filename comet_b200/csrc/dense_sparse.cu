// Dense x sparse  C[a,c] = C[a,c] (+) sum_b A[a,b] (x) B[b,c]  with A dense
// (m rows; m = 1 is the vector form) and B sparse (CSR / DCSR rows, COO through
// the row-pointer adapter), C dense.
//
// One warp owns a row b of B and a tile of rows of A: its lanes hold the row's
// (column, value) entries, and for every a of the tile the warp adds
// A[a,b] * value to C[a, column] with f64 atomics (different rows of B name the
// same columns, so the additions of different warps meet in C).  C is cleared
// first when the caller does not accumulate.
//
// Bound: HBM for large m (C is read-modify-written once per stored entry and
// row of A); this form is outside the five benchmark configurations.
//
// From DS_SPMM_MIN rows of A on, with B in plain CSR, the product is computed transposed instead:
// C^T = B^T A^T is an SpMM with the sparse operand on the left, so B is transposed once
// (counting sort of its entries by column), A and the result are transposed through shared memory,
// and the entry-stream / row-panel SpMM kernels do the arithmetic without one atomic per product.  The
// terms of every C[a,c] are added in ascending b, as the reference's loop nest does.
#include "common.cuh"

namespace cb200 {

static const int DS_THREADS = 256;
static const int DS_TILE = 8;      // rows of A per warp pass
static const int64_t DS_SPMM_MIN = 32;   // rows of A from which the transposed SpMM form is used (measured crossover,
                                         // R-MAT scale 18: 16 rows 1.60 against 0.90 ms, 64 rows 1.37 against 2.56 ms)

__global__ void __launch_bounds__(DS_THREADS)
dense_times_sparse_kernel(int64_t m, int64_t nstored, const int64_t *__restrict__ row_ids,
                          const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                          const double *__restrict__ val, const double *__restrict__ a, int64_t lda,
                          double *__restrict__ c, int64_t ldc, int pair)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * DS_THREADS + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * DS_THREADS) >> 5;
    const int64_t tiles = (m + DS_TILE - 1) / DS_TILE;
    for (int64_t item = warp; item < nstored * tiles; item += nwarps) {
        const int64_t r = item / tiles;
        const int64_t a0 = (item % tiles) * DS_TILE;
        const int64_t a1 = a0 + DS_TILE < m ? a0 + DS_TILE : m;
        const int64_t b = row_ids ? row_ids[r] : r;
        const int64_t s = pos[r], e = pos[r + 1];
        for (int64_t p = s + lane; p < e; p += 32) {
            const int64_t col = ld_stream(crd + p);
            const double v = pair ? 1.0 : ld_stream(val + p);
            for (int64_t i = a0; i < a1; i++) {
                const double av = pair ? 1.0 : __ldg(a + i * lda + b);
                atomicAdd(c + i * ldc + col, av * v);
            }
        }
    }
}

// C (m x p) = [C +] A (m x n) * B (n x p, CSR) through C^T = B^T A^T.
static int dense_times_sparse_transposed(int64_t m, int64_t p, int64_t n, int64_t nnz, const int64_t *pos,
                                         const int64_t *crd, const double *val, const double *a, int64_t lda,
                                         double *c, int64_t ldc, int semiring, int accumulate, cudaStream_t st)
{
    const int64_t mp = (m + 1) & ~(int64_t)1;          // even width: the SpMM kernels move 16-byte vectors
    int64_t *tpos = nullptr, *tcrd = nullptr;
    double *tval = nullptr, *at = nullptr, *ct = nullptr;
    int rc = 0;
    auto get = [&](void **ptr, size_t bytes) {
        if (!rc && cudaMallocAsync(ptr, bytes ? bytes : 8, st) != cudaSuccess) rc = fail("dense x sparse: allocation failed");
    };
    get((void **)&tpos, (size_t)(p + 1) * 8);
    get((void **)&tcrd, (size_t)nnz * 8);
    get((void **)&tval, (size_t)nnz * 8);
    get((void **)&at, (size_t)n * mp * 8);
    get((void **)&ct, (size_t)p * mp * 8);
    if (!rc && mp != m) {
        // the padding column of A^T takes part in the arithmetic (its results are dropped): keep it finite
        if (cudaMemsetAsync(at, 0, (size_t)n * mp * 8, st) != cudaSuccess ||
            (accumulate && cudaMemsetAsync(ct, 0, (size_t)p * mp * 8, st) != cudaSuccess))
            rc = fail("dense x sparse: clearing the padded operands failed");
    }
    if (!rc) rc = comet_b200_dev_csr_transpose_f64_i64(n, p, nnz, pos, crd, val, tpos, tcrd, tval, st);
    if (!rc) rc = comet_b200_dev_transpose_f64(m, n, a, lda, at, mp, st);
    if (!rc && accumulate) rc = comet_b200_dev_transpose_f64(m, p, c, ldc, ct, mp, st);
    if (!rc) rc = comet_b200_dev_spmm_f64_i64(p, n, nnz, mp, nullptr, tpos, tcrd, tval, at, mp, ct, mp, semiring,
                                              accumulate, 0, st);
    if (!rc) rc = comet_b200_dev_transpose_f64(p, m, ct, mp, c, ldc, st);
    if (tpos) cudaFreeAsync(tpos, st);
    if (tcrd) cudaFreeAsync(tcrd, st);
    if (tval) cudaFreeAsync(tval, st);
    if (at) cudaFreeAsync(at, st);
    if (ct) cudaFreeAsync(ct, st);
    return rc;
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_dense_times_sparse_f64_i64(
    int64_t m, int64_t ncols, int64_t nstored, int64_t nnz, const int64_t *row_ids, const int64_t *pos,
    const int64_t *crd, const double *val, const double *a, int64_t lda, double *c, int64_t ldc,
    int32_t semiring, int32_t accumulate, void *stream)
{
    using namespace cb200;
    clear_error();
    if (semiring != COMET_B200_PLUS_TIMES && semiring != COMET_B200_PLUS_PAIR)
        return fail("dense x sparse: unsupported semiring %d", semiring);
    if (m <= 0 || ncols <= 0) return 0;
    if (ldc < ncols) return fail("dense x sparse: leading dimension of C smaller than its width");
    cudaStream_t st = (cudaStream_t)stream;
    if (m >= DS_SPMM_MIN && !row_ids && nstored > 0 && nnz > 0 && !getenv("COMET_B200_DENSE_SPARSE_ATOMICS"))
        return dense_times_sparse_transposed(m, ncols, nstored, nnz, pos, crd, val, a, lda, c, ldc, semiring, accumulate,
                                             st);
    if (!accumulate) {
        if (ldc == ncols) CB_CUDA(cudaMemsetAsync(c, 0, (size_t)m * ncols * 8, st));
        else CB_CUDA(cudaMemset2DAsync(c, (size_t)ldc * 8, 0, (size_t)ncols * 8, (size_t)m, st));
    }
    if (nstored <= 0 || nnz <= 0) return 0;
    const int64_t tiles = ceil_div(m, DS_TILE);
    int64_t blocks = ceil_div(nstored * tiles, DS_THREADS / 32);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    dense_times_sparse_kernel<<<(unsigned)blocks, DS_THREADS, 0, st>>>(
        m, nstored, row_ids, pos, crd, val, a, lda, c, ldc, semiring == COMET_B200_PLUS_PAIR);
    CB_LAUNCH_CHECK();
    return 0;
}
