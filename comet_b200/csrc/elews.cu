// Elementwise multiply  C = A .* B  with sparse A (CSR or COO) and dense row-major B:
// C keeps A's pattern, C.val[p] = A.val[p] * B[row(p), crd[p]].
// Bound: HBM (24 bytes streamed per entry plus one gathered f64).
#include "common.cuh"

namespace cb200 {

__global__ void __launch_bounds__(256)
elews_coo_kernel(int64_t nnz, const int64_t *__restrict__ rows, const int64_t *__restrict__ crd,
                 const double *__restrict__ val, const double *__restrict__ b, int64_t ldb,
                 double *__restrict__ out)
{
    for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz;
         p += (int64_t)gridDim.x * blockDim.x)
        out[p] = ld_stream(val + p) * __ldg(b + ld_stream(rows + p) * ldb + ld_stream(crd + p));
}

// 8 lanes per row
__global__ void __launch_bounds__(256)
elews_csr_kernel(int64_t nrows, const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                 const double *__restrict__ val, const double *__restrict__ b, int64_t ldb,
                 double *__restrict__ out)
{
    const int l = threadIdx.x & 7;
    int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int64_t ng = ((int64_t)gridDim.x * blockDim.x) >> 3;
    for (int64_t r = g; r < nrows; r += ng) {
        const double *brow = b + r * ldb;
        for (int64_t p = pos[r] + l; p < pos[r + 1]; p += 8)
            out[p] = ld_stream(val + p) * __ldg(brow + ld_stream(crd + p));
    }
}

// Dense output: C[row, col] = A.val * B[row, col] at A's stored positions, the rest of C untouched
// (the reduce operator of ta.elews_mul is "noop": the product is assigned, not added).
// 8 lanes per stored row; COO entries carry their own row.
__global__ void __launch_bounds__(256)
elews_to_dense_kernel(int64_t nstored, int64_t nnz, const int64_t *__restrict__ row_ids,
                      const int64_t *__restrict__ pos, const int64_t *__restrict__ rows,
                      const int64_t *__restrict__ crd, const double *__restrict__ val,
                      const double *__restrict__ b, int64_t ldb, double *__restrict__ c, int64_t ldc)
{
    if (rows) {
        for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < nnz;
             p += (int64_t)gridDim.x * blockDim.x) {
            const int64_t r = rows[p], col = crd[p];
            c[r * ldc + col] = val[p] * __ldg(b + r * ldb + col);
        }
        return;
    }
    const int l = threadIdx.x & 7;
    int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int64_t ng = ((int64_t)gridDim.x * blockDim.x) >> 3;
    for (int64_t s = g; s < nstored; s += ng) {
        const int64_t r = row_ids ? row_ids[s] : s;
        for (int64_t p = pos[s] + l; p < pos[s + 1]; p += 8) {
            const int64_t col = crd[p];
            c[r * ldc + col] = val[p] * __ldg(b + r * ldb + col);
        }
    }
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_elews_mul_sparse_dense_to_dense_f64_i64(
    int64_t nstored, int64_t nnz, const int64_t *row_ids, const int64_t *pos, const int64_t *rows,
    const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
    void *stream)
{
    using namespace cb200;
    clear_error();
    if (nnz <= 0) return 0;
    const int64_t work = rows ? nnz : nstored * 8;
    int64_t blocks = ceil_div(work, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    elews_to_dense_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(nstored, nnz, row_ids, pos, rows, crd,
                                                                            val, b, ldb, c, ldc);
    CB_LAUNCH_CHECK();
    return 0;
}

extern "C" int32_t comet_b200_dev_elews_mul_sparse_dense_f64_i64(
    int64_t nrows, int64_t nnz, const int64_t *pos, const int64_t *rows, const int64_t *crd,
    const double *val, const double *b, int64_t ldb, double *out, void *stream)
{
    using namespace cb200;
    clear_error();
    if (nnz <= 0 || nrows <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    int64_t cap = (int64_t)sm_count() * 16;
    if (rows) {
        int64_t blocks = ceil_div(nnz, 256);
        if (blocks > cap) blocks = cap;
        elews_coo_kernel<<<(unsigned)blocks, 256, 0, st>>>(nnz, rows, crd, val, b, ldb, out);
    } else {
        int64_t blocks = ceil_div(nrows * 8, 256);
        if (blocks > cap) blocks = cap;
        elews_csr_kernel<<<(unsigned)blocks, 256, 0, st>>>(nrows, pos, crd, val, b, ldb, out);
    }
    CB_LAUNCH_CHECK();
    return 0;
}
