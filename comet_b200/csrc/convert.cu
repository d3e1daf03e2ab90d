// Format conversions on the device: stable sort of coordinate entries, COO -> CSR, and the
// transpose of a CSR matrix (CSR of the transposed matrix, i.e. the CSC arrays of the input).
//
// COMET does these on the host with one thread: the reader sorts the parsed entries with
// std::stable_sort by (row, col) and keeps duplicates (lib/ExecutionEngine/SparseUtils.cpp:360-367,
// 404-533), and transpose_2D turns CSR into coordinates, sorts them by (col, row) and rebuilds the
// row pointer (lib/ExecutionEngine/TransposeUtils.cpp:738-812).  Here both are one radix sort of
// 64-bit keys major * extent + minor carrying the entry's position (least significant digit first,
// stable, so equal coordinates keep their input order like stable_sort), a gather of the values, and
// the row pointer from the sorted majors.
//
// The sort is this file's own: per 8-bit digit, a counting kernel (digit histogram per tile), one
// exclusive scan over the digit-major table of counts, and a scatter kernel that ranks every key
// inside its tile.  Ranking is what makes it stable: a warp walks its part of the tile 32
// consecutive keys at a time, `__match_any_sync` names the lanes that hold the same digit, a key's
// rank is the number of such lanes below it plus the count its warp has already seen for the digit,
// and warps are ordered by a prefix over their counts.
//
// Bound: HBM (a pass reads 32 and writes 16 bytes per entry; passes = key bits / 8).
#include "common.cuh"

namespace cb200 {

// ---------------------------------------------------------------------------
// Stable LSD radix sort of (uint64 key, int64 payload) pairs.
// ---------------------------------------------------------------------------
static const int RS_THREADS = 256;                    // 8 warps
static const int RS_ROUNDS = 16;                      // rounds of 32 keys per warp
static const int RS_TILE = RS_THREADS * RS_ROUNDS;    // keys per CTA
static const int RS_DIGITS = 256;

// Walks this warp's part of the tile in order.  On return cnt[d] (this warp's row of shared counters) holds
// the number of keys with digit d, and offs[r] the rank of the key of round r among the warp's keys with the
// same digit.  SCATTER = false only counts.
template <bool SCATTER>
__device__ __forceinline__ void rs_rank_warp(const uint64_t *__restrict__ keys, int64_t base, int64_t n, int shift,
                                             unsigned *cnt, uint64_t (&k)[RS_ROUNDS], unsigned (&offs)[RS_ROUNDS])
{
    const int lane = threadIdx.x & 31;
    const unsigned below = (1u << lane) - 1u;
#pragma unroll
    for (int r = 0; r < RS_ROUNDS; r++) {
        const int64_t i = base + r * 32 + lane;
        const bool live = i < n;
        const uint64_t key = live ? keys[i] : 0;
        const unsigned d = live ? (unsigned)((key >> shift) & (RS_DIGITS - 1)) : RS_DIGITS;   // dead lanes form their own group
        const unsigned peers = __match_any_sync(0xffffffffu, d);
        const int leader = __ffs(peers) - 1;
        unsigned old = 0;
        if (live && lane == leader) {
            old = cnt[d];
            cnt[d] = old + __popc(peers);
        }
        old = __shfl_sync(0xffffffffu, old, leader);
        __syncwarp();
        if (SCATTER) {
            k[r] = key;
            offs[r] = old + __popc(peers & below);
        }
    }
}

// hist[d * ntiles + tile] = number of keys of the tile with digit d
__global__ void __launch_bounds__(RS_THREADS)
rs_count_kernel(const uint64_t *__restrict__ keys, int64_t n, int shift, int64_t ntiles, int64_t *__restrict__ hist)
{
    __shared__ unsigned cnt[RS_THREADS / 32][RS_DIGITS];
    const int w = threadIdx.x >> 5;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < (RS_THREADS / 32) * RS_DIGITS; i += RS_THREADS) (&cnt[0][0])[i] = 0;
        __syncthreads();
        uint64_t k[RS_ROUNDS];
        unsigned offs[RS_ROUNDS];
        rs_rank_warp<false>(keys, tile * RS_TILE + (int64_t)w * 32 * RS_ROUNDS, n, shift, cnt[w], k, offs);
        __syncthreads();
        if (threadIdx.x < RS_DIGITS) {
            unsigned t = 0;
            for (int i = 0; i < RS_THREADS / 32; i++) t += cnt[i][threadIdx.x];
            hist[(int64_t)threadIdx.x * ntiles + tile] = t;
        }
        __syncthreads();
    }
}

// base[d * ntiles + tile] = first output position of the tile's keys with digit d (exclusive scan of hist)
__global__ void __launch_bounds__(RS_THREADS)
rs_scatter_kernel(const uint64_t *__restrict__ keys, const int64_t *__restrict__ vals, int64_t n, int shift,
                  int64_t ntiles, const int64_t *__restrict__ base, uint64_t *__restrict__ keys_out,
                  int64_t *__restrict__ vals_out)
{
    __shared__ unsigned cnt[RS_THREADS / 32][RS_DIGITS];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
        for (int i = threadIdx.x; i < (RS_THREADS / 32) * RS_DIGITS; i += RS_THREADS) (&cnt[0][0])[i] = 0;
        __syncthreads();
        uint64_t k[RS_ROUNDS];
        unsigned offs[RS_ROUNDS];
        const int64_t wbase = tile * RS_TILE + (int64_t)w * 32 * RS_ROUNDS;
        rs_rank_warp<true>(keys, wbase, n, shift, cnt[w], k, offs);
        __syncthreads();
        if (threadIdx.x < RS_DIGITS) {        // counts per warp -> start of each warp's keys inside the tile's run of the digit
            unsigned run = 0;
            for (int i = 0; i < RS_THREADS / 32; i++) {
                const unsigned c = cnt[i][threadIdx.x];
                cnt[i][threadIdx.x] = run;
                run += c;
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RS_ROUNDS; r++) {
            const int64_t i = wbase + r * 32 + lane;
            if (i < n) {
                const unsigned d = (unsigned)((k[r] >> shift) & (RS_DIGITS - 1));
                const int64_t at = base[(int64_t)d * ntiles + tile] + cnt[w][d] + offs[r];
                keys_out[at] = k[r];
                vals_out[at] = vals[i];
            }
        }
        __syncthreads();
    }
}

// Sorts n pairs by the low `bits` bits of the key.  The result is in (keys, vals) or (keys2, vals2): *in_second
// tells which.  hist / base: scratch of 256 * ntiles + 1 int64 each.
static int radix_sort_pairs(uint64_t *keys, uint64_t *keys2, int64_t *vals, int64_t *vals2, int64_t n, int bits,
                            int64_t *hist, int64_t *base, bool *in_second, cudaStream_t st)
{
    const int64_t ntiles = ceil_div(n, RS_TILE);
    int64_t grid = ntiles;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (grid > cap) grid = cap;
    bool second = false;
    for (int shift = 0; shift < bits; shift += 8) {
        uint64_t *kin = second ? keys2 : keys, *kout = second ? keys : keys2;
        int64_t *vin = second ? vals2 : vals, *vout = second ? vals : vals2;
        rs_count_kernel<<<(unsigned)grid, RS_THREADS, 0, st>>>(kin, n, shift, ntiles, hist);
        CB_LAUNCH_CHECK();
        CB_TRY(exclusive_scan_i64(hist, base, RS_DIGITS * ntiles, st));
        rs_scatter_kernel<<<(unsigned)grid, RS_THREADS, 0, st>>>(kin, vin, n, shift, ntiles, base, kout, vout);
        CB_LAUNCH_CHECK();
        second = !second;
    }
    *in_second = second;
    return 0;
}

__global__ void __launch_bounds__(256)
make_keys_kernel(int64_t n, const int64_t *__restrict__ major, const int64_t *__restrict__ minor,
                 int64_t nmajor, int64_t nminor, uint64_t *__restrict__ keys, int64_t *__restrict__ idx,
                 int *__restrict__ bad)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t a = major[i], b = minor[i];
        if (a < 0 || a >= nmajor || b < 0 || b >= nminor) {
            *bad = 1;                                   // reported by the host; the key stays in range
            keys[i] = 0;
        } else {
            keys[i] = (uint64_t)a * (uint64_t)nminor + (uint64_t)b;
        }
        idx[i] = i;
    }
}

__global__ void __launch_bounds__(256)
gather_sorted_kernel(int64_t n, const uint64_t *__restrict__ keys, const int64_t *__restrict__ idx,
                     int64_t nminor, const double *__restrict__ vals, int64_t *__restrict__ major_out,
                     int64_t *__restrict__ minor_out, double *__restrict__ vals_out)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint64_t k = keys[i];
        if (major_out) major_out[i] = (int64_t)(k / (uint64_t)nminor);
        if (minor_out) minor_out[i] = (int64_t)(k % (uint64_t)nminor);
        if (vals_out) vals_out[i] = vals[idx[i]];
    }
}

// row of every stored entry of a CSR matrix: 8 lanes per row
__global__ void __launch_bounds__(256)
expand_rows_kernel(int64_t nrows, const int64_t *__restrict__ pos, int64_t *__restrict__ rows)
{
    const int l = threadIdx.x & 7;
    const int64_t g = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int64_t ng = ((int64_t)gridDim.x * blockDim.x) >> 3;
    for (int64_t r = g; r < nrows; r += ng)
        for (int64_t p = pos[r] + l; p < pos[r + 1]; p += 8) rows[p] = r;
}

static unsigned grid_for(int64_t work)
{
    int64_t blocks = ceil_div(work > 0 ? work : 1, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(blocks > cap ? cap : blocks);
}

static int key_bits(int64_t nmajor, int64_t nminor, int *bits)
{
    if (nmajor <= 0 || nminor <= 0) return fail("sort: empty coordinate space");
    const unsigned __int128 space = (unsigned __int128)nmajor * (unsigned __int128)nminor;
    if (space >> 63) return fail("sort: rows x cols = %lld x %lld does not fit a 63-bit key", (long long)nmajor,
                                 (long long)nminor);
    int b = 1;
    while (b < 63 && ((unsigned __int128)1 << b) < space) b++;
    *bits = b;
    return 0;
}

// Entries sorted by (major, minor), equal coordinates in input order.  Any of the outputs may be null.
int sort_coo(int64_t n, int64_t nmajor, int64_t nminor, const int64_t *major, const int64_t *minor,
             const double *vals, int64_t *major_out, int64_t *minor_out, double *vals_out, cudaStream_t st)
{
    if (n <= 0) return 0;
    int bits = 0;
    CB_TRY(key_bits(nmajor, nminor, &bits));
    uint64_t *keys = nullptr, *keys2 = nullptr;
    int64_t *idx = nullptr, *idx2 = nullptr, *hist = nullptr, *base = nullptr;
    int *bad = nullptr;
    const size_t table = (size_t)RS_DIGITS * (size_t)ceil_div(n, RS_TILE) + 1;
    int rc = 0;
    auto alloc = [&](void **p, size_t bytes) {
        if (rc) return;
        if (cudaMallocAsync(p, bytes ? bytes : 8, st) != cudaSuccess) {
            *p = nullptr;
            rc = fail("sort: device allocation of %zu bytes failed", bytes);
        }
    };
    alloc((void **)&keys, (size_t)n * 8);
    alloc((void **)&keys2, (size_t)n * 8);
    alloc((void **)&idx, (size_t)n * 8);
    alloc((void **)&idx2, (size_t)n * 8);
    alloc((void **)&bad, sizeof(int));
    alloc((void **)&hist, table * 8);
    alloc((void **)&base, table * 8);
    int bad_host = 0;
    bool second = false;
    if (!rc) {
        cudaMemsetAsync(bad, 0, sizeof(int), st);
        make_keys_kernel<<<grid_for(n), 256, 0, st>>>(n, major, minor, nmajor, nminor, keys, idx, bad);
        rc = radix_sort_pairs(keys, keys2, idx, idx2, n, bits, hist, base, &second, st);
    }
    if (!rc) {
        gather_sorted_kernel<<<grid_for(n), 256, 0, st>>>(n, second ? keys2 : keys, second ? idx2 : idx, nminor, vals,
                                                          major_out, minor_out, vals ? vals_out : nullptr);
        if (cudaMemcpyAsync(&bad_host, bad, sizeof(int), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess || cudaGetLastError() != cudaSuccess)
            rc = fail("sort: kernels failed");
        else if (bad_host)
            rc = fail("sort: a coordinate lies outside %lld x %lld", (long long)nmajor, (long long)nminor);
    }
    void *all[] = {keys, keys2, idx, idx2, bad, hist, base};
    for (void *p : all)
        if (p) cudaFreeAsync(p, st);
    return rc;
}

}  // namespace cb200

using namespace cb200;

extern "C" int32_t comet_b200_dev_sort_coo_f64_i64(int64_t n, int64_t nmajor, int64_t nminor, const int64_t *major,
                                                   const int64_t *minor, const double *vals, int64_t *major_out,
                                                   int64_t *minor_out, double *vals_out, void *stream)
{
    clear_error();
    return sort_coo(n, nmajor, nminor, major, minor, vals, major_out, minor_out, vals_out, (cudaStream_t)stream);
}

extern "C" int32_t comet_b200_dev_coo_to_csr_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz, const int64_t *rows,
                                                     const int64_t *cols, const double *vals, int64_t *pos,
                                                     int64_t *crd, double *val, void *stream)
{
    clear_error();
    cudaStream_t st = (cudaStream_t)stream;
    if (nrows < 0 || ncols < 0 || nnz < 0) return fail("coo_to_csr: negative size");
    if (nnz == 0) {
        CB_CUDA(cudaMemsetAsync(pos, 0, (size_t)(nrows + 1) * 8, st));
        return 0;
    }
    int64_t *srows = nullptr;
    int *flag = nullptr;
    CB_CUDA(cudaMallocAsync((void **)&srows, (size_t)nnz * 8, st));
    int rc = sort_coo(nnz, nrows, ncols, rows, cols, vals, srows, crd, val, st);
    if (!rc && cudaMallocAsync((void **)&flag, sizeof(int), st) != cudaSuccess) rc = fail("coo_to_csr: allocation failed");
    if (!rc) {
        int one = 1;
        cudaMemcpyAsync(flag, &one, sizeof(int), cudaMemcpyHostToDevice, st);
        rc = coo_rows_to_pos(srows, nnz, nrows, pos, flag, st);
    }
    cudaFreeAsync(srows, st);
    if (flag) cudaFreeAsync(flag, st);
    return rc;
}

extern "C" int32_t comet_b200_dev_csr_transpose_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz, const int64_t *pos,
                                                        const int64_t *crd, const double *val, int64_t *tpos,
                                                        int64_t *tcrd, double *tval, void *stream)
{
    clear_error();
    cudaStream_t st = (cudaStream_t)stream;
    if (nrows < 0 || ncols < 0 || nnz < 0) return fail("transpose: negative size");
    if (nnz == 0) {
        CB_CUDA(cudaMemsetAsync(tpos, 0, (size_t)(ncols + 1) * 8, st));
        return 0;
    }
    int64_t *rows = nullptr, *scols = nullptr;
    int *flag = nullptr;
    CB_CUDA(cudaMallocAsync((void **)&rows, (size_t)nnz * 8, st));
    if (cudaMallocAsync((void **)&scols, (size_t)nnz * 8, st) != cudaSuccess) {
        cudaFreeAsync(rows, st);
        return fail("transpose: allocation failed");
    }
    expand_rows_kernel<<<grid_for(nrows * 8), 256, 0, st>>>(nrows, pos, rows);
    // major = column of the input, minor = its row: the transposed matrix in row-major order
    int rc = sort_coo(nnz, ncols, nrows, crd, rows, val, scols, tcrd, tval, st);
    if (!rc && cudaMallocAsync((void **)&flag, sizeof(int), st) != cudaSuccess) rc = fail("transpose: allocation failed");
    if (!rc) {
        int one = 1;
        cudaMemcpyAsync(flag, &one, sizeof(int), cudaMemcpyHostToDevice, st);
        rc = coo_rows_to_pos(scols, nnz, ncols, tpos, flag, st);
    }
    cudaFreeAsync(rows, st);
    cudaFreeAsync(scols, st);
    if (flag) cudaFreeAsync(flag, st);
    return rc;
}
