// Small shared device routines: index narrowing, exclusive scan, COO adapter, transpose.
#include "common.cuh"

namespace cb200 {

// ---------------------------------------------------------------------------
// int64 -> int32 copy of a coordinate array (columns < 2^31), 2 elements/thread.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) narrow_kernel(const int64_t *__restrict__ src,
                                                     int32_t *__restrict__ dst, int64_t n)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x * 2;
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 2; i < n; i += stride) {
        if (i + 1 < n) {
            longlong2 v = __ldcs((const longlong2 *)(src + i));
            *(int2 *)(dst + i) = make_int2((int)v.x, (int)v.y);
        } else {
            dst[i] = (int32_t)src[i];
        }
    }
}

__global__ void __launch_bounds__(256) widen_kernel(const int32_t *__restrict__ src,
                                                    int64_t *__restrict__ dst, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = (int64_t)__ldcs(src + i);
}

__global__ void __launch_bounds__(256) narrow_scalar_kernel(const int64_t *__restrict__ src,
                                                            int32_t *__restrict__ dst, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = (int32_t)src[i];
}

// float <-> double copies for the _f32_ entry points (values are widened once after the upload and results
// narrowed once before the download; every kernel computes in double)
__global__ void __launch_bounds__(256) widen_f32_kernel(const float *__restrict__ src, double *__restrict__ dst, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = (double)__ldcs(src + i);
}

__global__ void __launch_bounds__(256) narrow_f64_kernel(const double *__restrict__ src, float *__restrict__ dst, int64_t n)
{
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = (float)__ldcs(src + i);
}

static unsigned stream_grid(int64_t n)
{
    int64_t blocks = ceil_div(n, 256);
    int64_t cap = (int64_t)sm_count() * 16;
    return (unsigned)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

int widen_f32_to_f64(const float *src, double *dst, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    widen_f32_kernel<<<stream_grid(n), 256, 0, st>>>(src, dst, n);
    CB_LAUNCH_CHECK();
    return 0;
}

int narrow_f64_to_f32(const double *src, float *dst, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    narrow_f64_kernel<<<stream_grid(n), 256, 0, st>>>(src, dst, n);
    CB_LAUNCH_CHECK();
    return 0;
}

int widen_i32_to_i64(const int32_t *src, int64_t *dst, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    widen_kernel<<<stream_grid(n), 256, 0, st>>>(src, dst, n);
    CB_LAUNCH_CHECK();
    return 0;
}

// no alignment requirement (the vectorised narrow_i64_to_i32 wants 16-byte aligned input)
int narrow_any_i64_to_i32(const int64_t *src, int32_t *dst, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    narrow_scalar_kernel<<<stream_grid(n), 256, 0, st>>>(src, dst, n);
    CB_LAUNCH_CHECK();
    return 0;
}

int narrow_i64_to_i32(const int64_t *src, int32_t *dst, int64_t n, cudaStream_t st)
{
    if (n <= 0) return 0;
    if (((uintptr_t)src & 15) || ((uintptr_t)dst & 7))
        return fail("narrow_i64_to_i32: arrays must be 16-byte (src) and 8-byte (dst) aligned");
    int64_t blocks = ceil_div(n, 512);
    int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    narrow_kernel<<<(unsigned)blocks, 256, 0, st>>>(src, dst, n);
    CB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Exclusive scan of int64 (reduce, scan of tile sums, scan with offsets).
// ---------------------------------------------------------------------------
static const int SCAN_THREADS = 256;
static const int SCAN_ITEMS = 8;
static const int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *total)
{
    __shared__ int64_t warp_sums[SCAN_THREADS / 32];
    __shared__ int64_t block_total;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int64_t t = __shfl_up_sync(0xffffffffu, (long long)inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) warp_sums[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int64_t w = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
        int64_t winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int64_t t = __shfl_up_sync(0xffffffffu, (long long)winc, o);
            if (lane >= o) winc += t;
        }
        if (lane < SCAN_THREADS / 32) warp_sums[lane] = winc - w;
        if (lane == 31) block_total = winc;
    }
    __syncthreads();
    int64_t r = inc - v + warp_sums[warp];
    *total = block_total;
    __syncthreads();
    return r;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_sums(const int64_t *__restrict__ in,
                                                               int64_t *__restrict__ sums, int64_t n)
{
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++)
        if (base + i < n) s += in[base + i];
    int64_t total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_sums_inplace(int64_t *sums, int64_t ntiles,
                                                                  int64_t *grand_total)
{
    int64_t carry = 0;
    for (int64_t base = 0; base < ntiles; base += SCAN_THREADS) {
        int64_t i = base + threadIdx.x;
        int64_t v = i < ntiles ? sums[i] : 0;
        int64_t total;
        int64_t ex = block_exclusive_scan(v, &total);
        if (i < ntiles) sums[i] = ex + carry;
        carry += total;
    }
    if (threadIdx.x == 0) *grand_total = carry;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_apply(const int64_t *__restrict__ in,
                                                           const int64_t *__restrict__ sums,
                                                           int64_t *__restrict__ out, int64_t n)
{
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int64_t v[SCAN_ITEMS];
    int64_t s = 0;
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) {
        v[i] = base + i < n ? in[base + i] : 0;
        s += v[i];
    }
    int64_t total;
    int64_t ex = block_exclusive_scan(s, &total) + sums[blockIdx.x];
#pragma unroll
    for (int i = 0; i < SCAN_ITEMS; i++) {
        if (base + i < n) out[base + i] = ex;
        ex += v[i];
    }
}

int exclusive_scan_i64(const int64_t *in, int64_t *out, int64_t n, cudaStream_t st)
{
    if (n <= 0) {
        CB_CUDA(cudaMemsetAsync(out, 0, sizeof(int64_t), st));
        return 0;
    }
    int64_t ntiles = ceil_div(n, SCAN_TILE);
    void *p = nullptr;
    CB_TRY(scratch(SLOT_SCAN, (size_t)ntiles * sizeof(int64_t), &p));
    int64_t *sums = (int64_t *)p;
    scan_tile_sums<<<(unsigned)ntiles, SCAN_THREADS, 0, st>>>(in, sums, n);
    CB_LAUNCH_CHECK();
    scan_sums_inplace<<<1, SCAN_THREADS, 0, st>>>(sums, ntiles, out + n);
    CB_LAUNCH_CHECK();
    scan_apply<<<(unsigned)ntiles, SCAN_THREADS, 0, st>>>(in, sums, out, n);
    CB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// COO adapter: row coordinates sorted ascending (the reference reader sorts by
// (row, col), lib/ExecutionEngine/SparseUtils.cpp:1855) -> row pointer.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) coo_pos_kernel(const int64_t *__restrict__ rows, int64_t nnz,
                                                      int64_t nrows, int64_t *__restrict__ pos,
                                                      int *__restrict__ flag)
{
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t r = t0; r <= nrows; r += stride) {
        int64_t lo = 0, hi = nnz;   // first p with rows[p] >= r
        while (lo < hi) {
            int64_t mid = (lo + hi) >> 1;
            if (rows[mid] < r) lo = mid + 1; else hi = mid;
        }
        pos[r] = lo;
    }
    for (int64_t p = t0; p < nnz; p += stride) {
        int64_t r = rows[p];
        bool bad = r < 0 || r >= nrows || (p + 1 < nnz && rows[p + 1] < r);
        if (bad) *flag = 0;
    }
}

int coo_rows_to_pos(const int64_t *rows, int64_t nnz, int64_t nrows, int64_t *pos, int *flag_dev,
                    cudaStream_t st)
{
    int64_t work = nnz > nrows + 1 ? nnz : nrows + 1;
    int64_t blocks = ceil_div(work, 256);
    int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    coo_pos_kernel<<<(unsigned)blocks, 256, 0, st>>>(rows, nnz, nrows, pos, flag_dev);
    CB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Range check of a coordinate array: *flag_dev is set to 0 when some idx[i] lies outside [0, limit).
// The kernels index dense operands and bitmaps with these coordinates without further checks, so the
// host entry points run this once per uploaded array and refuse the call before any of them starts.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) index_range_kernel(const int64_t *__restrict__ idx, int64_t n, int64_t limit,
                                                          int *flag_dev)
{
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = idx[i];
        bad |= (v < 0) | (v >= limit);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *flag_dev = 0;
}

int check_index_range(const int64_t *idx, int64_t n, int64_t limit, int *flag_dev, cudaStream_t st)
{
    if (n <= 0) return 0;
    index_range_kernel<<<stream_grid(n), 256, 0, st>>>(idx, n, limit, flag_dev);
    CB_LAUNCH_CHECK();
    return 0;
}

// ---------------------------------------------------------------------------
// Tiled transpose of a row-major f64 matrix through shared memory.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose_kernel(int64_t rows, int64_t cols,
                                                        const double *__restrict__ src, int64_t lds,
                                                        double *__restrict__ dst, int64_t ldd)
{
    __shared__ double tile[32][33];
    int64_t tiles_x = (cols + 31) / 32;
    int64_t tiles = tiles_x * ((rows + 31) / 32);
    int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        int64_t r0 = (t / tiles_x) * 32, c0 = (t % tiles_x) * 32;
        for (int j = ty; j < 32; j += 8)
            if (r0 + j < rows && c0 + tx < cols) tile[j][tx] = src[(r0 + j) * lds + c0 + tx];
        __syncthreads();
        for (int j = ty; j < 32; j += 8)
            if (c0 + j < cols && r0 + tx < rows) dst[(c0 + j) * ldd + r0 + tx] = tile[tx][j];
        __syncthreads();
    }
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_transpose_f64(int64_t rows, int64_t cols, const double *src,
                                                int64_t lds, double *dst, int64_t ldd, void *stream)
{
    using namespace cb200;
    clear_error();
    if (rows <= 0 || cols <= 0) return 0;
    int64_t tiles = ceil_div(rows, 32) * ceil_div(cols, 32);
    int64_t cap = (int64_t)sm_count() * 8;
    if (tiles > cap) tiles = cap;
    transpose_kernel<<<(unsigned)tiles, 256, 0, (cudaStream_t)stream>>>(rows, cols, src, lds, dst, ldd);
    CB_LAUNCH_CHECK();
    return 0;
}
