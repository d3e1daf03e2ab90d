// SpMM  C[a,:] = C[a,:] (+) sum_b A[a,b] (x) B[b,:]   (CSR / DCSR rows, dense row-major B and C).
//
// Row-panel design.  A group of T lanes owns one row of A and a panel of W
// columns of B/C (2*NI doubles per lane, 128-bit loads); it loads T (crd, val)
// pairs at a time with one coalesced streaming load and broadcasts them with
// shuffles, so the only gathered traffic is B rows.  When W < K the grid walks
// the column panels one after the other ("slice-major"), so the slice of B in
// flight is K/W times smaller and stays in L2; crd is then narrowed to int32
// once, because A is re-read per slice.
//
// Rows longer than LONG_ROW entries are cut into chunks of CHUNK entries that
// go to a work list in scratch memory; a second launch gives each chunk to a
// whole CTA and adds its partial panel to C with f64 atomics (order of those
// few additions is not fixed; differences stay at rounding level).
//
// Bound: HBM.  Algorithmic bytes = 8(n+1) + 16 nnz + 8 ncols K + 8 nrows K.
#include "common.cuh"

namespace cb200 {

static const int SPMM_THREADS = 256;
static const int SPMM_FETCH = 8;            // rows per lane group per draw
static const int64_t SPMM_LONG_ROW = 512;
static const int64_t SPMM_CHUNK = 512;

template <int T, int NI, typename IdxT>
__device__ __forceinline__ void panel_accumulate(double2 (&acc)[NI], const IdxT *__restrict__ crd,
                                                 const double *__restrict__ val,
                                                 const double *__restrict__ bpanel, int64_t ldb,
                                                 int64_t s, int64_t e, int l, unsigned gmask,
                                                 int ncol2, bool pair)
{
    for (int64_t base = s; base < e; base += T) {
        int64_t p = base + l;
        IdxT c = 0;
        double v = 0.0;
        if (p < e) {
            c = ld_stream(crd + p);
            v = ld_stream(val + p);
        }
        int n = (e - base) < T ? (int)(e - base) : T;
        if (pair) {
#pragma unroll
            for (int i = 0; i < NI; i++) { acc[i].x += (double)n; acc[i].y += (double)n; }
            continue;
        }
#pragma unroll 4
        for (int t = 0; t < n; t++) {
            IdxT cc = __shfl_sync(gmask, c, t, T);
            double vv = __shfl_sync(gmask, v, t, T);
            const double2 *br = (const double2 *)(bpanel + (int64_t)cc * ldb);
#pragma unroll
            for (int i = 0; i < NI; i++) {
                if (l + i * T < ncol2) {
                    double2 b = __ldg(br + l + i * T);
                    acc[i].x = fma(vv, b.x, acc[i].x);
                    acc[i].y = fma(vv, b.y, acc[i].y);
                }
            }
        }
    }
}

template <int T, int NI, typename IdxT>
__global__ void __launch_bounds__(SPMM_THREADS)
spmm_rows_kernel(int64_t nrows, const int64_t *__restrict__ row_ids,
                 const int64_t *__restrict__ pos, const IdxT *__restrict__ crd,
                 const double *__restrict__ val, const double *__restrict__ b, int64_t ldb,
                 double *__restrict__ c, int64_t ldc, int k, int slice_cols, int64_t row_blocks,
                 int accumulate, int pair, WorkHeader *hdr, Chunk *chunks, unsigned chunk_cap)
{
    // Persistent warps draw blocks of rows from a counter (hdr->pad[0]): with rows of very
    // different lengths a static assignment leaves most warps of a CTA idle while one finishes.
    constexpr int GPW = 32 / T;                       // lane groups (rows in flight) per warp
    constexpr int BLOCK_ROWS = GPW * SPMM_FETCH;      // rows per draw
    const int l = threadIdx.x % T;
    const int lane = threadIdx.x & 31;
    const int gw = lane / T;
    const unsigned gmask = (T == 32) ? 0xffffffffu : (((1u << T) - 1u) << (lane & ~(T - 1)));
    const int64_t total_items = row_blocks * (int64_t)((k + slice_cols - 1) / slice_cols);
    while (true) {
        __syncwarp();
        unsigned item = 0;
        if (lane == 0) item = atomicAdd(&hdr->pad[0], 1u);
        item = __shfl_sync(0xffffffffu, item, 0);
        if ((int64_t)item >= total_items) break;
        const int slice = (int)(item / row_blocks);
        const int64_t row0 = (int64_t)(item % row_blocks) * BLOCK_ROWS;
        const int col0 = slice * slice_cols;
        const int ncol2 = ((k - col0) < slice_cols ? (k - col0) : slice_cols) / 2;
        const double *bpanel = b + col0;
    for (int pass = 0; pass < SPMM_FETCH; pass++) {
        int64_t r = row0 + pass * GPW + gw;
        if (r >= nrows) break;
        int64_t s = pos[r], e = pos[r + 1];
        int64_t out = row_ids ? row_ids[r] : r;
        double2 *crow = (double2 *)(c + out * ldc + col0);
        if (e - s > SPMM_LONG_ROW) {
            if (!accumulate) {
#pragma unroll
                for (int i = 0; i < NI; i++)
                    if (l + i * T < ncol2) crow[l + i * T] = make_double2(0.0, 0.0);
            }
            if (slice == 0 && l == 0) {
                unsigned n = (unsigned)((e - s + SPMM_CHUNK - 1) / SPMM_CHUNK);
                unsigned at = atomicAdd(&hdr->count, n);
                if (at + n <= chunk_cap) {
                    for (unsigned i = 0; i < n; i++) {
                        chunks[at + i].row = r;
                        chunks[at + i].begin = s + (int64_t)i * SPMM_CHUNK;
                    }
                } else {
                    hdr->overflow = 1;
                }
            }
            continue;
        }
        double2 acc[NI];
#pragma unroll
        for (int i = 0; i < NI; i++) acc[i] = make_double2(0.0, 0.0);
        panel_accumulate<T, NI, IdxT>(acc, crd, val, bpanel, ldb, s, e, l, gmask, ncol2, pair != 0);
#pragma unroll
        for (int i = 0; i < NI; i++) {
            if (l + i * T < ncol2) {
                double2 o = acc[i];
                if (accumulate) {
                    double2 old = __ldcs(crow + l + i * T);
                    o.x += old.x;
                    o.y += old.y;
                }
                __stcs(crow + l + i * T, o);   // written once, never re-read: keep it out of B's way in L2
            }
        }
    }
    }
}

template <int T, int NI, typename IdxT>
__global__ void __launch_bounds__(SPMM_THREADS)
spmm_chunks_kernel(const int64_t *__restrict__ row_ids, const int64_t *__restrict__ pos,
                   const IdxT *__restrict__ crd, const double *__restrict__ val,
                   const double *__restrict__ b, int64_t ldb, double *__restrict__ c, int64_t ldc,
                   int k, int slice_cols, int nslices, int pair, const WorkHeader *hdr,
                   const Chunk *chunks, unsigned chunk_cap)
{
    constexpr int GROUPS = SPMM_THREADS / T;
    __shared__ double2 part[GROUPS][NI][T];
    const int g = threadIdx.x / T, l = threadIdx.x % T;
    const int lane = threadIdx.x & 31;
    const unsigned gmask = (T == 32) ? 0xffffffffu : (((1u << T) - 1u) << (lane & ~(T - 1)));
    unsigned count = hdr->count;
    if (count > chunk_cap) count = 0;   // cannot happen when nnz == pos[nrows] (the list's capacity is a bound for that nnz); never read past the list
    const int64_t total = (int64_t)count * nslices;
    for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
        const int slice = (int)(w / count);
        const Chunk ch = chunks[w % count];
        const int col0 = slice * slice_cols;
        const int ncol2 = ((k - col0) < slice_cols ? (k - col0) : slice_cols) / 2;
        int64_t cend = pos[ch.row + 1];
        if (cend > ch.begin + SPMM_CHUNK) cend = ch.begin + SPMM_CHUNK;
        const int64_t per = (cend - ch.begin + GROUPS - 1) / GROUPS;
        int64_t s = ch.begin + (int64_t)g * per, e = s + per;
        if (e > cend) e = cend;
        double2 acc[NI];
#pragma unroll
        for (int i = 0; i < NI; i++) acc[i] = make_double2(0.0, 0.0);
        if (s < e)
            panel_accumulate<T, NI, IdxT>(acc, crd, val, b + col0, ldb, s, e, l, gmask, ncol2, pair != 0);
#pragma unroll
        for (int i = 0; i < NI; i++) part[g][i][l] = acc[i];
        __syncthreads();
        if (g == 0) {
            int64_t out = row_ids ? row_ids[ch.row] : ch.row;
            double *crow = c + out * ldc + col0;
#pragma unroll
            for (int i = 0; i < NI; i++) {
                if (l + i * T < ncol2) {
                    double2 t = part[0][i][l];
                    for (int gg = 1; gg < GROUPS; gg++) {
                        t.x += part[gg][i][l].x;
                        t.y += part[gg][i][l].y;
                    }
                    atomicAdd(crow + 2 * (l + i * T), t.x);
                    atomicAdd(crow + 2 * (l + i * T) + 1, t.y);
                }
            }
        }
        __syncthreads();
    }
}

// Any K, any alignment: one thread per output element.  Correctness path for
// shapes the panel kernels do not take (odd K, unaligned or odd leading dimensions).
__global__ void __launch_bounds__(256)
spmm_scalar_kernel(int64_t nrows, const int64_t *__restrict__ row_ids,
                   const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                   const double *__restrict__ val, const double *__restrict__ b, int64_t ldb,
                   double *__restrict__ c, int64_t ldc, int64_t k, int accumulate, int pair)
{
    int64_t total = nrows * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / k, j = i % k;
        double sum = 0.0;
        for (int64_t p = pos[r]; p < pos[r + 1]; p++)
            sum += pair ? 1.0 : val[p] * b[crd[p] * ldb + j];
        int64_t out = row_ids ? row_ids[r] : r;
        c[out * ldc + j] = accumulate ? c[out * ldc + j] + sum : sum;
    }
}

int spmm_stream(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k, const int64_t *row_ids, const int64_t *pos,
                const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
                int accumulate, bool forced, cudaStream_t st);
int spmm_stream_tma(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k, const int64_t *row_ids, const int64_t *pos,
                    const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
                    int accumulate, bool gather4, cudaStream_t st);

// Shapes the entry-stream path takes without being asked.
// From 64 columns on a row of B fills the lanes of a warp and the stream wins on uniform and
// skewed matrices alike (R-MAT scale 20, K = 128: 1.19 ms against 1.83 ms); below that the
// lane groups of the panel kernels waste less.
static bool spmm_stream_preferred(int64_t nrows, int64_t nnz, int64_t k)
{
    (void)nrows; (void)nnz;
    return k >= 64;
}

struct SpmmArgs {
    int64_t nrows, nnz;
    const int64_t *row_ids, *pos;
    const void *crd;
    const double *val, *b;
    int64_t ldb;
    double *c;
    int64_t ldc;
    int k, slice_cols, nslices, accumulate, pair;
    WorkHeader *hdr;
    Chunk *chunks;
    unsigned chunk_cap;
    cudaStream_t st;
};

template <int T, int NI, typename IdxT>
static int launch_panels(const SpmmArgs &a)
{
    constexpr int BLOCK_ROWS = (32 / T) * SPMM_FETCH;
    int64_t row_blocks = ceil_div(a.nrows, BLOCK_ROWS);
    int64_t items = row_blocks * a.nslices;
    if (items > 0xfffffff0LL) return fail("spmm: too many row blocks");
    int64_t grid = ceil_div(items, SPMM_THREADS / 32);
    const int64_t persistent = (int64_t)sm_count() * 8;
    if (grid > persistent) grid = persistent;
    spmm_rows_kernel<T, NI, IdxT><<<(unsigned)grid, SPMM_THREADS, 0, a.st>>>(
        a.nrows, a.row_ids, a.pos, (const IdxT *)a.crd, a.val, a.b, a.ldb, a.c, a.ldc, a.k,
        a.slice_cols, row_blocks, a.accumulate, a.pair, a.hdr, a.chunks, a.chunk_cap);
    CB_LAUNCH_CHECK();
    if (a.nnz > SPMM_LONG_ROW) {   // otherwise no row can be long
        unsigned g2 = (unsigned)sm_count() * 8;
        spmm_chunks_kernel<T, NI, IdxT><<<g2, SPMM_THREADS, 0, a.st>>>(
            a.row_ids, a.pos, (const IdxT *)a.crd, a.val, a.b, a.ldb, a.c, a.ldc, a.k, a.slice_cols,
            a.nslices, a.pair, a.hdr, a.chunks, a.chunk_cap);
        CB_LAUNCH_CHECK();
    }
    return 0;
}

template <typename IdxT>
static int dispatch_panels(const SpmmArgs &a, int t, int ni)
{
#define CASE(TT, NN) if (t == TT && ni == NN) return launch_panels<TT, NN, IdxT>(a)
    CASE(2, 1); CASE(2, 2); CASE(2, 4);
    CASE(4, 1); CASE(4, 2); CASE(4, 4);
    CASE(8, 1); CASE(8, 2); CASE(8, 4);
    CASE(16, 1); CASE(16, 2); CASE(16, 4);
    CASE(32, 1); CASE(32, 2); CASE(32, 4);
#undef CASE
    return fail("spmm: no kernel for %d lanes x %d vectors per row", t, ni);
}

static int next_pow2(int v)
{
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

int spmm_rows(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k, const int64_t *row_ids,
              const int64_t *pos, const int64_t *crd, const double *val, const double *b,
              int64_t ldb, double *c, int64_t ldc, int semiring, int accumulate, int variant,
              cudaStream_t st)
{
    if (nrows <= 0 || k <= 0) return 0;
    int pair = semiring == COMET_B200_PLUS_PAIR;
    bool vec_ok = (k % 2 == 0) && (ldb % 2 == 0) && (ldc % 2 == 0) &&
                  ((((uintptr_t)b | (uintptr_t)c) & 15) == 0) && k <= (1 << 24);
    if (!vec_ok) {
        int64_t blocks = ceil_div(nrows * k, 256);
        int64_t cap = (int64_t)sm_count() * 32;
        if (blocks > cap) blocks = cap;
        spmm_scalar_kernel<<<(unsigned)blocks, 256, 0, st>>>(nrows, row_ids, pos, crd, val, b, ldb, c,
                                                           ldc, k, accumulate, pair);
        CB_LAUNCH_CHECK();
        return 0;
    }
    // bits 24-25 of the variant pick the path: 0 = by shape, 1 = entry stream (rows of B staged in shared memory by
    // cp.async), 2 = row panels, 3 = entry stream with the rows staged by TMA bulk copies (bit 26 in addition: one
    // tile::gather4 tensor copy per stage instead of one bulk copy per row)
    const int path = (variant >> 24) & 3;
    if (!pair && path == 3) {
        const int took = spmm_stream_tma(nrows, ncols, nnz, k, row_ids, pos, crd, val, b, ldb, c, ldc, accumulate,
                                         ((variant >> 26) & 1) != 0, st);
        if (took < 0) return -1;
        if (took > 0) return 0;
    }
    if (!pair && path != 2 && (path == 1 || spmm_stream_preferred(nrows, nnz, k))) {
        const int took = spmm_stream(nrows, ncols, nnz, k, row_ids, pos, crd, val, b, ldb, c, ldc, accumulate, path == 1, st);
        if (took < 0) return -1;
        if (took > 0) return 0;
    }
    // panel width W (columns per pass over A), lanes per row T, 128-bit vectors per lane NI
    int w = variant & 0xffff, t = (variant >> 16) & 0xff;
    if (w <= 0 || w > k) w = k > 256 ? 256 : (int)k;
    if (w % 2) w += 1;
    if (w > 256) w = 256;
    if (t == 0) {
        t = next_pow2((w + 1) / 2);
        if (t > 32) t = 32;
        if (t < 2) t = 2;
    }
    int ni = next_pow2((int)ceil_div(w, 2 * t));
    if (ni > 4) return fail("spmm: panel of %d columns needs more than 4 vectors per lane at %d lanes", w, t);
    int nslices = (int)ceil_div(k, w);

    SpmmArgs a;
    a.nrows = nrows; a.nnz = nnz; a.row_ids = row_ids; a.pos = pos; a.crd = crd; a.val = val;
    a.b = b; a.ldb = ldb; a.c = c; a.ldc = ldc; a.k = (int)k; a.slice_cols = w; a.nslices = nslices;
    a.accumulate = accumulate; a.pair = pair; a.st = st;

    size_t cap = (size_t)(nnz / SPMM_CHUNK + nnz / SPMM_LONG_ROW + 16);
    void *wl = nullptr;
    CB_TRY(scratch(SLOT_WORKLIST, sizeof(WorkHeader) + cap * sizeof(Chunk), &wl));
    a.hdr = (WorkHeader *)wl;
    a.chunks = (Chunk *)((char *)wl + sizeof(WorkHeader));
    a.chunk_cap = (unsigned)cap;
    CB_CUDA(cudaMemsetAsync(a.hdr, 0, sizeof(WorkHeader), st));

    bool narrow = nslices > 1 && ncols < 0x7fffffffLL && (((uintptr_t)crd & 15) == 0);
    if (narrow) {
        void *n32 = nullptr;
        CB_TRY(scratch(SLOT_NARROW_A, (size_t)nnz * sizeof(int32_t), &n32));
        CB_TRY(narrow_i64_to_i32(crd, (int32_t *)n32, nnz, st));
        a.crd = n32;
        return dispatch_panels<int32_t>(a, t, ni);
    }
    return dispatch_panels<int64_t>(a, t, ni);
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_spmm_f64_i64(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k,
                                               const int64_t *row_ids, const int64_t *pos,
                                               const int64_t *crd, const double *val,
                                               const double *b, int64_t ldb, double *c, int64_t ldc,
                                               int32_t semiring, int32_t accumulate, int32_t variant,
                                               void *stream)
{
    cb200::clear_error();
    if (semiring != COMET_B200_PLUS_TIMES && semiring != COMET_B200_PLUS_PAIR)
        return cb200::fail("spmm: unsupported semiring %d", semiring);
    if (ldb < k || ldc < k) return cb200::fail("spmm: leading dimension smaller than K");
    return cb200::spmm_rows(nrows, ncols, nnz, k, row_ids, pos, crd, val, b, ldb, c, ldc, semiring,
                            accumulate, variant, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// SpMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot tolerate a cudaMalloc inside the call: a
// COMET-generated program that runs with a fixed memory budget handed out at
// start-up, a serving loop that forbids anything that may synchronise the
// device, or an embedding runtime that owns the whole heap.  The regular entry
// point keeps its long-row work list in scratch memory that grows on demand;
// this variant keeps that list in a fixed array that is part of the loaded
// library image instead, so the call itself allocates nothing.
//
// The price is a size limit (the list holds NOALLOC_MAX_CHUNKS entries, which
// bounds the number of stored entries of A) and sharing: every call on a device
// uses the same array, which still holds the previous call's list when the next
// one starts.  The header is therefore cleared at the start of each call, and
// two calls that may overlap on the GPU (different streams) would corrupt each
// other's list and must be serialised by the caller.
// ---------------------------------------------------------------------------
namespace cb200 {

static const size_t NOALLOC_BYTES = (size_t)4 << 20;   // 4 MiB per device that loads the library
static const size_t NOALLOC_MAX_CHUNKS = (NOALLOC_BYTES - sizeof(WorkHeader)) / sizeof(Chunk);

// Device-side storage.  In host code this name only stands for the symbol; the
// address kernels can use is obtained with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_worklist[NOALLOC_BYTES];

static void *g_noalloc_addr[64] = {nullptr};   // per device, filled on first use

static int noalloc_worklist(void **out)
{
    int d = 0;
    CB_CUDA(cudaGetDevice(&d));
    if (d < 0 || d >= 64) return fail("spmm (no-alloc): device index %d out of range", d);
    if (!g_noalloc_addr[d]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_worklist);
        if (e != cudaSuccess || !p)
            return fail("spmm (no-alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        g_noalloc_addr[d] = p;
    }
    *out = g_noalloc_addr[d];
    return 0;
}

int spmm_rows_noalloc(int64_t nrows, int64_t nnz, int64_t k, const int64_t *row_ids,
                      const int64_t *pos, const int64_t *crd, const double *val, const double *b,
                      int64_t ldb, double *c, int64_t ldc, int semiring, int accumulate,
                      cudaStream_t st)
{
    if (nrows <= 0 || k <= 0) return 0;
    if (nnz < 0) return fail("spmm (no-alloc): negative nnz");
    const size_t need = (size_t)(nnz / SPMM_CHUNK + nnz / SPMM_LONG_ROW + 16);
    if (need > NOALLOC_MAX_CHUNKS)
        return fail("spmm (no-alloc): %lld stored entries need a work list of %zu chunks, the built-in "
                    "list holds %zu (about %lld entries); use comet_b200_dev_spmm_f64_i64",
                    (long long)nnz, need, NOALLOC_MAX_CHUNKS,
                    (long long)((NOALLOC_MAX_CHUNKS - 16) * SPMM_CHUNK / 2));
    if (k % 2 != 0 || ldb % 2 != 0 || ldc % 2 != 0 || ((((uintptr_t)b | (uintptr_t)c) & 15) != 0))
        return fail("spmm (no-alloc): K and both leading dimensions must be even and B, C 16-byte aligned");
    if (k > 256) return fail("spmm (no-alloc): at most 256 columns per call (got %lld)", (long long)k);
    void *wl = nullptr;
    CB_TRY(noalloc_worklist(&wl));

    int w = (int)k;
    int t = next_pow2((w + 1) / 2);
    if (t > 32) t = 32;
    if (t < 2) t = 2;
    int ni = next_pow2((int)ceil_div(w, 2 * t));

    SpmmArgs a;
    a.nrows = nrows; a.nnz = nnz; a.row_ids = row_ids; a.pos = pos; a.crd = crd; a.val = val;
    a.b = b; a.ldb = ldb; a.c = c; a.ldc = ldc; a.k = (int)k; a.slice_cols = w; a.nslices = 1;
    a.accumulate = accumulate; a.pair = semiring == COMET_B200_PLUS_PAIR; a.st = st;
    a.hdr = (WorkHeader *)wl;
    a.chunks = (Chunk *)((char *)wl + sizeof(WorkHeader));
    a.chunk_cap = (unsigned)NOALLOC_MAX_CHUNKS;
    // the array keeps the previous call's list: the count has to start at zero
    CB_CUDA(cudaMemsetAsync(a.hdr, 0, sizeof(WorkHeader), st));
    return dispatch_panels<int64_t>(a, t, ni);
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_spmm_noalloc_f64_i64(int64_t nrows, int64_t nnz, int64_t k,
                                                       const int64_t *row_ids, const int64_t *pos,
                                                       const int64_t *crd, const double *val,
                                                       const double *b, int64_t ldb, double *c,
                                                       int64_t ldc, int32_t semiring,
                                                       int32_t accumulate, void *stream)
{
    cb200::clear_error();
    if (semiring != COMET_B200_PLUS_TIMES && semiring != COMET_B200_PLUS_PAIR)
        return cb200::fail("spmm (no-alloc): unsupported semiring %d", semiring);
    if (ldb < k || ldc < k) return cb200::fail("spmm (no-alloc): leading dimension smaller than K");
    return cb200::spmm_rows_noalloc(nrows, nnz, k, row_ids, pos, crd, val, b, ldb, c, ldc, semiring,
                                    accumulate, (cudaStream_t)stream);
}
