// SDDMM  out[p] = S.val[p] * sum_k X[i,k] * Y[j,k]   for every stored (i,j) of S (CSR).
//
// Two launches share the work by row length.
//   rows of at most LONG_ROW entries: warps draw blocks of BLOCK_ROWS consecutive rows from a
//     counter and walk the block's entries as ONE stream, 32 entries per batch; the row of every
//     entry is found once per batch by a shuffle binary search over the block's row pointers, the
//     next batch's coordinates are fetched before the current one is worked on, and groups of G
//     lanes gather X[i,:] and Y[j,:] with 128-bit loads and finish each dot product with
//     xor-shuffles.  The 32 results of a batch are scaled by S.val and leave in one coalesced store.
//   longer rows: cut into CHUNK-entry pieces on a work list in scratch memory by the first launch;
//     the second launch gives every piece to a warp that keeps X[i,:] in registers.  On power-law
//     matrices this balanced path carries most of the entries.
//
// Bound: HBM.  Algorithmic bytes = 8(n+1) + 24 nnz + 8 K (nrows + ncols).
#include "common.cuh"

namespace cb200 {

static const int SDDMM_THREADS = 256;
static const int64_t SDDMM_LONG_ROW = 32;
static const int64_t SDDMM_CHUNK = 64;
static const int SDDMM_BLOCK_ROWS = 8;     // consecutive rows a warp draws at a time (power of two <= 32)

// Entries [s, e) of row `row`; xr holds this lane's part of X[row,:].
template <int G, int NI>
__device__ __forceinline__ void sample_range(const double2 (&xr)[NI], const int64_t *__restrict__ crd,
                                             const double *__restrict__ sval,
                                             const double *__restrict__ y, int64_t ldy,
                                             double *__restrict__ out, int64_t s, int64_t e, int lane,
                                             int k2)
{
    constexpr int P = 32 / G;                 // entries in flight per step
    const int g = lane / G, l = lane % G;
    for (int64_t base = s; base < e; base += 32) {
        const int64_t p = base + lane;
        int64_t c = 0;
        if (p < e) c = ld_stream(crd + p);
        const int n = (e - base) < 32 ? (int)(e - base) : 32;
        double mine = 0.0;
        const int steps = (n + P - 1) / P;
#pragma unroll 2
        for (int t = 0; t < steps; t++) {
            const int idx = t * P + g;        // entry of this batch handled by my group
            const int64_t cc = __shfl_sync(0xffffffffu, (long long)c, idx & 31);
            double d0 = 0.0, d1 = 0.0;
            if (idx < n) {
                const double2 *yr = (const double2 *)(y + cc * ldy);
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    if (l + i * G < k2) {
                        double2 yy = __ldg(yr + l + i * G);
                        d0 = fma(xr[i].x, yy.x, d0);
                        d1 = fma(xr[i].y, yy.y, d1);
                    }
                }
            }
            double d = d0 + d1;
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            // a batch has at most 32 / P = G steps, so lane l == t of each group can keep step t's result
            if (l == t) mine = d;
        }
        // lane (g, l) now holds the result of batch entry l*P + g: a permutation of the batch,
        // so the store below is one coalesced 256-byte write per warp
        const int idx = l * P + g;
        if (idx < n) out[base + idx] = ld_stream(sval + base + idx) * mine;
    }
}

template <int G, int NI>
__device__ __forceinline__ void load_x(double2 (&xr)[NI], const double *__restrict__ x, int64_t ldx,
                                       int64_t row, int l, int k2)
{
    const double2 *xp = (const double2 *)(x + row * ldx);
#pragma unroll
    for (int i = 0; i < NI; i++)
        xr[i] = (l + i * G < k2) ? __ldg(xp + l + i * G) : make_double2(0.0, 0.0);
}

// Entries [a, b) of a run of consecutive rows, as one stream: a batch of 32
// consecutive entries may span several rows, so each entry carries its row
// (found once per batch by a shuffle binary search over the 32 row pointers the
// lanes hold) and X[row,:] is read through L1 next to Y[col,:].  The next
// batch's coordinates and rows are fetched before the current batch is worked
// on, so no load depends on another one inside the loop.
template <int G, int NI>
__device__ __forceinline__ void sample_stream(int64_t row0, int64_t rp, const int64_t *__restrict__ crd,
                                              const double *__restrict__ sval,
                                              const double *__restrict__ x, int64_t ldx,
                                              const double *__restrict__ y, int64_t ldy,
                                              double *__restrict__ out, int64_t a, int64_t b, int lane,
                                              int k2)
{
    constexpr int P = 32 / G;
    const int g = lane / G, l = lane % G;
    auto fetch = [&](int64_t base, int64_t &c, int &row) {
        const int64_t p = base + lane;
        c = 0;
        if (p < b) c = ld_stream(crd + p);
        // last t in [0, BLOCK_ROWS) with pos[row0 + t] <= p  (rp = this lane's row pointer)
        int lo = 0;
#pragma unroll
        for (int step = SDDMM_BLOCK_ROWS / 2; step > 0; step >>= 1) {
            const int64_t v = __shfl_sync(0xffffffffu, (long long)rp, lo + step);
            if (v <= p) lo += step;
        }
        row = lo;
    };
    int64_t c_next;
    int row_next;
    fetch(a, c_next, row_next);
    for (int64_t base = a; base < b; base += 32) {
        const int64_t c = c_next;
        const int row = row_next;
        if (base + 32 < b) fetch(base + 32, c_next, row_next);
        const int n = (b - base) < 32 ? (int)(b - base) : 32;
        const int steps = (n + P - 1) / P;
        double mine = 0.0;
#pragma unroll 2
        for (int t = 0; t < steps; t++) {
            const int idx = t * P + g;
            const int64_t cc = __shfl_sync(0xffffffffu, (long long)c, idx & 31);
            const int rr = __shfl_sync(0xffffffffu, row, idx & 31);
            double d0 = 0.0, d1 = 0.0;
            if (idx < n) {
                const double2 *yr = (const double2 *)(y + cc * ldy);
                const double2 *xp = (const double2 *)(x + (row0 + rr) * ldx);
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    if (l + i * G < k2) {
                        const double2 yy = __ldg(yr + l + i * G);
                        const double2 xx = __ldg(xp + l + i * G);
                        d0 = fma(xx.x, yy.x, d0);
                        d1 = fma(xx.y, yy.y, d1);
                    }
                }
            }
            double d = d0 + d1;
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (l == t) mine = d;
        }
        const int idx = l * P + g;
        if (idx < n) out[base + idx] = ld_stream(sval + base + idx) * mine;
    }
}

// Warps draw blocks of SDDMM_BLOCK_ROWS consecutive rows from a counter and walk each block's
// entries as a stream; rows longer than LONG_ROW are cut out of the stream and
// go to the chunk list.
template <int G, int NI>
__global__ void __launch_bounds__(SDDMM_THREADS)
sddmm_rows_kernel(int64_t nrows, const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                  const double *__restrict__ sval, const double *__restrict__ x, int64_t ldx,
                  const double *__restrict__ y, int64_t ldy, double *__restrict__ out, int k,
                  WorkHeader *hdr, Chunk *chunks, unsigned chunk_cap)
{
    const int lane = threadIdx.x & 31;
    const int k2 = k / 2;
    const int64_t nblocks = (nrows + SDDMM_BLOCK_ROWS - 1) / SDDMM_BLOCK_ROWS;
    while (true) {
        unsigned blk = 0;
        if (lane == 0) blk = atomicAdd(&hdr->pad[0], 1u);
        blk = __shfl_sync(0xffffffffu, blk, 0);
        if ((int64_t)blk >= nblocks) break;
        const int64_t row0 = (int64_t)blk * SDDMM_BLOCK_ROWS;
        const int nr = (nrows - row0) < SDDMM_BLOCK_ROWS ? (int)(nrows - row0) : SDDMM_BLOCK_ROWS;
        const int64_t rp = pos[row0 + (lane < nr ? lane : nr)];      // lanes past the block hold its end
        const int64_t rnext = pos[row0 + (lane < nr ? lane + 1 : nr)];
        const bool is_long = lane < nr && (rnext - rp) > SDDMM_LONG_ROW;
        if (is_long) {
            unsigned n = (unsigned)((rnext - rp + SDDMM_CHUNK - 1) / SDDMM_CHUNK);
            unsigned at = atomicAdd(&hdr->count, n);
            if (at + n <= chunk_cap) {
                for (unsigned i = 0; i < n; i++) {
                    chunks[at + i].row = row0 + lane;
                    chunks[at + i].begin = rp + (int64_t)i * SDDMM_CHUNK;
                }
            } else {
                hdr->overflow = 1;
            }
        }
        const unsigned longmask = __ballot_sync(0xffffffffu, is_long);
        int t0 = 0;
        while (t0 < nr) {
            const unsigned m = longmask >> t0;
            const int run = m ? (__ffs(m) - 1) : (nr - t0);      // rows [t0, t0 + run) hold no long row
            if (run > 0) {
                const int64_t a = __shfl_sync(0xffffffffu, (long long)rp, t0);
                const int last = t0 + run - 1;
                const int64_t b = __shfl_sync(0xffffffffu, (long long)rnext, last);
                if (b > a) sample_stream<G, NI>(row0, rp, crd, sval, x, ldx, y, ldy, out, a, b, lane, k2);
            }
            t0 += run + 1;
        }
    }
}

template <int G, int NI>
__global__ void __launch_bounds__(SDDMM_THREADS)
sddmm_chunks_kernel(const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                    const double *__restrict__ sval, const double *__restrict__ x, int64_t ldx,
                    const double *__restrict__ y, int64_t ldy, double *__restrict__ out, int k,
                    const WorkHeader *hdr, const Chunk *chunks, unsigned chunk_cap)
{
    const int lane = threadIdx.x & 31;
    const int k2 = k / 2;
    const unsigned warp = (blockIdx.x * SDDMM_THREADS + threadIdx.x) >> 5;
    const unsigned nwarps = (gridDim.x * SDDMM_THREADS) >> 5;
    unsigned count = hdr->count;
    if (count > chunk_cap) count = 0;
    for (unsigned w = warp; w < count; w += nwarps) {
        const Chunk ch = chunks[w];
        int64_t cend = pos[ch.row + 1];
        if (cend > ch.begin + SDDMM_CHUNK) cend = ch.begin + SDDMM_CHUNK;
        double2 xr[NI];
        load_x<G, NI>(xr, x, ldx, ch.row, lane % G, k2);
        sample_range<G, NI>(xr, crd, sval, y, ldy, out, ch.begin, cend, lane, k2);
    }
}

// Any K and alignment: one thread per row (correctness path).
__global__ void __launch_bounds__(256)
sddmm_scalar_kernel(int64_t nrows, const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                    const double *__restrict__ sval, const double *__restrict__ x, int64_t ldx,
                    const double *__restrict__ y, int64_t ldy, double *__restrict__ out, int64_t k)
{
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < nrows;
         r += (int64_t)gridDim.x * blockDim.x) {
        for (int64_t p = pos[r]; p < pos[r + 1]; p++) {
            const double *xr = x + r * ldx, *yr = y + crd[p] * ldy;
            double t = 0.0;
            for (int64_t kk = 0; kk < k; kk++) t = fma(xr[kk], yr[kk], t);
            out[p] = sval[p] * t;
        }
    }
}

template <int G, int NI>
static int launch_sddmm(int64_t nrows, int64_t nnz, const int64_t *pos, const int64_t *crd,
                        const double *sval, const double *x, int64_t ldx, const double *y,
                        int64_t ldy, double *out, int k, WorkHeader *hdr, Chunk *chunks,
                        unsigned cap, cudaStream_t st)
{
    int64_t grid = ceil_div(nrows, SDDMM_THREADS / 32);
    const int64_t full = (int64_t)sm_count() * 16;
    if (grid > full) grid = full;
    sddmm_rows_kernel<G, NI><<<(unsigned)grid, SDDMM_THREADS, 0, st>>>(nrows, pos, crd, sval, x, ldx, y, ldy,
                                                                     out, k, hdr, chunks, cap);
    CB_LAUNCH_CHECK();
    if (nnz > SDDMM_LONG_ROW) {
        sddmm_chunks_kernel<G, NI><<<(unsigned)sm_count() * 8, SDDMM_THREADS, 0, st>>>(
            pos, crd, sval, x, ldx, y, ldy, out, k, hdr, chunks, cap);
        CB_LAUNCH_CHECK();
    }
    return 0;
}

int sddmm_csr(int64_t nrows, int64_t nnz, int64_t k, const int64_t *pos, const int64_t *crd,
              const double *sval, const double *x, int64_t ldx, const double *y, int64_t ldy,
              double *out, cudaStream_t st)
{
    if (nrows <= 0 || nnz <= 0) return 0;
    bool vec_ok = k > 0 && k % 2 == 0 && k <= 256 && ldx % 2 == 0 && ldy % 2 == 0 &&
                  ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
    if (!vec_ok) {
        int64_t blocks = ceil_div(nrows, 256);
        sddmm_scalar_kernel<<<(unsigned)blocks, 256, 0, st>>>(nrows, pos, crd, sval, x, ldx, y, ldy, out, k);
        CB_LAUNCH_CHECK();
        return 0;
    }
    size_t cap = (size_t)(nnz / SDDMM_CHUNK + nnz / SDDMM_LONG_ROW + 16);
    void *wl = nullptr;
    CB_TRY(scratch(SLOT_WORKLIST, sizeof(WorkHeader) + cap * sizeof(Chunk), &wl));
    WorkHeader *hdr = (WorkHeader *)wl;
    Chunk *chunks = (Chunk *)((char *)wl + sizeof(WorkHeader));
    CB_CUDA(cudaMemsetAsync(hdr, 0, sizeof(WorkHeader), st));
#define GO(GG, NN) return launch_sddmm<GG, NN>(nrows, nnz, pos, crd, sval, x, ldx, y, ldy, out, (int)k, hdr, chunks, (unsigned)cap, st)
    if (k <= 8) GO(1, 4);
    if (k <= 16) GO(2, 4);
    if (k <= 32) GO(4, 4);
    if (k <= 64) GO(8, 4);
    if (k <= 128) GO(16, 4);
    GO(32, 4);
#undef GO
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_sddmm_f64_i64(int64_t nrows, int64_t nnz, int64_t k,
                                                const int64_t *pos, const int64_t *crd,
                                                const double *sval, const double *x, int64_t ldx,
                                                const double *y, int64_t ldy, double *out,
                                                void *stream)
{
    cb200::clear_error();
    if (ldx < k || ldy < k) return cb200::fail("sddmm: leading dimension smaller than K");
    return cb200::sddmm_csr(nrows, nnz, k, pos, crd, sval, x, ldx, y, ldy, out, (cudaStream_t)stream);
}
