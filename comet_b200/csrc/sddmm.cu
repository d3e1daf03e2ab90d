// SDDMM  out[p] = S.val[p] * sum_k X[i,k] * Y[j,k]   for every stored (i,j) of S (CSR).
//
// A group of G lanes owns one row i: it keeps its part of X[i,:] in registers
// (2*NI doubles per lane), loads G column coordinates at a time with one
// coalesced streaming load, and for each of them gathers Y[j,:] with 128-bit
// loads, multiplies, and finishes the dot product with xor-shuffles inside the
// group.  The G results of a batch are written with one coalesced store.
// Rows longer than LONG_ROW entries go through the chunk work list (scratch
// memory) and a second launch where a whole CTA shares one chunk.
//
// Bound: HBM.  Algorithmic bytes = 8(n+1) + 24 nnz + 8 K (nrows + ncols).
#include "common.cuh"

namespace cb200 {

static const int SDDMM_THREADS = 256;
static const int SDDMM_PASSES = 2;
static const int64_t SDDMM_LONG_ROW = 512;
static const int64_t SDDMM_CHUNK = 512;

template <int G, int NI>
__device__ __forceinline__ void sample_range(const double2 (&xr)[NI], const int64_t *__restrict__ crd,
                                             const double *__restrict__ sval,
                                             const double *__restrict__ y, int64_t ldy,
                                             double *__restrict__ out, int64_t s, int64_t e, int l,
                                             unsigned gmask, int k2)
{
    for (int64_t base = s; base < e; base += G) {
        int64_t p = base + l;
        int64_t c = 0;
        if (p < e) c = ld_stream(crd + p);
        int n = (e - base) < G ? (int)(e - base) : G;
        double mine = 0.0;
#pragma unroll 2
        for (int t = 0; t < n; t++) {
            int64_t cc = __shfl_sync(gmask, (long long)c, t, G);
            const double2 *yr = (const double2 *)(y + cc * ldy);
            double d0 = 0.0, d1 = 0.0;
#pragma unroll
            for (int i = 0; i < NI; i++) {
                if (l + i * G < k2) {
                    double2 yy = __ldg(yr + l + i * G);
                    d0 = fma(xr[i].x, yy.x, d0);
                    d1 = fma(xr[i].y, yy.y, d1);
                }
            }
            double d = d0 + d1;
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) d += __shfl_xor_sync(gmask, d, o, G);
            if (l == t) mine = d;
        }
        if (p < e) out[p] = ld_stream(sval + p) * mine;
    }
}

template <int G, int NI>
__device__ __forceinline__ void load_x(double2 (&xr)[NI], const double *__restrict__ x, int64_t ldx,
                                       int64_t row, int l, int k2)
{
    const double2 *xp = (const double2 *)(x + row * ldx);
#pragma unroll
    for (int i = 0; i < NI; i++)
        xr[i] = (l + i * G < k2) ? xp[l + i * G] : make_double2(0.0, 0.0);
}

template <int G, int NI>
__global__ void __launch_bounds__(SDDMM_THREADS)
sddmm_rows_kernel(int64_t nrows, const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                  const double *__restrict__ sval, const double *__restrict__ x, int64_t ldx,
                  const double *__restrict__ y, int64_t ldy, double *__restrict__ out, int k,
                  WorkHeader *hdr, Chunk *chunks, unsigned chunk_cap)
{
    constexpr int GROUPS = SDDMM_THREADS / G;
    constexpr int ROWS = GROUPS * SDDMM_PASSES;
    const int g = threadIdx.x / G, l = threadIdx.x % G;
    const int lane = threadIdx.x & 31;
    const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int k2 = k / 2;
    const int64_t row0 = (int64_t)blockIdx.x * ROWS;
    for (int pass = 0; pass < SDDMM_PASSES; pass++) {
        int64_t r = row0 + pass * GROUPS + g;
        if (r >= nrows) break;
        int64_t s = pos[r], e = pos[r + 1];
        if (s == e) continue;
        if (e - s > SDDMM_LONG_ROW) {
            if (l == 0) {
                unsigned n = (unsigned)((e - s + SDDMM_CHUNK - 1) / SDDMM_CHUNK);
                unsigned at = atomicAdd(&hdr->count, n);
                if (at + n <= chunk_cap) {
                    for (unsigned i = 0; i < n; i++) {
                        chunks[at + i].row = r;
                        chunks[at + i].begin = s + (int64_t)i * SDDMM_CHUNK;
                    }
                } else {
                    hdr->overflow = 1;
                }
            }
            continue;
        }
        double2 xr[NI];
        load_x<G, NI>(xr, x, ldx, r, l, k2);
        sample_range<G, NI>(xr, crd, sval, y, ldy, out, s, e, l, gmask, k2);
    }
}

template <int G, int NI>
__global__ void __launch_bounds__(SDDMM_THREADS)
sddmm_chunks_kernel(const int64_t *__restrict__ pos, const int64_t *__restrict__ crd,
                    const double *__restrict__ sval, const double *__restrict__ x, int64_t ldx,
                    const double *__restrict__ y, int64_t ldy, double *__restrict__ out, int k,
                    const WorkHeader *hdr, const Chunk *chunks, unsigned chunk_cap)
{
    constexpr int GROUPS = SDDMM_THREADS / G;
    const int g = threadIdx.x / G, l = threadIdx.x % G;
    const int lane = threadIdx.x & 31;
    const unsigned gmask = (G == 32) ? 0xffffffffu : (((1u << G) - 1u) << (lane & ~(G - 1)));
    const int k2 = k / 2;
    unsigned count = hdr->count;
    if (count > chunk_cap) count = 0;
    for (unsigned w = blockIdx.x; w < count; w += gridDim.x) {
        const Chunk ch = chunks[w];
        int64_t cend = pos[ch.row + 1];
        if (cend > ch.begin + SDDMM_CHUNK) cend = ch.begin + SDDMM_CHUNK;
        // contiguous sub-ranges whose length is a multiple of G keep the stores coalesced
        int64_t per = (cend - ch.begin + GROUPS - 1) / GROUPS;
        per = (per + G - 1) / G * G;
        int64_t s = ch.begin + (int64_t)g * per, e = s + per;
        if (e > cend) e = cend;
        if (s < e) {
            double2 xr[NI];
            load_x<G, NI>(xr, x, ldx, ch.row, l, k2);
            sample_range<G, NI>(xr, crd, sval, y, ldy, out, s, e, l, gmask, k2);
        }
    }
}

// Any K and alignment: one thread per stored entry (correctness path).
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
    constexpr int ROWS = (SDDMM_THREADS / G) * SDDMM_PASSES;
    unsigned grid = (unsigned)ceil_div(nrows, ROWS);
    sddmm_rows_kernel<G, NI><<<grid, SDDMM_THREADS, 0, st>>>(nrows, pos, crd, sval, x, ldx, y, ldy, out,
                                                           k, hdr, chunks, cap);
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
