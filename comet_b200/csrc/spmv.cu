// SpMV  y[a] = y[a] (+) sum_b A[a,b] (x) x[b]   (CSR / DCSR rows, f64 values, i64 indices).
//
// A group of T lanes (T chosen from the mean row length) walks one row with
// 128-bit loads of crd and val (two entries per load).
// Small matrices (< 2^20 stored entries): one launch, no scratch memory; rows
// longer than LONG_ROW entries are left to the end of the CTA, where all 256
// threads walk each of them together; the summation order per row is fixed.
// Larger matrices: rows longer than DEFER_ROW entries are cut into chunks that
// go to a work list in scratch memory, and a second launch gives each chunk to
// a warp that adds its partial sum to y with one f64 atomic -- on a power-law
// matrix the long rows sit next to each other and would otherwise all land in
// the first few CTAs.
//
// Bound: HBM.  Algorithmic bytes per call = 8(n+1) + 16 nnz + 8 ncols + 8 nrows.
#include "common.cuh"

namespace cb200 {

static const int SPMV_THREADS = 256;
static const int SPMV_PASSES = 4;          // most rows per lane group per CTA (fewer on small matrices)
static const int64_t LONG_ROW = 2048;
static const int64_t DEFER_ROW = 64;       // with a work list: rows above this go to it
static const int64_t SPMV_CHUNK = 256;     // entries per work-list chunk
static const int64_t DEFER_MIN_NNZ = 1 << 20;

template <bool PAIR>
__device__ __forceinline__ double combine(double a, double b)
{
    return PAIR ? 1.0 : a * b;
}

// Partial dot product of one row over entries handled by this lane; `nl` lanes
// share the row, lane index `l`.  VEC: crd/val are 16-byte aligned arrays.
template <bool PAIR, bool VEC>
__device__ __forceinline__ double row_partial(const int64_t *__restrict__ crd,
                                              const double *__restrict__ val,
                                              const double *__restrict__ x, int64_t s, int64_t e,
                                              int l, int nl)
{
    double sum0 = 0.0, sum1 = 0.0;
    if (VEC) {
        for (int64_t q = (s & ~(int64_t)1) + 2 * l; q < e; q += 2 * nl) {
            if (q >= s && q + 1 < e) {
                longlong2 c = __ldcs((const longlong2 *)(crd + q));
                double2 v = __ldcs((const double2 *)(val + q));
                sum0 += combine<PAIR>(v.x, PAIR ? 0.0 : __ldg(x + c.x));
                sum1 += combine<PAIR>(v.y, PAIR ? 0.0 : __ldg(x + c.y));
            } else {
                if (q >= s) sum0 += combine<PAIR>(val[q], PAIR ? 0.0 : __ldg(x + crd[q]));
                if (q + 1 < e) sum1 += combine<PAIR>(val[q + 1], PAIR ? 0.0 : __ldg(x + crd[q + 1]));
            }
        }
    } else {
        for (int64_t q = s + l; q < e; q += nl)
            sum0 += combine<PAIR>(val[q], PAIR ? 0.0 : __ldg(x + crd[q]));
    }
    return sum0 + sum1;
}

template <int T, bool PAIR, bool VEC>
__global__ void __launch_bounds__(SPMV_THREADS)
spmv_kernel(int64_t nrows, const int64_t *__restrict__ row_ids, const int64_t *__restrict__ pos,
            const int64_t *__restrict__ crd, const double *__restrict__ val,
            const double *__restrict__ x, double *__restrict__ y, int accumulate, int passes,
            WorkHeader *hdr, Chunk *chunks, unsigned chunk_cap)
{
    constexpr int GROUPS = SPMV_THREADS / T;
    constexpr int ROWS = GROUPS * SPMV_PASSES;
    __shared__ int64_t long_rows[ROWS];
    __shared__ int n_long;
    __shared__ double warp_part[SPMV_THREADS / 32];

    const int g = threadIdx.x / T, l = threadIdx.x % T;
    const int lane = threadIdx.x & 31;
    const unsigned gmask = (T == 32) ? 0xffffffffu : (((1u << T) - 1u) << (lane & ~(T - 1)));
    if (threadIdx.x == 0) n_long = 0;
    // Programmatic dependent launch: when the launch carries that attribute this grid may be set up while the
    // kernel before it in the stream is still running; nothing that kernel may have written (x, y, even A) is
    // touched before the wait, and the next kernel in the stream is allowed to set up from here on.  Without
    // the attribute both instructions do nothing.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();

    const int64_t row0 = (int64_t)blockIdx.x * (GROUPS * passes);
    for (int pass = 0; pass < passes; pass++) {
        int64_t r = row0 + pass * GROUPS + g;
        if (r >= nrows) break;
        int64_t s = pos[r], e = pos[r + 1];
        if (hdr && e - s > DEFER_ROW) {
            if (l == 0) {
                const unsigned n = (unsigned)((e - s + SPMV_CHUNK - 1) / SPMV_CHUNK);
                const unsigned at = atomicAdd(&hdr->count, n);
                if (at + n <= chunk_cap) {
                    for (unsigned i = 0; i < n; i++) {
                        chunks[at + i].row = r;
                        chunks[at + i].begin = s + (int64_t)i * SPMV_CHUNK;
                    }
                    if (!accumulate) y[row_ids ? row_ids[r] : r] = 0.0;     // the chunks add into it
                    continue;
                }
                hdr->overflow = 1;
            }
            // all lanes of the group must agree: the list cannot overflow (its capacity is a bound),
            // so a deferred row is always skipped here
            continue;
        }
        if (e - s > LONG_ROW) {
            if (l == 0) long_rows[atomicAdd(&n_long, 1)] = r;
            continue;
        }
        double sum = row_partial<PAIR, VEC>(crd, val, x, s, e, l, T);
#pragma unroll
        for (int o = T / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(gmask, sum, o, T);
        if (l == 0) {
            int64_t out = row_ids ? row_ids[r] : r;
            y[out] = accumulate ? y[out] + sum : sum;
        }
    }
    __syncthreads();
    const int nl = n_long;
    for (int i = 0; i < nl; i++) {
        int64_t r = long_rows[i];
        double sum = row_partial<PAIR, VEC>(crd, val, x, pos[r], pos[r + 1], threadIdx.x, SPMV_THREADS);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) warp_part[threadIdx.x >> 5] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < SPMV_THREADS / 32; w++) t += warp_part[w];
            int64_t out = row_ids ? row_ids[r] : r;
            y[out] = accumulate ? y[out] + t : t;
        }
        __syncthreads();
    }
}

template <bool PAIR, bool VEC>
__global__ void __launch_bounds__(SPMV_THREADS)
spmv_chunks_kernel(const int64_t *__restrict__ row_ids, const int64_t *__restrict__ pos,
                   const int64_t *__restrict__ crd, const double *__restrict__ val,
                   const double *__restrict__ x, double *__restrict__ y, const WorkHeader *hdr,
                   const Chunk *chunks, unsigned chunk_cap)
{
    const int lane = threadIdx.x & 31;
    const unsigned warp = (blockIdx.x * SPMV_THREADS + threadIdx.x) >> 5;
    const unsigned nwarps = (gridDim.x * SPMV_THREADS) >> 5;
    unsigned count = hdr->count;
    if (count > chunk_cap) count = 0;
    for (unsigned w = warp; w < count; w += nwarps) {
        const Chunk ch = chunks[w];
        int64_t e = pos[ch.row + 1];
        if (e > ch.begin + SPMV_CHUNK) e = ch.begin + SPMV_CHUNK;
        double sum = row_partial<PAIR, VEC>(crd, val, x, ch.begin, e, lane, 32);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == 0) atomicAdd(y + (row_ids ? row_ids[ch.row] : ch.row), sum);
    }
}

template <int T>
static int launch_spmv(int64_t nrows, const int64_t *row_ids, const int64_t *pos, const int64_t *crd,
                       const double *val, const double *x, double *y, bool pair, bool vec,
                       int accumulate, int64_t nnz, cudaStream_t st)
{
    WorkHeader *hdr = nullptr;
    Chunk *chunks = nullptr;
    size_t cap = 0;
    if (nnz >= DEFER_MIN_NNZ) {
        cap = (size_t)(nnz / SPMV_CHUNK + nnz / DEFER_ROW + 16);
        void *wl = nullptr;
        CB_TRY(scratch(SLOT_WORKLIST, sizeof(WorkHeader) + cap * sizeof(Chunk), &wl));
        hdr = (WorkHeader *)wl;
        chunks = (Chunk *)((char *)wl + sizeof(WorkHeader));
        CB_CUDA(cudaMemsetAsync(hdr, 0, sizeof(WorkHeader), st));
    }
    // small matrices: fewer rows per CTA so that the grid still covers every SM a few times
    constexpr int GROUPS = SPMV_THREADS / T;
    int passes = SPMV_PASSES;
    while (passes > 1 && ceil_div(nrows, (int64_t)GROUPS * passes) < (int64_t)sm_count() * 4) passes--;
    unsigned grid = (unsigned)ceil_div(nrows, (int64_t)GROUPS * passes);
    // One-launch calls (no chunk list) are a few microseconds long.  With COMET_B200_SPMV_PDL=1 they are launched
    // with programmatic stream serialization, which lets the next grid be set up under the tail of this one.
    // Off by default: measured on B200 in a CUDA graph of back-to-back calls (16384 rows x 16) it gave 3.49 against
    // 3.89 us per call at 10 calls and 4.04 against 3.56 us at 1000, so nothing consistent; the empty-kernel floor of
    // the same graphs is 0.73 us per launch, the rest is the kernel's own chain of dependent loads.
    static const bool pdl = [] { const char *e = getenv("COMET_B200_SPMV_PDL"); return e && e[0] == '1'; }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(SPMV_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (pdl && !hdr) ? 1 : 0;
    const unsigned ucap = (unsigned)cap;
#define GO(P, V) CB_CUDA(cudaLaunchKernelEx(&cfg, spmv_kernel<T, P, V>, nrows, row_ids, pos, crd, val, x, y, accumulate, passes, hdr, chunks, ucap))
    if (pair) { if (vec) GO(true, true); else GO(true, false); }
    else      { if (vec) GO(false, true); else GO(false, false); }
#undef GO
    CB_LAUNCH_CHECK();
    if (hdr) {
        const unsigned g2 = (unsigned)sm_count() * 8;
#define GO2(P, V) spmv_chunks_kernel<P, V><<<g2, SPMV_THREADS, 0, st>>>(row_ids, pos, crd, val, x, y, hdr, chunks, (unsigned)cap)
        if (pair) { if (vec) GO2(true, true); else GO2(true, false); }
        else      { if (vec) GO2(false, true); else GO2(false, false); }
#undef GO2
        CB_LAUNCH_CHECK();
    }
    return 0;
}

int spmv_rows(int64_t nrows, int64_t nnz, const int64_t *row_ids, const int64_t *pos,
              const int64_t *crd, const double *val, const double *x, double *y, int semiring,
              int accumulate, cudaStream_t st)
{
    if (nrows <= 0) return 0;
    bool vec = (((uintptr_t)crd | (uintptr_t)val) & 15) == 0;
    bool pair = semiring == COMET_B200_PLUS_PAIR;
    double mean = (double)nnz / (double)nrows;
    if (const char *env = getenv("COMET_B200_SPMV_LANES")) {        // tuning knob: lanes per row
        const int t = atoi(env);
        if (t == 2) mean = 4.0; else if (t == 4) mean = 8.0; else if (t == 8) mean = 24.0;
        else if (t == 16) mean = 48.0; else if (t == 32) mean = 1e9;
    }
    if (mean <= 4.0) return launch_spmv<2>(nrows, row_ids, pos, crd, val, x, y, pair, vec, accumulate, nnz, st);
    if (mean <= 8.0) return launch_spmv<4>(nrows, row_ids, pos, crd, val, x, y, pair, vec, accumulate, nnz, st);
    if (mean <= 24.0) return launch_spmv<8>(nrows, row_ids, pos, crd, val, x, y, pair, vec, accumulate, nnz, st);
    if (mean <= 48.0) return launch_spmv<16>(nrows, row_ids, pos, crd, val, x, y, pair, vec, accumulate, nnz, st);
    return launch_spmv<32>(nrows, row_ids, pos, crd, val, x, y, pair, vec, accumulate, nnz, st);
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_spmv_f64_i64(int64_t nrows, int64_t nnz, const int64_t *row_ids,
                                               const int64_t *pos, const int64_t *crd,
                                               const double *val, const double *x, double *y,
                                               int32_t semiring, int32_t accumulate, void *stream)
{
    cb200::clear_error();
    if (semiring != COMET_B200_PLUS_TIMES && semiring != COMET_B200_PLUS_PAIR)
        return cb200::fail("spmv: unsupported semiring %d", semiring);
    return cb200::spmv_rows(nrows, nnz, row_ids, pos, crd, val, x, y, semiring, accumulate,
                            (cudaStream_t)stream);
}
