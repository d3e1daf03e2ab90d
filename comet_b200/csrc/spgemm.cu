// Gustavson SpGEMM  C = A*B  (optionally C<M,push> = A*B), all CSR, f64 / i64,
// as a symbolic call (fills C.pos) and a numeric call (fills C.crd sorted, C.val).
//
// Rows are binned by an upper bound on their number of distinct columns
// (sum of the lengths of the B rows they touch, capped by the mask row):
//   bin 0  no products                     -> empty row
//   bin 1  bound <= HASH_ROW_MAX           -> one warp per row, hash table in
//          shared memory (int32 keys + f64 accumulators); output order by rank
//          counting among the row's distinct keys
//   bin 2  everything else                 -> one CTA per row, a bitmap over the
//          columns of B in shared memory (global memory when B has too many
//          columns); popcounts give the row's count, prefix popcounts give each
//          column's rank, so crd comes out sorted with no sort and val[rank] is
//          accumulated in place with f64 atomics on the output row, which the
//          CTA has just zeroed and which therefore sits in L2.
// This mirrors COMET's workspace transformation (dense row workspace + mark
// array, sort of the touched columns) with a bit per column instead of a mark
// word per column, and replaces std::sort by ranking.
//
// The bitmaps of bin-2 rows found by the symbolic call are kept (when they fit
// a budget) so that the numeric call does not have to traverse the products a
// second time to rebuild them.
//
// Accumulation order inside a row is not fixed (atomics); structure (pos, crd)
// is exact and values agree with a sequential sum to rounding.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace cb200 {

static const int HASH_ROW_MAX = 256;        // bound for bin 1
static const int HASH_SLOTS = 512;          // table size per warp (load factor <= 0.5)
static const int HASH_WARPS = 4;            // warps per CTA in the hash kernels
static const int BM_THREADS = 512;          // CTA size of the bitmap kernels
static const size_t BM_SMEM_LIMIT = 200 * 1024;
static const size_t BM_STORE_BUDGET = (size_t)12 << 30;

struct Plan {
    int kind;                // 0 = spgemm, 1 = elementwise CSR .* CSR
    int64_t nrows, ncols, nnz_b;
    const int64_t *apos, *acrd, *bpos, *bcrd, *mpos, *mcrd;
    const double *aval, *bval;
    int semi;                // semiring code
    int64_t *cpos;           // caller's array
    int64_t nnz_c;
    // owned device memory
    int32_t *bcrd32;
    int64_t *cnt;            // per-row distinct count
    int32_t *list1, *list2;  // rows of bin 1 / bin 2
    unsigned *bin_counts;    // [2] on device
    unsigned n1, n2;
    uint32_t *bm_store;      // n2 * words, or null
    int words;
    cudaStream_t last;       // stream of the latest call on this plan: its arrays are released in that stream's order
};

static std::mutex g_plans_mu;
static std::unordered_map<int64_t, Plan *> g_plans;
static int64_t g_next_handle = 1;

static void plan_free(Plan *p, cudaStream_t st)
{
    if (!p) return;
    if (p->bcrd32) cudaFreeAsync(p->bcrd32, st);
    if (p->cnt) cudaFreeAsync(p->cnt, st);
    if (p->list1) cudaFreeAsync(p->list1, st);
    if (p->list2) cudaFreeAsync(p->list2, st);
    if (p->bin_counts) cudaFreeAsync(p->bin_counts, st);
    if (p->bm_store) cudaFreeAsync(p->bm_store, st);
    delete p;
}

static int pool_setup()
{
    static bool done[64] = {false};
    int d = 0;
    CB_CUDA(cudaGetDevice(&d));
    if (d >= 0 && d < 64 && !done[d]) {
        cudaMemPool_t pool;
        CB_CUDA(cudaDeviceGetDefaultMemPool(&pool, d));
        uint64_t keep = ~(uint64_t)0;   // keep freed blocks cached for the next call
        CB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        done[d] = true;
    }
    return 0;
}

template <typename T>
static int dev_alloc(T **p, size_t n, cudaStream_t st)
{
    if (n == 0) n = 1;
    cudaError_t e = cudaMallocAsync((void **)p, n * sizeof(T), st);
    if (e != cudaSuccess) {
        *p = nullptr;
        return fail("device allocation of %zu bytes failed: %s", n * sizeof(T), cudaGetErrorString(e));
    }
    return 0;
}

// --------------------------------------------------------------------------
// mask membership: is column j stored in the (ascending) mask row [ms, me)?
// --------------------------------------------------------------------------
__device__ __forceinline__ bool in_mask(const int64_t *__restrict__ mcrd, int64_t ms, int64_t me,
                                        int64_t j)
{
    while (ms < me) {
        int64_t mid = (ms + me) >> 1;
        int64_t v = mcrd[mid];
        if (v == j) return true;
        if (v < j) ms = mid + 1; else me = mid;
    }
    return false;
}

// --------------------------------------------------------------------------
// Semiring arithmetic (codes of include/comet_b200.h).  The second operator
// combines A[i,k] and B[k,j]; the first one folds the products of one output.
// "any" is only offered with "pair", where every product is 1, so it can share
// the min fold.
// --------------------------------------------------------------------------
__device__ __forceinline__ double sr_combine(int semi, double a, double b)
{
    switch (semi) {
    case COMET_B200_PLUS_PAIR: case COMET_B200_ANY_PAIR: return 1.0;
    case COMET_B200_PLUS_FIRST: case COMET_B200_MIN_FIRST: return a;
    case COMET_B200_PLUS_SECOND: case COMET_B200_MIN_SECOND: return b;
    case COMET_B200_MIN_PLUS: return a + b;
    default: return a * b;
    }
}

__host__ __device__ __forceinline__ bool sr_is_min(int semi) { return semi >= COMET_B200_MIN_PLUS; }

__device__ __forceinline__ double sr_identity(int semi) { return sr_is_min(semi) ? __longlong_as_double(0x7ff0000000000000LL) : 0.0; }

// min fold on an f64 in shared or global memory (there is no native one)
__device__ __forceinline__ void atomic_min_f64(double *addr, double v)
{
    unsigned long long *a = (unsigned long long *)addr;
    unsigned long long old = *a;
    while (v < __longlong_as_double((long long)old)) {
        const unsigned long long assumed = old;
        old = atomicCAS(a, assumed, (unsigned long long)__double_as_longlong(v));
        if (old == assumed) break;
    }
}

__device__ __forceinline__ void sr_fold(int semi, double *addr, double v)
{
    if (sr_is_min(semi)) atomic_min_f64(addr, v);
    else atomicAdd(addr, v);
}

// --------------------------------------------------------------------------
// Binning: 8 lanes per row sum the lengths of the B rows it touches.
// --------------------------------------------------------------------------
static const int BIN_THREADS = 256;
static const int BIN_ROWS = (BIN_THREADS / 8) * 4;
static const int64_t BIN_LONG_ROW = 1024;

__global__ void __launch_bounds__(BIN_THREADS)
bin_rows_kernel(int64_t nrows, const int64_t *__restrict__ apos, const int64_t *__restrict__ acrd,
                const int64_t *__restrict__ bpos, const int64_t *__restrict__ mpos,
                int64_t *__restrict__ cnt, int32_t *__restrict__ list1, int32_t *__restrict__ list2,
                unsigned *__restrict__ bin_counts)
{
    __shared__ unsigned char bin_of[BIN_ROWS];
    __shared__ unsigned short local_at[BIN_ROWS];
    __shared__ unsigned local_cnt[2], base[2], n_long;
    __shared__ unsigned short long_slot[BIN_ROWS];
    __shared__ int64_t warp_sum[BIN_THREADS / 32];
    const int g = threadIdx.x / 8, l = threadIdx.x % 8;
    const unsigned gmask = 0xffu << ((threadIdx.x & 31) & ~7);
    if (threadIdx.x < 2) local_cnt[threadIdx.x] = 0;
    if (threadIdx.x == 2) n_long = 0;
    __syncthreads();
    const int64_t row0 = (int64_t)blockIdx.x * BIN_ROWS;
    // the bin of a row from the upper bound ub of its distinct columns
    auto place = [&](int slot, int64_t r, int64_t ub) {
        if (mpos) {
            int64_t ml = mpos[r + 1] - mpos[r];
            if (ml < ub) ub = ml;
        }
        int b = ub == 0 ? 0 : (ub <= HASH_ROW_MAX ? 1 : 2);
        bin_of[slot] = (unsigned char)b;
        if (b == 0) cnt[r] = 0;
        else local_at[slot] = (unsigned short)atomicAdd(&local_cnt[b - 1], 1u);
    };
    for (int pass = 0; pass < 4; pass++) {
        int slot = pass * (BIN_THREADS / 8) + g;
        int64_t r = row0 + slot;
        if (r >= nrows) break;
        const int64_t as = apos[r], ae = apos[r + 1];
        if (ae - as > BIN_LONG_ROW) {                    // a hub row: left to the whole CTA below
            if (l == 0) long_slot[atomicAdd(&n_long, 1u)] = (unsigned short)slot;
            continue;
        }
        int64_t ub = 0;
        for (int64_t p = as + l; p < ae; p += 8) {
            int64_t k = acrd[p];
            ub += bpos[k + 1] - bpos[k];
        }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) ub += __shfl_xor_sync(gmask, (long long)ub, o, 8);
        if (l == 0) place(slot, r, ub);
    }
    __syncthreads();
    // rows of A with thousands of entries: eight lanes would walk them for a millisecond while the rest of
    // the grid has finished
    const unsigned nl = n_long;
    for (unsigned i = 0; i < nl; i++) {
        const int slot = long_slot[i];
        const int64_t r = row0 + slot;
        int64_t ub = 0;
        for (int64_t p = apos[r] + threadIdx.x; p < apos[r + 1]; p += BIN_THREADS) {
            int64_t k = acrd[p];
            ub += bpos[k + 1] - bpos[k];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ub += __shfl_xor_sync(0xffffffffu, (long long)ub, o);
        if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = ub;
        __syncthreads();
        if (threadIdx.x == 0) {
            int64_t t = 0;
            for (int w = 0; w < BIN_THREADS / 32; w++) t += warp_sum[w];
            place(slot, r, t);
        }
        __syncthreads();
    }
    __syncthreads();
    if (threadIdx.x < 2) base[threadIdx.x] = atomicAdd(&bin_counts[threadIdx.x], local_cnt[threadIdx.x]);
    __syncthreads();
    for (int slot = threadIdx.x; slot < BIN_ROWS; slot += BIN_THREADS) {
        int64_t r = row0 + slot;
        if (r >= nrows) break;
        int b = bin_of[slot];
        if (b == 1) list1[base[0] + local_at[slot]] = (int32_t)r;
        else if (b == 2) list2[base[1] + local_at[slot]] = (int32_t)r;
    }
}

// --------------------------------------------------------------------------
// Bin 1: warp per row, hash table in shared memory.
// --------------------------------------------------------------------------
__device__ __forceinline__ int hash_slot(int32_t j)
{
    return (int)(((uint32_t)j * 0x9E3779B1u) >> 23);   // top 9 bits: 0..511
}

// Inserts j; returns the slot, sets *fresh when this call created the entry.
__device__ __forceinline__ int hash_insert(int32_t *keys, int32_t j, bool *fresh)
{
    int h = hash_slot(j);
    *fresh = false;
    for (int probe = 0; probe < HASH_SLOTS; probe++) {
        int32_t old = atomicCAS(&keys[h], -1, j);
        if (old == -1) { *fresh = true; return h; }
        if (old == j) return h;
        h = (h + 1) & (HASH_SLOTS - 1);
    }
    return -1;   // cannot happen: at most HASH_ROW_MAX distinct keys in HASH_SLOTS slots
}

template <bool NUMERIC>
__global__ void __launch_bounds__(HASH_WARPS * 32)
hash_rows_kernel(unsigned nlist, const int32_t *__restrict__ list, const int64_t *__restrict__ apos,
                 const int64_t *__restrict__ acrd, const double *__restrict__ aval,
                 const int64_t *__restrict__ bpos, const int32_t *__restrict__ bcrd,
                 const double *__restrict__ bval, const int64_t *__restrict__ mpos,
                 const int64_t *__restrict__ mcrd, int semi, int64_t *__restrict__ cnt,
                 const int64_t *__restrict__ cpos, int64_t *__restrict__ ccrd,
                 double *__restrict__ cval)
{
    __shared__ int32_t s_keys[HASH_WARPS][HASH_SLOTS];
    __shared__ double s_vals[NUMERIC ? HASH_WARPS : 1][NUMERIC ? HASH_SLOTS : 1];
    __shared__ int32_t s_ckeys[NUMERIC ? HASH_WARPS : 1][NUMERIC ? HASH_ROW_MAX : 1];
    __shared__ unsigned short s_cslot[NUMERIC ? HASH_WARPS : 1][NUMERIC ? HASH_ROW_MAX : 1];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int32_t *keys = s_keys[w];
    const unsigned nwarps = gridDim.x * HASH_WARPS;
    for (unsigned it = blockIdx.x * HASH_WARPS + w; it < nlist; it += nwarps) {
        const int64_t r = list[it];
        for (int s = lane; s < HASH_SLOTS; s += 32) {
            keys[s] = -1;
            if (NUMERIC) s_vals[w][s] = sr_identity(semi);
        }
        __syncwarp();
        int64_t ms = 0, me = 0;
        if (mpos) { ms = mpos[r]; me = mpos[r + 1]; }
        int fresh_count = 0;
        for (int64_t p = apos[r]; p < apos[r + 1]; p++) {
            const int64_t k = acrd[p];
            const double av = NUMERIC ? aval[p] : 0.0;
            for (int64_t q = bpos[k] + lane; q < bpos[k + 1]; q += 32) {
                int32_t j = bcrd[q];
                if (mpos && !in_mask(mcrd, ms, me, j)) continue;
                bool fresh;
                int h = hash_insert(keys, j, &fresh);
                fresh_count += fresh ? 1 : 0;
                if (NUMERIC && h >= 0) sr_fold(semi, &s_vals[w][h], sr_combine(semi, av, bval[q]));
            }
        }
        __syncwarp();
        if (!NUMERIC) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) fresh_count += __shfl_xor_sync(0xffffffffu, fresh_count, o);
            if (lane == 0) cnt[r] = fresh_count;
        } else {
            // compact the occupied slots, then place each key at its rank among them
            int n = 0;
            for (int s0 = 0; s0 < HASH_SLOTS; s0 += 32) {
                int32_t key = keys[s0 + lane];
                unsigned occ = __ballot_sync(0xffffffffu, key != -1);
                if (key != -1) {
                    int at = n + __popc(occ & ((1u << lane) - 1u));
                    s_ckeys[w][at] = key;
                    s_cslot[w][at] = (unsigned short)(s0 + lane);
                }
                n += __popc(occ);
            }
            __syncwarp();
            const int64_t base = cpos[r];
            for (int i = lane; i < n; i += 32) {
                int32_t key = s_ckeys[w][i];
                int rank = 0;
                for (int t = 0; t < n; t++) rank += s_ckeys[w][t] < key ? 1 : 0;
                ccrd[base + rank] = key;
                cval[base + rank] = s_vals[w][s_cslot[w][i]];
            }
        }
        __syncwarp();
    }
}

// --------------------------------------------------------------------------
// Bin 2: CTA per row, bitmap over B's columns.
// --------------------------------------------------------------------------
__device__ __forceinline__ unsigned block_sum_u32(unsigned v, unsigned *s_warp)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = v;
    __syncthreads();
    unsigned t = 0;
    for (int i = 0; i < BM_THREADS / 32; i++) t += s_warp[i];
    return t;
}

// Rows of B longer than this are walked by the whole CTA instead of one warp: in a power-law
// product a few such rows hold most of the work of an output row, and one warp working alone while
// fifteen wait at the next barrier was the largest stall of both passes.
static const int64_t LONG_B_ROW = 1024;

static const unsigned BM_DENSE_ROW = 512;   // bits in 32 consecutive bitmap words from which crd is written word by word (measured: 96 / 192 / 320 / 512 / 768 / never = 22.9 / 21.8 / 21.5 / 21.45 / 21.65 / 21.7 ms numeric at config 4)
static const int LONG_LIST = 1024;          // long rows of B remembered per pass over a row of A

// Calls f(j, bv, av) for every product of row r of A with B in this CTA's share: j and bv are the column and
// value of an entry of row acrd[p] of B (bv = 0 when bval is null), av = aval[p] (0 when aval is null).  A team
// of `team` CTAs deals the entries of the A row out over its warps one by one.  The loads are arranged so that
// no warp waits on a chain: 32 entries of a warp's share look up their rows of B lane-parallel (acrd, then
// bpos, once per batch), the first 32 entries of the next row of B are fetched before the current row is
// worked on, and longer rows are walked two vectors per step with both loads issued first.
// Short rows of B are walked by one warp; long ones are remembered in s_long and then walked by the
// whole CTA.  s_ctl: [0] entries in s_long, [1] set when the list was too small (then the share is
// scanned again for long rows).  All threads of the CTA must call this.
template <typename F>
__device__ __forceinline__ void for_each_product(int64_t r, unsigned part, unsigned team,
                                                 const int64_t *__restrict__ apos,
                                                 const int64_t *__restrict__ acrd,
                                                 const double *__restrict__ aval,
                                                 const int64_t *__restrict__ bpos,
                                                 const int32_t *__restrict__ bcrd,
                                                 const double *__restrict__ bval, int *s_long,
                                                 unsigned *s_ctl, F f)
{
    constexpr int NW = BM_THREADS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t as = apos[r], ae = apos[r + 1];
    if (threadIdx.x == 0) { s_ctl[0] = 0; s_ctl[1] = 0; }
    __syncthreads();
    // this warp's entries of the A row: first, first + stride, ... (dealt one by one, so that the warps of a
    // team share a row of any length evenly); 32 of them at a time are looked up lane-parallel
    const int64_t stride = (int64_t)team * NW;
    const int64_t first = as + (int64_t)part * NW + warp;
    for (int64_t p0 = first; p0 < ae; p0 += 32 * stride) {
        const int64_t p = p0 + lane * stride;
        int64_t s_l = 0;
        int n_l = 0;                     // entries of this lane's row of B; 0 for lanes past the A row and long rows
        double av_l = 0.0;
        if (p < ae) {
            const int64_t k = acrd[p];
            s_l = bpos[k];
            const int64_t len = bpos[k + 1] - s_l;
            if (aval) av_l = aval[p];
            if (len > LONG_B_ROW) {
                const unsigned at = atomicAdd(&s_ctl[0], 1u);
                if (at < (unsigned)LONG_LIST) s_long[at] = (int)(p - as);
                else s_ctl[1] = 1;
            } else {
                n_l = (int)len;
            }
        }
        const int64_t left = (ae - p0 + stride - 1) / stride;      // entries of the sequence from p0 on
        const int n = left < 32 ? (int)left : 32;
        // row t of the batch: start, length, value of A, and the first vector of its entries
        int64_t s0 = __shfl_sync(0xffffffffu, (long long)s_l, 0);
        int n0 = __shfl_sync(0xffffffffu, n_l, 0);
        double a0 = shfl_f64(av_l, 0, 32);
        int32_t j0 = 0;
        double v0 = 0.0;
        if (lane < n0) {
            j0 = bcrd[s0 + lane];
            if (bval) v0 = bval[s0 + lane];
        }
        for (int t = 0; t < n; t++) {
            const int tn = (t + 1) & 31;                 // past the batch: lane 0 again, never used
            const int64_t s1 = __shfl_sync(0xffffffffu, (long long)s_l, tn);
            int n1 = __shfl_sync(0xffffffffu, n_l, tn);
            if (t + 1 >= n) n1 = 0;
            const double a1 = shfl_f64(av_l, tn, 32);
            int32_t j1 = 0;
            double v1 = 0.0;
            if (lane < n1) {
                j1 = bcrd[s1 + lane];
                if (bval) v1 = bval[s1 + lane];
            }
            if (lane < n0) f(j0, v0, a0);
            for (int64_t q = s0 + 32 + lane; q < s0 + n0; q += 64) {
                const bool two = q + 32 < s0 + n0;
                const int32_t ja = bcrd[q];
                const int32_t jb = two ? bcrd[q + 32] : 0;
                const double va = bval ? bval[q] : 0.0;
                const double vb = (bval && two) ? bval[q + 32] : 0.0;
                f(ja, va, a0);
                if (two) f(jb, vb, a0);
            }
            s0 = s1; n0 = n1; a0 = a1; j0 = j1; v0 = v1;
        }
    }
    __syncthreads();
    auto whole_cta = [&](int64_t sl, int64_t el, double avl) {
        for (int64_t q = sl + threadIdx.x; q < el; q += 2 * BM_THREADS) {
            const bool two = q + BM_THREADS < el;
            const int32_t ja = bcrd[q];
            const int32_t jb = two ? bcrd[q + BM_THREADS] : 0;
            const double va = bval ? bval[q] : 0.0;
            const double vb = (bval && two) ? bval[q + BM_THREADS] : 0.0;
            f(ja, va, avl);
            if (two) f(jb, vb, avl);
        }
    };
    if (!s_ctl[1]) {
        const unsigned n = s_ctl[0];
        for (unsigned i = 0; i < n; i++) {
            const int64_t pl = as + s_long[i];
            const int64_t k = acrd[pl];
            whole_cta(bpos[k], bpos[k + 1], aval ? aval[pl] : 0.0);
        }
    } else {
        for (int64_t p0 = as + (int64_t)part * NW; p0 < ae; p0 += stride)
            for (int64_t pl = p0; pl < p0 + NW && pl < ae; pl++) {
                const int64_t k = acrd[pl];
                const int64_t sl = bpos[k], el = bpos[k + 1];
                if (el - sl <= LONG_B_ROW) continue;
                whole_cta(sl, el, aval ? aval[pl] : 0.0);
            }
    }
}

// marks the columns of row r's products in bm (bm cleared by the caller)
__device__ __forceinline__ void mark_products(uint32_t *bm, int64_t r, const int64_t *__restrict__ apos,
                                              const int64_t *__restrict__ acrd,
                                              const int64_t *__restrict__ bpos,
                                              const int32_t *__restrict__ bcrd,
                                              const int64_t *__restrict__ mpos,
                                              const int64_t *__restrict__ mcrd, int *s_long, unsigned *s_ctl)
{
    int64_t ms = 0, me = 0;
    if (mpos) { ms = mpos[r]; me = mpos[r + 1]; }
    for_each_product(r, 0u, 1u, apos, acrd, nullptr, bpos, bcrd, nullptr, s_long, s_ctl, [&](int32_t j, double, double) {
        if (mpos && !in_mask(mcrd, ms, me, j)) return;
        atomicOr(&bm[j >> 5], 1u << (j & 31));          // testing the bit first was measured slower (6.4 vs 5.2 ms)
    });
}

template <bool SMEM>
__global__ void __launch_bounds__(BM_THREADS)
bitmap_symbolic_kernel(unsigned nlist, const int32_t *__restrict__ list, int words,
                       uint32_t *__restrict__ gbm, const int64_t *__restrict__ apos,
                       const int64_t *__restrict__ acrd, const int64_t *__restrict__ bpos,
                       const int32_t *__restrict__ bcrd, const int64_t *__restrict__ mpos,
                       const int64_t *__restrict__ mcrd, int64_t *__restrict__ cnt,
                       uint32_t *__restrict__ bm_store)
{
    extern __shared__ uint32_t s_dyn[];
    __shared__ unsigned s_warp[BM_THREADS / 32];
    __shared__ int s_long[LONG_LIST];
    __shared__ unsigned s_ctl[2];
    uint32_t *bm = SMEM ? s_dyn : gbm + (size_t)blockIdx.x * words;
    for (unsigned it = blockIdx.x; it < nlist; it += gridDim.x) {
        const int64_t r = list[it];
        for (int w = threadIdx.x; w < words; w += BM_THREADS) bm[w] = 0;
        __syncthreads();
        mark_products(bm, r, apos, acrd, bpos, bcrd, mpos, mcrd, s_long, s_ctl);
        __syncthreads();
        unsigned c = 0;
        uint32_t *keep = bm_store ? bm_store + (size_t)it * words : nullptr;
        for (int w = threadIdx.x; w < words; w += BM_THREADS) {
            uint32_t v = bm[w];
            c += __popc(v);
            if (keep) keep[w] = v;
        }
        unsigned total = block_sum_u32(c, s_warp);
        if (threadIdx.x == 0) cnt[r] = total;
        __syncthreads();
    }
}

// --------------------------------------------------------------------------
// Teams for the numeric pass of bin-2 rows.
//
// f64 atomics run at ~200 G/s while their targets stay in L2 and at 20-80 G/s once the rows being
// accumulated no longer fit (measured on this part with a stand-alone probe).  With one CTA per row
// the rows in flight of a power-law product hold far more than L2, so a row whose output is large
// is given to a team of T CTAs instead: they split the entries of the A row, add into the same
// output row, and T is chosen so that (CTAs in flight / T) rows of that size fit the budget.
// Teams are laid out contiguously in an item list and CTAs draw items in order, so the members of a
// team run at about the same time.  The values of team rows are cleared by a separate launch
// (a member must not start adding before another has cleared); single-CTA rows clear their own.
// --------------------------------------------------------------------------
struct TeamHeader {
    unsigned nitems;
    unsigned next;
    unsigned overflow;
    unsigned pad;
};
static const unsigned TEAM_MAX = 64;

__device__ __forceinline__ uint64_t team_pack(unsigned it, unsigned part, unsigned t)
{
    return (uint64_t)it | ((uint64_t)part << 32) | ((uint64_t)t << 48);
}

__global__ void __launch_bounds__(256)
team_items_kernel(unsigned nlist, const int32_t *__restrict__ list, const int64_t *__restrict__ cpos,
                  double ctas_per_budget_entry, TeamHeader *th, uint64_t *items, unsigned cap)
{
    // consecutive list entries in consecutive slots (one warp-wide scan per 32 rows keeps the list ordered)
    const unsigned it = blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    unsigned t = 0;
    if (it < nlist) {
        const int64_t r = list[it];
        const double want = (double)(cpos[r + 1] - cpos[r]) * ctas_per_budget_entry;
        t = want <= 1.0 ? 1u : (want >= (double)TEAM_MAX ? TEAM_MAX : (unsigned)ceil(want));
    }
    unsigned incl = t;
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    unsigned base = 0;
    if (lane == 31) base = atomicAdd(&th->nitems, incl);
    base = __shfl_sync(0xffffffffu, base, 31) + incl - t;
    if (t) {
        if (base + t <= cap) {
            for (unsigned i = 0; i < t; i++) items[base + i] = team_pack(it, i, t);
        } else {
            th->overflow = 1;
        }
    }
}

__global__ void __launch_bounds__(256)
team_clear_kernel(const TeamHeader *th, const uint64_t *__restrict__ items, unsigned cap,
                  const int32_t *__restrict__ list, const int64_t *__restrict__ cpos, int semi,
                  double *__restrict__ cval)
{
    unsigned n = th->nitems;
    if (n > cap) n = 0;
    const double ident = sr_identity(semi);
    for (unsigned i = blockIdx.x; i < n; i += gridDim.x) {
        const uint64_t v = items[i];
        const unsigned t = (unsigned)(v >> 48), part = (unsigned)(v >> 32) & 0xffffu;
        if (t <= 1) continue;
        const int64_t r = list[(unsigned)v];
        const int64_t base = cpos[r], n_out = cpos[r + 1] - base;
        const int64_t per = (n_out + t - 1) / t;
        const int64_t s = base + (int64_t)part * per;
        int64_t e = s + per;
        if (e > base + n_out) e = base + n_out;
        for (int64_t q = s + threadIdx.x; q < e; q += blockDim.x) cval[q] = ident;
    }
}

template <bool SMEM, bool PLUS_TIMES>
__global__ void __launch_bounds__(BM_THREADS, SMEM ? 3 : 1)
bitmap_numeric_kernel(unsigned nlist, const int32_t *__restrict__ list, int words,
                      uint32_t *__restrict__ gbm, const int64_t *__restrict__ apos,
                      const int64_t *__restrict__ acrd, const double *__restrict__ aval,
                      const int64_t *__restrict__ bpos, const int32_t *__restrict__ bcrd,
                      const double *__restrict__ bval, const int64_t *__restrict__ mpos,
                      const int64_t *__restrict__ mcrd, int semi,
                      const uint32_t *__restrict__ bm_store, const int64_t *__restrict__ cpos,
                      int64_t *__restrict__ ccrd, double *__restrict__ cval, TeamHeader *th,
                      const uint64_t *__restrict__ items)
{
    extern __shared__ uint32_t s_dyn[];
    __shared__ unsigned s_item;
    __shared__ unsigned s_scan[BM_THREADS / 32];
    __shared__ int s_long[LONG_LIST];
    __shared__ unsigned s_ctl[2];
    uint32_t *bm = SMEM ? s_dyn : gbm + (size_t)blockIdx.x * 2 * words;
    uint32_t *pre = bm + words;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int NW = BM_THREADS / 32;
    for (unsigned iter = blockIdx.x;; iter += gridDim.x) {
        // one row per CTA, or (with an item list) the next member of a team
        unsigned it = iter, part = 0, team = 1;
        if (th) {
            if (threadIdx.x == 0) s_item = atomicAdd(&th->next, 1u);
            __syncthreads();
            const unsigned idx = s_item;
            if (idx >= th->nitems) break;
            const uint64_t v = items[idx];
            it = (unsigned)v;
            part = (unsigned)(v >> 32) & 0xffffu;
            team = (unsigned)(v >> 48);
        } else if (iter >= nlist) {
            break;
        }
        const int64_t r = list[it];
        if (bm_store) {
            const uint32_t *keep = bm_store + (size_t)it * words;
            for (int w = threadIdx.x; w < words; w += BM_THREADS) bm[w] = __ldcs(keep + w);     // read once per member
            __syncthreads();
        } else {
            for (int w = threadIdx.x; w < words; w += BM_THREADS) bm[w] = 0;
            __syncthreads();
            mark_products(bm, r, apos, acrd, bpos, bcrd, mpos, mcrd, s_long, s_ctl);
            __syncthreads();
        }
        // Exclusive prefix popcount per word, and the row's coordinates.  A warp owns a run of whole rows of 32
        // consecutive words; lane l of the warp holds word l of the current row, so every shared-memory access
        // below is conflict-free and the prefix inside a row is a warp scan.
        const int nrow32 = (words + 31) >> 5;
        const int rows_per_warp = (nrow32 + NW - 1) / NW;
        const int i0 = warp * rows_per_warp, i1 = min(i0 + rows_per_warp, nrow32);
        unsigned mine = 0;
        for (int i = i0; i < i1; i++) {
            const int w = i * 32 + lane;
            if (w < words) mine += __popc(bm[w]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        if (lane == 0) s_scan[warp] = mine;
        __syncthreads();
        unsigned run = 0;
        for (int w2 = 0; w2 < warp; w2++) run += s_scan[w2];
        const int64_t base = cpos[r];
        const int64_t rown = cpos[r + 1] - base;
        for (int i = i0; i < i1; i++) {
            const int w = i * 32 + lane;
            uint32_t v = w < words ? bm[w] : 0u;
            const unsigned c = __popc(v);
            unsigned incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const unsigned excl = run + incl - c;
            if (w < words) pre[w] = excl;
            const unsigned rowtotal = __shfl_sync(0xffffffffu, incl, 31);
            run += rowtotal;
            // the members of a team share the writing of crd by rows of 32 words
            if (rowtotal == 0 || (team > 1 && (unsigned)i % team != part)) continue;
            if (rowtotal >= BM_DENSE_ROW) {
                // many bits per word: one word at a time, lane b writes column 32 w + b at its rank, so a
                // store instruction covers consecutive addresses
                // (all 32 words in a fixed-trip loop: the shuffles of different words do not depend on each
                // other, so they overlap; a loop over the non-empty words only ran one word per shuffle latency)
                long long *out = (long long *)ccrd + base;
                const unsigned below = (1u << lane) - 1u;
#pragma unroll 8
                for (int l = 0; l < 32; l++) {
                    const uint32_t wv = __shfl_sync(0xffffffffu, v, l);
                    const unsigned wp = __shfl_sync(0xffffffffu, excl, l);
                    if ((wv >> lane) & 1u) __stcs(out + wp + __popc(wv & below), (long long)(i * 32 + l) * 32 + lane);
                }
            } else {
                unsigned at = excl;
                while (v) {
                    const int b = __ffs(v) - 1;
                    v &= v - 1;
                    __stcs((long long *)ccrd + base + at, (long long)w * 32 + b);   // written once, not read here again
                    at++;
                }
            }
        }
        if (team == 1)
            for (int64_t t = threadIdx.x; t < rown; t += BM_THREADS) cval[base + t] = sr_identity(semi);
        __syncthreads();
        // accumulate every product at the rank of its column
        double *crow = cval + base;
        for_each_product(r, part, team, apos, acrd, aval, bpos, bcrd, bval, s_long, s_ctl, [&](int32_t j, double bv, double av) {
            uint32_t word = bm[j >> 5];
            uint32_t bit = 1u << (j & 31);
            if (!(word & bit)) return;          // filtered out by the mask
            unsigned rank = pre[j >> 5] + __popc(word & (bit - 1u));
            if (PLUS_TIMES) atomicAdd(crow + rank, av * bv);
            else sr_fold(semi, crow + rank, sr_combine(semi, av, bv));
        });
        __syncthreads();
    }
    (void)mpos; (void)mcrd;
}

// --------------------------------------------------------------------------
// Elementwise CSR .* CSR: two-pointer intersection, one thread per row.
// --------------------------------------------------------------------------
template <bool NUMERIC>
__global__ void __launch_bounds__(256)
elews_ss_kernel(int64_t nrows, const int64_t *__restrict__ apos, const int64_t *__restrict__ acrd,
                const double *__restrict__ aval, const int64_t *__restrict__ bpos,
                const int64_t *__restrict__ bcrd, const double *__restrict__ bval,
                int64_t *__restrict__ cnt, const int64_t *__restrict__ cpos,
                int64_t *__restrict__ ccrd, double *__restrict__ cval)
{
    int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= nrows) return;
    int64_t p = apos[r], pe = apos[r + 1], q = bpos[r], qe = bpos[r + 1];
    int64_t n = 0, at = NUMERIC ? cpos[r] : 0;
    while (p < pe && q < qe) {
        int64_t ca = acrd[p], cb = bcrd[q];
        if (ca == cb) {
            if (NUMERIC) { ccrd[at + n] = ca; cval[at + n] = aval[p] * bval[q]; }
            n++;
        }
        if (ca <= cb) p++;
        if (cb <= ca) q++;
    }
    if (!NUMERIC) cnt[r] = n;
}

// --------------------------------------------------------------------------
// Host side
// --------------------------------------------------------------------------
static int64_t register_plan(Plan *p)
{
    std::lock_guard<std::mutex> lk(g_plans_mu);
    int64_t h = g_next_handle++;
    g_plans[h] = p;
    return h;
}

static Plan *find_plan(int64_t h, bool remove)
{
    std::lock_guard<std::mutex> lk(g_plans_mu);
    auto it = g_plans.find(h);
    if (it == g_plans.end()) return nullptr;
    Plan *p = it->second;
    if (remove) g_plans.erase(it);
    return p;
}

static int bitmap_grid(unsigned nlist, size_t smem_bytes)
{
    int per_sm = smem_bytes ? (int)((220 * 1024) / (smem_bytes + 1024)) : 2;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 2048 / BM_THREADS) per_sm = 2048 / BM_THREADS;
    int64_t g = (int64_t)sm_count() * per_sm;
    if (g > nlist) g = nlist;
    return (int)(g < 1 ? 1 : g);
}

int spgemm_symbolic(int64_t nrows, int64_t ncols_b, int64_t nnz_b, const int64_t *apos,
                    const int64_t *acrd, const double *aval, const int64_t *bpos,
                    const int64_t *bcrd, const double *bval, const int64_t *mpos,
                    const int64_t *mcrd, int semiring, int64_t *cpos, int64_t *nnz_host,
                    int64_t *handle_out, cudaStream_t st)
{
    if (ncols_b >= 0x7fffffffLL || nrows >= 0x7fffffffLL)
        return fail("spgemm: more than 2^31-1 rows or columns is not supported");
    if (((uintptr_t)bcrd & 15) != 0) return fail("spgemm: B.crd must be 16-byte aligned");
    CB_TRY(pool_setup());
    Plan *p = new Plan();
    memset(p, 0, sizeof(Plan));
    p->kind = 0; p->nrows = nrows; p->ncols = ncols_b; p->nnz_b = nnz_b;
    p->last = st;
    p->apos = apos; p->acrd = acrd; p->aval = aval; p->bpos = bpos; p->bcrd = bcrd; p->bval = bval;
    p->mpos = mpos; p->mcrd = mpos ? mcrd : nullptr; p->semi = semiring;
    p->cpos = cpos;
    p->words = (int)ceil_div(ncols_b, 32);
    int rc = 0;
#define STEP(expr) do { if (!rc) rc = (expr); } while (0)
#define STEP_CUDA(expr) do { if (!rc) { cudaError_t e_ = (expr); if (e_ != cudaSuccess) rc = fail("%s failed: %s", #expr, cudaGetErrorString(e_)); } } while (0)
    STEP(dev_alloc(&p->bcrd32, (size_t)nnz_b, st));
    STEP(dev_alloc(&p->cnt, (size_t)nrows + 1, st));
    STEP(dev_alloc(&p->list1, (size_t)nrows, st));
    STEP(dev_alloc(&p->list2, (size_t)nrows, st));
    STEP(dev_alloc(&p->bin_counts, 2, st));
    STEP_CUDA(cudaMemsetAsync(p->bin_counts, 0, 2 * sizeof(unsigned), st));
    STEP(narrow_i64_to_i32(bcrd, p->bcrd32, nnz_b, st));
    if (!rc && nrows > 0) {
        bin_rows_kernel<<<(unsigned)ceil_div(nrows, BIN_ROWS), BIN_THREADS, 0, st>>>(
            nrows, apos, acrd, bpos, mpos, p->cnt, p->list1, p->list2, p->bin_counts);
        STEP_CUDA(cudaGetLastError());
    }
    unsigned counts[2] = {0, 0};
    STEP_CUDA(cudaMemcpyAsync(counts, p->bin_counts, sizeof(counts), cudaMemcpyDeviceToHost, st));
    STEP_CUDA(cudaStreamSynchronize(st));
    p->n1 = counts[0]; p->n2 = counts[1];
    if (!rc && p->n1) {
        unsigned grid = (unsigned)ceil_div(p->n1, HASH_WARPS);
        unsigned cap = (unsigned)sm_count() * 16;
        if (grid > cap) grid = cap;
        hash_rows_kernel<false><<<grid, HASH_WARPS * 32, 0, st>>>(
            p->n1, p->list1, apos, acrd, aval, bpos, p->bcrd32, bval, mpos, p->mcrd, p->semi, p->cnt,
            nullptr, nullptr, nullptr);
        STEP_CUDA(cudaGetLastError());
    }
    if (!rc && p->n2) {
        size_t store = (size_t)p->n2 * p->words * sizeof(uint32_t);
        // the symbolic pass's bitmaps are kept for the numeric pass while they fit the budget
        // (COMET_B200_SPGEMM_BITMAP_GB overrides it; 0 makes the numeric pass mark its rows again)
        size_t budget = BM_STORE_BUDGET;
        if (const char *e = getenv("COMET_B200_SPGEMM_BITMAP_GB")) budget = (size_t)(atof(e) * (double)(1ull << 30));
        if (store <= budget) {
            cudaError_t e = cudaMallocAsync((void **)&p->bm_store, store, st);
            if (e != cudaSuccess) { p->bm_store = nullptr; (void)cudaGetLastError(); }
        }
        size_t smem = (size_t)p->words * sizeof(uint32_t);
        if (2 * smem <= BM_SMEM_LIMIT) {
            int grid = bitmap_grid(p->n2, smem);
            STEP_CUDA(cudaFuncSetAttribute(bitmap_symbolic_kernel<true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (!rc)
                bitmap_symbolic_kernel<true><<<grid, BM_THREADS, smem, st>>>(
                    p->n2, p->list2, p->words, nullptr, apos, acrd, bpos, p->bcrd32, mpos, p->mcrd,
                    p->cnt, p->bm_store);
        } else {
            int grid = bitmap_grid(p->n2, 0);
            void *gbm = nullptr;
            STEP(scratch(SLOT_BITMAP, (size_t)grid * 2 * smem, &gbm));
            if (!rc)
                bitmap_symbolic_kernel<false><<<grid, BM_THREADS, 0, st>>>(
                    p->n2, p->list2, p->words, (uint32_t *)gbm, apos, acrd, bpos, p->bcrd32, mpos,
                    p->mcrd, p->cnt, p->bm_store);
        }
        STEP_CUDA(cudaGetLastError());
    }
    STEP(exclusive_scan_i64(p->cnt, cpos, nrows, st));
    STEP_CUDA(cudaMemcpyAsync(&p->nnz_c, cpos + nrows, sizeof(int64_t), cudaMemcpyDeviceToHost, st));
    STEP_CUDA(cudaStreamSynchronize(st));
#undef STEP
#undef STEP_CUDA
    if (rc) { plan_free(p, st); return rc; }
    *nnz_host = p->nnz_c;
    *handle_out = register_plan(p);
    return 0;
}

int elews_ss_symbolic(int64_t nrows, const int64_t *apos, const int64_t *acrd, const double *aval,
                      const int64_t *bpos, const int64_t *bcrd, const double *bval, int64_t *cpos,
                      int64_t *nnz_host, int64_t *handle_out, cudaStream_t st)
{
    CB_TRY(pool_setup());
    Plan *p = new Plan();
    memset(p, 0, sizeof(Plan));
    p->kind = 1; p->nrows = nrows;
    p->last = st;
    p->apos = apos; p->acrd = acrd; p->aval = aval; p->bpos = bpos; p->bcrd = bcrd; p->bval = bval;
    p->cpos = cpos;
    int rc = dev_alloc(&p->cnt, (size_t)nrows + 1, st);
    if (!rc && nrows > 0) {
        elews_ss_kernel<false><<<(unsigned)ceil_div(nrows, 256), 256, 0, st>>>(
            nrows, apos, acrd, aval, bpos, bcrd, bval, p->cnt, nullptr, nullptr, nullptr);
        if (cudaGetLastError() != cudaSuccess) rc = fail("elews symbolic launch failed");
    }
    if (!rc) rc = exclusive_scan_i64(p->cnt, cpos, nrows, st);
    if (!rc && cudaMemcpyAsync(&p->nnz_c, cpos + nrows, sizeof(int64_t), cudaMemcpyDeviceToHost, st) != cudaSuccess)
        rc = fail("elews symbolic: copy of nnz failed");
    if (!rc && cudaStreamSynchronize(st) != cudaSuccess) rc = fail("elews symbolic: synchronize failed");
    if (rc) { plan_free(p, st); return rc; }
    *nnz_host = p->nnz_c;
    *handle_out = register_plan(p);
    return 0;
}

int sparse_out_numeric(int64_t handle, int64_t *ccrd, double *cval, int keep, cudaStream_t st)
{
    Plan *p = find_plan(handle, !keep);
    if (!p) return fail("numeric phase: unknown handle %lld", (long long)handle);
    p->last = st;
    int rc = 0;
    if (p->kind == 1) {
        if (p->nrows > 0) {
            elews_ss_kernel<true><<<(unsigned)ceil_div(p->nrows, 256), 256, 0, st>>>(
                p->nrows, p->apos, p->acrd, p->aval, p->bpos, p->bcrd, p->bval, nullptr, p->cpos, ccrd,
                cval);
            if (cudaGetLastError() != cudaSuccess) rc = fail("elews numeric launch failed");
        }
    } else {
        if (p->n1) {
            unsigned grid = (unsigned)ceil_div(p->n1, HASH_WARPS);
            unsigned cap = (unsigned)sm_count() * 16;
            if (grid > cap) grid = cap;
            hash_rows_kernel<true><<<grid, HASH_WARPS * 32, 0, st>>>(
                p->n1, p->list1, p->apos, p->acrd, p->aval, p->bpos, p->bcrd32, p->bval, p->mpos,
                p->mcrd, p->semi, nullptr, p->cpos, ccrd, cval);
            if (cudaGetLastError() != cudaSuccess) rc = fail("spgemm numeric (hash) launch failed");
        }
        if (!rc && p->n2) {
            size_t smem = (size_t)p->words * sizeof(uint32_t) * 2;
            if (smem <= BM_SMEM_LIMIT) {
                // full occupancy grid even for few rows: teams give every CTA work
                int grid = bitmap_grid(0xffffffffu, smem);
                // team size of a row = its output entries * 8 bytes * CTAs in flight / budget
                double budget_mb = 60.0;                 // measured best on R-MAT scale 18 (25 / 40 / 60 / 160 MB)
                if (const char *e = getenv("COMET_B200_SPGEMM_TEAM_MB")) budget_mb = atof(e);
                if (budget_mb < 0.001) budget_mb = 0.001;
                const double per_entry = 8.0 * grid / (budget_mb * 1048576.0);
                const size_t cap = (size_t)p->n2 + (size_t)((double)p->nnz_c * per_entry) + 64;
                void *tm = nullptr;
                rc = cap > 0xfffffff0u ? fail("spgemm numeric: too many team items")
                                       : scratch(SLOT_TEAMS, sizeof(TeamHeader) + cap * sizeof(uint64_t), &tm);
                TeamHeader *th = (TeamHeader *)tm;
                uint64_t *items = (uint64_t *)((char *)tm + sizeof(TeamHeader));
                if (!rc && cudaMemsetAsync(th, 0, sizeof(TeamHeader), st) != cudaSuccess)
                    rc = fail("spgemm numeric: clearing the team header failed");
                if (!rc) {
                    team_items_kernel<<<(unsigned)ceil_div(p->n2, 256), 256, 0, st>>>(
                        p->n2, p->list2, p->cpos, per_entry, th, items, (unsigned)cap);
                    team_clear_kernel<<<(unsigned)sm_count() * 8, 256, 0, st>>>(th, items, (unsigned)cap, p->list2,
                                                                                p->cpos, p->semi, cval);
                    if (p->semi == COMET_B200_PLUS_TIMES) {
                        cudaFuncSetAttribute(bitmap_numeric_kernel<true, true>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                        bitmap_numeric_kernel<true, true><<<grid, BM_THREADS, smem, st>>>(
                            p->n2, p->list2, p->words, nullptr, p->apos, p->acrd, p->aval, p->bpos, p->bcrd32,
                            p->bval, p->mpos, p->mcrd, p->semi, p->bm_store, p->cpos, ccrd, cval, th, items);
                    } else {
                        cudaFuncSetAttribute(bitmap_numeric_kernel<true, false>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                        bitmap_numeric_kernel<true, false><<<grid, BM_THREADS, smem, st>>>(
                            p->n2, p->list2, p->words, nullptr, p->apos, p->acrd, p->aval, p->bpos, p->bcrd32,
                            p->bval, p->mpos, p->mcrd, p->semi, p->bm_store, p->cpos, ccrd, cval, th, items);
                    }
                }
            } else {
                int grid = bitmap_grid(p->n2, 0);
                void *gbm = nullptr;
                rc = scratch(SLOT_BITMAP, (size_t)grid * smem, &gbm);
                if (!rc)
                    bitmap_numeric_kernel<false, false><<<grid, BM_THREADS, 0, st>>>(
                        p->n2, p->list2, p->words, (uint32_t *)gbm, p->apos, p->acrd, p->aval, p->bpos,
                        p->bcrd32, p->bval, p->mpos, p->mcrd, p->semi, p->bm_store, p->cpos, ccrd, cval, nullptr,
                        nullptr);
            }
            if (!rc && cudaGetLastError() != cudaSuccess) rc = fail("spgemm numeric (bitmap) launch failed");
        }
    }
    if (!keep) plan_free(p, st);
    return rc;
}

void destroy_plan(int64_t handle)
{
    // a numeric launch of a kept plan may still be running: free behind it, in its own stream's order
    Plan *p = find_plan(handle, true);
    if (p) plan_free(p, p->last);
}

}  // namespace cb200

extern "C" {

int32_t comet_b200_dev_spgemm_symbolic_f64_i64(int64_t nrows, int64_t ncols_b, int64_t nnz_b,
                                               const int64_t *apos, const int64_t *acrd,
                                               const double *aval, const int64_t *bpos,
                                               const int64_t *bcrd, const double *bval,
                                               const int64_t *mpos, const int64_t *mcrd,
                                               int32_t semiring, int64_t *cpos, int64_t *nnz_host,
                                               int64_t *handle_out, void *stream)
{
    cb200::clear_error();
    if (semiring < COMET_B200_PLUS_TIMES || semiring > COMET_B200_ANY_PAIR)
        return cb200::fail("spgemm: unsupported semiring %d", semiring);
    return cb200::spgemm_symbolic(nrows, ncols_b, nnz_b, apos, acrd, aval, bpos, bcrd, bval, mpos, mcrd,
                                  semiring, cpos, nnz_host, handle_out, (cudaStream_t)stream);
}

int32_t comet_b200_dev_elews_mul_sparse_sparse_symbolic_f64_i64(
    int64_t nrows, const int64_t *apos, const int64_t *acrd, const double *aval,
    const int64_t *bpos, const int64_t *bcrd, const double *bval, int64_t *cpos, int64_t *nnz_host,
    int64_t *handle_out, void *stream)
{
    cb200::clear_error();
    return cb200::elews_ss_symbolic(nrows, apos, acrd, aval, bpos, bcrd, bval, cpos, nnz_host,
                                    handle_out, (cudaStream_t)stream);
}

int32_t comet_b200_dev_spgemm_numeric_f64_i64(int64_t handle, int64_t *ccrd, double *cval,
                                              int32_t keep, void *stream)
{
    cb200::clear_error();
    return cb200::sparse_out_numeric(handle, ccrd, cval, keep, (cudaStream_t)stream);
}

void comet_b200_handle_destroy(int64_t handle) { cb200::destroy_plan(handle); }

}
