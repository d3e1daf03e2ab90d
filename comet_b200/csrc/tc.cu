// Masked SpGEMM reduced to a scalar under plus-pair:
//   count = sum over stored A[i,k] of | row k of B  intersect  row i of M |
// which is SUM(C<M,push> = A*B) with every product worth 1.  With A = B = M = L
// (strict lower triangle of a symmetric graph) it is the triangle count.
//
// Work is split by stored entries of A, not by rows: a group of 8 lanes takes
// 32 consecutive entries, finds their row once by binary search in A.pos, and
// for each entry walks the shorter of the two sorted lists with its lanes while
// binary-searching the longer one.  (The reference probes a bitmap of the mask
// row with every element of B's row; the number of hits is the same, the
// number of probes is min(len) * log(max len) instead of len(B row).)
// Coordinates are narrowed to int32 once per call (scratch memory).
//
// Counts are exact int64; no floating point is involved.
#include "common.cuh"

namespace cb200 {

static const int TC_THREADS = 256;
static const int TC_GROUP = 8;
static const int TC_EDGES = 32;   // entries of A per group per step

__device__ __forceinline__ bool contains(const int32_t *__restrict__ a, int64_t lo, int64_t hi,
                                         int32_t key)
{
    while (lo < hi) {
        int64_t mid = (lo + hi) >> 1;
        int32_t v = __ldg(a + mid);
        if (v == key) return true;
        if (v < key) lo = mid + 1; else hi = mid;
    }
    return false;
}

__global__ void __launch_bounds__(TC_THREADS)
masked_pair_count_kernel(int64_t row_lo, int64_t row_hi, const int64_t *__restrict__ apos,
                         const int32_t *__restrict__ acrd, const int64_t *__restrict__ bpos,
                         const int32_t *__restrict__ bcrd, const int64_t *__restrict__ mpos,
                         const int32_t *__restrict__ mcrd, unsigned long long *__restrict__ count)
{
    __shared__ unsigned long long s_part[TC_THREADS / 32];
    const int l = threadIdx.x % TC_GROUP;
    const int64_t group = ((int64_t)blockIdx.x * TC_THREADS + threadIdx.x) / TC_GROUP;
    const int64_t ngroups = (int64_t)gridDim.x * TC_THREADS / TC_GROUP;
    const int64_t e_begin = apos[row_lo], e_end = apos[row_hi];
    const int64_t nchunks = (e_end - e_begin + TC_EDGES - 1) / TC_EDGES;
    unsigned long long hits = 0;
    for (int64_t ch = group; ch < nchunks; ch += ngroups) {
        int64_t p0 = e_begin + ch * TC_EDGES;
        int64_t p1 = p0 + TC_EDGES < e_end ? p0 + TC_EDGES : e_end;
        // row of p0: last r in [row_lo, row_hi) with apos[r] <= p0
        int64_t lo = row_lo, hi = row_hi;
        while (hi - lo > 1) {
            int64_t mid = (lo + hi) >> 1;
            if (apos[mid] <= p0) lo = mid; else hi = mid;
        }
        int64_t i = lo, i_end = apos[i + 1];
        int64_t ms = mpos[i], me = mpos[i + 1];
        for (int64_t p = p0; p < p1; p++) {
            while (p >= i_end) {   // skip to the row that holds p (empty rows in between)
                i++;
                i_end = apos[i + 1];
                ms = mpos[i];
                me = mpos[i + 1];
            }
            if (ms == me) continue;
            const int64_t k = acrd[p];
            const int64_t bs = bpos[k], be = bpos[k + 1];
            if (bs == be) continue;
            if (be - bs <= me - ms) {
                for (int64_t q = bs + l; q < be; q += TC_GROUP)
                    hits += contains(mcrd, ms, me, __ldg(bcrd + q)) ? 1 : 0;
            } else {
                for (int64_t q = ms + l; q < me; q += TC_GROUP)
                    hits += contains(bcrd, bs, be, __ldg(mcrd + q)) ? 1 : 0;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = hits;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < TC_THREADS / 32; w++) t += s_part[w];
        if (t) atomicAdd(count, t);
    }
}

int masked_pair_count(int64_t row_lo, int64_t row_hi, int64_t ncols, int64_t nnz_a, int64_t nnz_b,
                      int64_t nnz_m, const int64_t *apos, const int64_t *acrd, const int64_t *bpos,
                      const int64_t *bcrd, const int64_t *mpos, const int64_t *mcrd,
                      int64_t *count_dev, cudaStream_t st)
{
    CB_CUDA(cudaMemsetAsync(count_dev, 0, sizeof(int64_t), st));
    if (row_hi <= row_lo || nnz_a <= 0 || nnz_b <= 0 || nnz_m <= 0) return 0;
    if (ncols >= 0x7fffffffLL) return fail("masked count: more than 2^31-1 columns is not supported");
    if ((((uintptr_t)acrd | (uintptr_t)bcrd | (uintptr_t)mcrd) & 15) != 0)
        return fail("masked count: crd arrays must be 16-byte aligned");
    void *a32 = nullptr, *b32 = nullptr, *m32 = nullptr;
    CB_TRY(scratch(SLOT_NARROW_A, (size_t)nnz_a * sizeof(int32_t), &a32));
    CB_TRY(narrow_i64_to_i32(acrd, (int32_t *)a32, nnz_a, st));
    if (bcrd == acrd && nnz_b == nnz_a) b32 = a32;
    else {
        CB_TRY(scratch(SLOT_NARROW_B, (size_t)nnz_b * sizeof(int32_t), &b32));
        CB_TRY(narrow_i64_to_i32(bcrd, (int32_t *)b32, nnz_b, st));
    }
    if (mcrd == acrd && nnz_m == nnz_a) m32 = a32;
    else if (mcrd == bcrd && nnz_m == nnz_b) m32 = b32;
    else {
        CB_TRY(scratch(SLOT_NARROW_M, (size_t)nnz_m * sizeof(int32_t), &m32));
        CB_TRY(narrow_i64_to_i32(mcrd, (int32_t *)m32, nnz_m, st));
    }
    int64_t groups = ceil_div(nnz_a, TC_EDGES);
    int64_t blocks = ceil_div(groups * TC_GROUP, TC_THREADS);
    int64_t cap = (int64_t)sm_count() * 64;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    masked_pair_count_kernel<<<(unsigned)blocks, TC_THREADS, 0, st>>>(
        row_lo, row_hi, apos, (const int32_t *)a32, bpos, (const int32_t *)b32, mpos,
        (const int32_t *)m32, (unsigned long long *)count_dev);
    CB_LAUNCH_CHECK();
    return 0;
}

}  // namespace cb200

extern "C" int32_t comet_b200_dev_masked_spgemm_count_f64_i64(
    int64_t row_lo, int64_t row_hi, int64_t ncols, int64_t nnz_a, int64_t nnz_b, int64_t nnz_m,
    const int64_t *apos, const int64_t *acrd, const int64_t *bpos, const int64_t *bcrd,
    const int64_t *mpos, const int64_t *mcrd, int64_t *count_dev, void *stream)
{
    cb200::clear_error();
    return cb200::masked_pair_count(row_lo, row_hi, ncols, nnz_a, nnz_b, nnz_m, apos, acrd, bpos, bcrd,
                                    mpos, mcrd, count_dev, (cudaStream_t)stream);
}
