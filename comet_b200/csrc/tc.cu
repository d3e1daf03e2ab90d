// Masked SpGEMM reduced to a scalar under plus-pair:
//   count = sum over stored A[i,k] of the number of entries of row k of B whose
//           column is stored in row i of M
// which is SUM(C<M,push> = A*B) with every product worth 1.  With A = B = M = L
// (strict lower triangle of a symmetric graph) it is the triangle count.
//
// Same structure as the reference's push mask (set the bits of M's row i, test
// every product's column, clear them).  The bit array over all columns does not
// fit shared memory, so the mask row is held there as a cuckoo hash set: two
// tables, two hash functions, every coordinate sits in one of its two slots.  A
// probe is therefore two 32-bit shared-memory loads and two compares -- the same
// short instruction sequence for a hit and for a miss, with no loop, so the
// lanes of a warp do not diverge (about one probe in fourteen is a hit, so a
// filter in front of a looping table sent almost every warp down the slow path).
// The set is built at a load factor of 1/4; if an insertion chain does not end
// within its bound the row falls back to linear probing in the same memory.
// Rows are binned by the length of their mask row:
//   <= 128 entries   one warp per row
//   <= 2048 entries  one CTA per row
//   longer           cut into units of (4096 mask entries) x (2048 entries of A),
//                    one CTA per unit, so a huge row spreads over many SMs; the mask row is
//                    ascending, and a segment leaves out the coordinate its predecessor ended
//                    with, so a coordinate stored twice in M still counts once
// and rows / units are handed out dynamically (one atomic each), because the work
// per row (sum of the lengths of the B rows it touches) is very uneven.
// Every element of every touched B row is read (coalesced, 128-bit loads of int32
// coordinates) and tested once per mask segment, so the number of probes equals
// the reference's.  Coordinates are narrowed to int32 once per call (scratch memory).
//
// Counts are exact int64; no floating point is involved.
#include "common.cuh"

namespace cb200 {

static const int TC_WARP_MAX = 128;      // mask-row length handled by a warp
static const int TC_WARP_LOG2 = 9;       // log2 slots of its set (both tables together)
static const int TC_WARPS = 8;           // warps per CTA in the warp kernel
static const int TC_MID_MAX = 2048;
static const int TC_MID_LOG2 = 13;
static const int TC_BIG_SEG = 4096;      // mask entries per unit
static const int TC_BIG_SLICE = 2048;    // entries of A per unit
static const int TC_BIG_LOG2 = 14;
static const int TC_CUCKOO_CHAIN = 48;   // longest eviction chain before the row falls back

struct TcUnit {
    int32_t row;
    int32_t mask_off;    // first mask entry of the unit, relative to the row
    int32_t edge_off;    // first entry of A of the unit, relative to the row
};

struct TcHeader {
    unsigned count[4];   // rows in the warp bin, rows in the CTA bin, units, rows whose units did not fit
    unsigned next[4];    // next item to hand out per list
};

// --- cuckoo set: tables T0 = tab[0, H) and T1 = tab[H, 2H), H = 2^(LOG2-1) -------------------------
template <int LOG2>
__device__ __forceinline__ unsigned tc_h0(int32_t j)
{
    return ((uint32_t)j * 0x9E3779B1u) >> (33 - LOG2);
}

template <int LOG2>
__device__ __forceinline__ unsigned tc_h1(int32_t j)
{
    return (1u << (LOG2 - 1)) + (((uint32_t)j * 0x85EBCA6Bu + 0x6D2B79F5u) >> (33 - LOG2));
}

// Returns false if the eviction chain did not end.
template <int LOG2>
__device__ __forceinline__ bool tc_cuckoo_insert(int32_t *tab, int32_t key)
{
    bool second = false;
    for (int it = 0; it < TC_CUCKOO_CHAIN; it++) {
        const unsigned pos = second ? tc_h1<LOG2>(key) : tc_h0<LOG2>(key);
        const int32_t old = atomicExch(&tab[pos], key);
        if (old == -1 || old == key) return true;
        key = old;                 // the evicted coordinate moves to its slot in the other table
        second = !second;
    }
    return false;
}

// --- fallback: linear probing over all 2^LOG2 slots -------------------------------------------
template <int LOG2>
__device__ __forceinline__ unsigned tc_slot(int32_t j)
{
    return ((uint32_t)j * 0x9E3779B1u) >> (32 - LOG2);
}

template <int LOG2>
__device__ __forceinline__ void tc_linear_insert(int32_t *tab, int32_t j)
{
    unsigned h = tc_slot<LOG2>(j);
    for (int probe = 0; probe < (1 << LOG2); probe++) {
        int32_t old = atomicCAS(&tab[h], -1, j);
        if (old == -1 || old == j) return;
        h = (h + 1) & ((1u << LOG2) - 1u);
    }
}

template <int LOG2>
__device__ __forceinline__ unsigned tc_linear_probe(const int32_t *tab, int32_t j)
{
    unsigned h = tc_slot<LOG2>(j);
    for (int probe = 0; probe < (1 << LOG2); probe++) {
        int32_t k = tab[h];
        if (k == j) return 1u;
        if (k == -1) return 0u;
        h = (h + 1) & ((1u << LOG2) - 1u);
    }
    return 0u;
}

// `linear` is uniform over the threads that share the set.
template <int LOG2>
__device__ __forceinline__ unsigned tc_probe(const int32_t *tab, bool linear, int32_t j)
{
    if (linear) return tc_linear_probe<LOG2>(tab, j);
    return (unsigned)(tab[tc_h0<LOG2>(j)] == j) | (unsigned)(tab[tc_h1<LOG2>(j)] == j);
}

// Clears and fills the set with mask entries [ms, me); `nthreads` threads with index `tid` cooperate
// (a warp when !block, the whole CTA otherwise; `flag` is a shared-memory word they all see).
// `skip` (-1 = none) is a coordinate already counted with the segment before this one: the mask row is
// ascending, so a coordinate stored twice sits at adjacent positions, and when a segment boundary
// falls between the two copies the later segment must not hold it again (a mask bit counts once).
// Returns true if the set had to fall back to linear probing.
template <int LOG2>
__device__ __forceinline__ bool tc_fill(int32_t *tab, unsigned *flag, const int32_t *__restrict__ mcrd,
                                        int64_t ms, int64_t me, int tid, int nthreads, bool block,
                                        int32_t skip = -1)
{
    for (int s = tid; s < (1 << LOG2); s += nthreads) tab[s] = -1;
    if (tid == 0) *flag = 0u;
    if (block) __syncthreads(); else __syncwarp();
    bool ok = true;
    for (int64_t t = ms + tid; t < me; t += nthreads) {
        const int32_t key = mcrd[t];
        if (key != skip) ok = tc_cuckoo_insert<LOG2>(tab, key) && ok;
    }
    if (!ok) *flag = 1u;
    if (block) __syncthreads(); else __syncwarp();
    const bool linear = *flag != 0u;
    if (linear) {
        if (block) __syncthreads(); else __syncwarp();
        for (int s = tid; s < (1 << LOG2); s += nthreads) tab[s] = -1;
        if (block) __syncthreads(); else __syncwarp();
        for (int64_t t = ms + tid; t < me; t += nthreads) {
            const int32_t key = mcrd[t];
            if (key != skip) tc_linear_insert<LOG2>(tab, key);
        }
        if (block) __syncthreads(); else __syncwarp();
    }
    return linear;
}

// Streams the B rows named by entries [as, ae) of A's row and counts the elements
// found in the set.  Entries are taken in batches of 32: with `next`
// null the calling warp walks all batches itself; otherwise the warps of a CTA
// draw batch numbers from the shared counter `*next`, so a warp that meets short
// B rows simply draws more batches.  A batch's B-row bounds are fetched by the 32
// lanes at once and broadcast with shuffles, so the dependent chain
// acrd -> bpos -> bcrd is paid once per 32 entries.  Elements are read with
// 128-bit loads (four coordinates per lane, two loads in flight); a B row is
// entered at the 16-byte boundary below its first element and the elements
// outside [bs, be) are masked off.
template <int LOG2>
__device__ __forceinline__ unsigned long long tc_stream_rows(const int32_t *tab, bool linear,
                                                            int64_t as, int64_t ae, unsigned *next,
                                                            int lane, const int32_t *__restrict__ acrd,
                                                            const int64_t *__restrict__ bpos,
                                                            const int32_t *__restrict__ bcrd)
{
    unsigned long long total = 0;
    const int64_t nbatches = (ae - as + 31) >> 5;
    int64_t batch = 0;
    while (true) {
        if (next) {
            unsigned b = 0;
            if (lane == 0) b = atomicAdd(next, 1u);
            batch = __shfl_sync(0xffffffffu, b, 0);
        }
        if (batch >= nbatches) break;
        const int64_t pb = as + (batch << 5);
        int64_t bs_l = 0, be_l = 0;
        if (pb + lane < ae) {
            const int64_t k = __ldg(acrd + pb + lane);
            bs_l = __ldg(bpos + k);
            be_l = __ldg(bpos + k + 1);
        }
        const int n = (ae - pb) < 32 ? (int)(ae - pb) : 32;
        unsigned h32 = 0;
        for (int t = 0; t < n; t++) {
            const int64_t bs = __shfl_sync(0xffffffffu, (long long)bs_l, t);
            const int64_t be = __shfl_sync(0xffffffffu, (long long)be_l, t);
            for (int64_t q = (bs & ~(int64_t)3) + 4 * lane; q < be; q += 256) {
                int4 v0 = make_int4(0, 0, 0, 0), v1 = make_int4(0, 0, 0, 0);
                v0 = __ldg((const int4 *)(bcrd + q));
                const bool two = q + 128 < be;
                if (two) v1 = __ldg((const int4 *)(bcrd + q + 128));
                if (q >= bs && q + 3 < be) {
                    h32 += tc_probe<LOG2>(tab, linear, v0.x) + tc_probe<LOG2>(tab, linear, v0.y) +
                           tc_probe<LOG2>(tab, linear, v0.z) + tc_probe<LOG2>(tab, linear, v0.w);
                } else {
                    if (q >= bs) h32 += tc_probe<LOG2>(tab, linear, v0.x);
                    if (q + 1 >= bs && q + 1 < be) h32 += tc_probe<LOG2>(tab, linear, v0.y);
                    if (q + 2 >= bs && q + 2 < be) h32 += tc_probe<LOG2>(tab, linear, v0.z);
                    if (q + 3 >= bs && q + 3 < be) h32 += tc_probe<LOG2>(tab, linear, v0.w);
                }
                if (two) {
                    const int64_t r = q + 128;           // r >= bs always: it lies past the first vector
                    if (r + 3 < be) {
                        h32 += tc_probe<LOG2>(tab, linear, v1.x) + tc_probe<LOG2>(tab, linear, v1.y) +
                               tc_probe<LOG2>(tab, linear, v1.z) + tc_probe<LOG2>(tab, linear, v1.w);
                    } else {
                        h32 += tc_probe<LOG2>(tab, linear, v1.x);
                        if (r + 1 < be) h32 += tc_probe<LOG2>(tab, linear, v1.y);
                        if (r + 2 < be) h32 += tc_probe<LOG2>(tab, linear, v1.z);
                    }
                }
            }
        }
        total += h32;
        if (!next) batch++;
    }
    return total;
}

__global__ void __launch_bounds__(256)
tc_bin_kernel(int64_t row_lo, int64_t row_hi, const int64_t *__restrict__ apos,
              const int64_t *__restrict__ mpos, TcHeader *hdr, int32_t *__restrict__ list0,
              int32_t *__restrict__ list1, int32_t *__restrict__ slow, TcUnit *__restrict__ units,
              unsigned unit_cap)
{
    int64_t r = row_lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int bin = -1;
    int64_t al = 0, ml = 0;
    if (r < row_hi) {
        al = apos[r + 1] - apos[r];
        ml = mpos[r + 1] - mpos[r];
        if (al > 0 && ml > 0) bin = ml <= TC_WARP_MAX ? 0 : (ml <= TC_MID_MAX ? 1 : 2);
    }
    // one atomic per warp and bin
    const int lane = threadIdx.x & 31;
    for (int b = 0; b < 2; b++) {
        unsigned m = __ballot_sync(0xffffffffu, bin == b);
        if (!m) continue;
        unsigned base = 0;
        int leader = __ffs(m) - 1;
        if (lane == leader) base = atomicAdd(&hdr->count[b], (unsigned)__popc(m));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (bin == b) (b == 0 ? list0 : list1)[base + __popc(m & ((1u << lane) - 1u))] = (int32_t)r;
    }
    if (bin == 2) {
        const unsigned nseg = (unsigned)((ml + TC_BIG_SEG - 1) / TC_BIG_SEG);
        const unsigned nsl = (unsigned)((al + TC_BIG_SLICE - 1) / TC_BIG_SLICE);
        const unsigned long long want = (unsigned long long)nseg * nsl;
        bool placed = false;
        if (want <= unit_cap) {
            unsigned at = atomicAdd(&hdr->count[2], (unsigned)want);
            if ((unsigned long long)at + want <= unit_cap) {
                for (unsigned a = 0; a < nseg; a++)
                    for (unsigned b = 0; b < nsl; b++) {
                        TcUnit u;
                        u.row = (int32_t)r;
                        u.mask_off = (int32_t)(a * TC_BIG_SEG);
                        u.edge_off = (int32_t)(b * TC_BIG_SLICE);
                        units[at + a * nsl + b] = u;
                    }
                placed = true;
            } else if (at < unit_cap) {
                // the reservation ran past the end: neutralise the part of it that lies inside the list
                for (unsigned t = at; t < unit_cap; t++) { TcUnit u; u.row = -1; u.mask_off = 0; u.edge_off = 0; units[t] = u; }
            }
        }
        if (!placed) slow[atomicAdd(&hdr->count[3], 1u)] = (int32_t)r;   // whole row by one CTA
    }
}

__global__ void __launch_bounds__(TC_WARPS * 32)
tc_warp_kernel(TcHeader *hdr, const int32_t *__restrict__ list, const int64_t *__restrict__ apos,
               const int32_t *__restrict__ acrd, const int64_t *__restrict__ bpos,
               const int32_t *__restrict__ bcrd, const int64_t *__restrict__ mpos,
               const int32_t *__restrict__ mcrd, unsigned long long *__restrict__ count)
{
    __shared__ int32_t s_tab[TC_WARPS][1 << TC_WARP_LOG2];
    __shared__ unsigned s_flag[TC_WARPS];
    __shared__ unsigned long long s_part[TC_WARPS];
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned nlist = hdr->count[0];
    unsigned long long hits = 0;
    while (true) {
        unsigned idx = 0;
        if (lane == 0) idx = atomicAdd(&hdr->next[0], 1u);
        idx = __shfl_sync(0xffffffffu, idx, 0);
        if (idx >= nlist) break;
        const int64_t i = list[idx];
        const bool linear = tc_fill<TC_WARP_LOG2>(s_tab[w], &s_flag[w], mcrd, mpos[i], mpos[i + 1], lane, 32, false);
        hits += tc_stream_rows<TC_WARP_LOG2>(s_tab[w], linear, apos[i], apos[i + 1], nullptr,
                                                           lane, acrd, bpos, bcrd);
        __syncwarp();
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    if (lane == 0) s_part[w] = hits;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int i = 0; i < TC_WARPS; i++) t += s_part[i];
        if (t) atomicAdd(count, t);
    }
}

// MODE 0: list of rows, whole row per CTA (mask taken in segments of SEG entries).
// MODE 1: list of units (mask segment x slice of A's entries).
template <int THREADS, int LOG2, int SEG, int MODE>
__global__ void __launch_bounds__(THREADS)
tc_block_kernel(TcHeader *hdr, int which, const int32_t *__restrict__ list,
                const TcUnit *__restrict__ units, const int64_t *__restrict__ apos,
                const int32_t *__restrict__ acrd, const int64_t *__restrict__ bpos,
                const int32_t *__restrict__ bcrd, const int64_t *__restrict__ mpos,
                const int32_t *__restrict__ mcrd, unsigned unit_cap,
                unsigned long long *__restrict__ count)
{
    extern __shared__ int32_t s_dyn_tc[];
    __shared__ unsigned long long s_part[THREADS / 32];
    __shared__ unsigned s_idx, s_batch;
    int32_t *tab = s_dyn_tc;
    __shared__ unsigned s_flag;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned nlist = hdr->count[which];
    if (MODE == 1 && nlist > unit_cap) nlist = unit_cap;
    unsigned long long hits = 0;
    while (true) {
        if (threadIdx.x == 0) s_idx = atomicAdd(&hdr->next[which], 1u);
        __syncthreads();
        const unsigned idx = s_idx;
        __syncthreads();
        if (idx >= nlist) break;
        int64_t i, ms, me, as, ae;
        if (MODE == 1) {
            const TcUnit u = units[idx];
            if (u.row < 0) continue;
            i = u.row;
            ms = mpos[i] + u.mask_off;
            me = mpos[i + 1] < ms + SEG ? mpos[i + 1] : ms + SEG;
            as = apos[i] + u.edge_off;
            ae = apos[i + 1] < as + TC_BIG_SLICE ? apos[i + 1] : as + TC_BIG_SLICE;
        } else {
            i = list[idx];
            ms = mpos[i]; me = mpos[i + 1]; as = apos[i]; ae = apos[i + 1];
        }
        for (int64_t seg = ms; seg < me; seg += SEG) {
            const int64_t seg_end = seg + SEG < me ? seg + SEG : me;
            if (threadIdx.x == 0) s_batch = 0;
            const int32_t skip = seg > mpos[i] ? mcrd[seg - 1] : -1;     // last coordinate of the segment before
            const bool linear = tc_fill<LOG2>(tab, &s_flag, mcrd, seg, seg_end, threadIdx.x, THREADS, true, skip);
            hits += tc_stream_rows<LOG2>(tab, linear, as, ae, &s_batch, lane, acrd, bpos, bcrd);
            __syncthreads();
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) hits += __shfl_xor_sync(0xffffffffu, hits, o);
    if (lane == 0) s_part[w] = hits;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int i = 0; i < THREADS / 32; i++) t += s_part[i];
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
    if (ncols >= 0x7fffffffLL || row_hi >= 0x7fffffffLL)
        return fail("masked count: more than 2^31-1 rows or columns is not supported");
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
    const int64_t nrows = row_hi - row_lo;
    const size_t unit_cap = (size_t)(nnz_a / 256 + 65536);
    void *lists = nullptr, *hdrp = nullptr;
    CB_TRY(scratch(SLOT_BINS, (size_t)nrows * 3 * sizeof(int32_t) + unit_cap * sizeof(TcUnit), &lists));
    CB_TRY(scratch(SLOT_MISC, sizeof(TcHeader), &hdrp));
    TcHeader *hdr = (TcHeader *)hdrp;
    int32_t *list0 = (int32_t *)lists, *list1 = list0 + nrows, *slow = list1 + nrows;
    TcUnit *units = (TcUnit *)(slow + nrows);
    CB_CUDA(cudaMemsetAsync(hdr, 0, sizeof(TcHeader), st));
    tc_bin_kernel<<<(unsigned)ceil_div(nrows, 256), 256, 0, st>>>(row_lo, row_hi, apos, mpos, hdr, list0,
                                                                   list1, slow, units, (unsigned)unit_cap);
    CB_LAUNCH_CHECK();
    const int32_t *A = (const int32_t *)a32, *B = (const int32_t *)b32, *M = (const int32_t *)m32;
    unsigned long long *cnt = (unsigned long long *)count_dev;
    const unsigned sms = (unsigned)sm_count();
    {   // longest rows first
        constexpr int T = 512;
        const size_t smem = sizeof(int32_t) << TC_BIG_LOG2;
        auto kunits = tc_block_kernel<T, TC_BIG_LOG2, TC_BIG_SEG, 1>;
        auto kslow = tc_block_kernel<T, TC_BIG_LOG2, TC_BIG_SEG, 0>;
        CB_CUDA(cudaFuncSetAttribute(kunits, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        CB_CUDA(cudaFuncSetAttribute(kslow, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kunits<<<sms * 3, T, smem, st>>>(hdr, 2, nullptr, units, apos, A, bpos, B, mpos, M, (unsigned)unit_cap, cnt);
        CB_LAUNCH_CHECK();
        kslow<<<sms, T, smem, st>>>(hdr, 3, slow, nullptr, apos, A, bpos, B, mpos, M, (unsigned)unit_cap, cnt);
        CB_LAUNCH_CHECK();
    }
    {
        constexpr int T = 256;
        const size_t smem = sizeof(int32_t) << TC_MID_LOG2;
        tc_block_kernel<T, TC_MID_LOG2, TC_MID_MAX, 0><<<sms * 6, T, smem, st>>>(
            hdr, 1, list1, nullptr, apos, A, bpos, B, mpos, M, (unsigned)unit_cap, cnt);
        CB_LAUNCH_CHECK();
    }
    tc_warp_kernel<<<sms * 8, TC_WARPS * 32, 0, st>>>(hdr, list0, apos, A, bpos, B, mpos, M, cnt);
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
