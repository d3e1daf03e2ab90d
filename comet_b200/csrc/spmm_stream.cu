// SpMM over the entry stream, rows of B staged in shared memory by asynchronous copies.
//
// The row-panel kernels of spmm.cu keep the gathered rows of B in flight in
// registers and hand out whole rows of A, so a power-law matrix needs a second
// pass for its hub rows and the bytes in flight follow occupancy.  Here every
// warp owns a ring of shared-memory stages (SB_G rows of B each) and a piece of
// the ENTRY stream of A: per stored entry its lanes issue 16-byte cp.async
// copies of B[crd, :] into the ring, several stages ahead of the stage being
// multiplied, so the gather runs ahead of the arithmetic without holding
// registers.  (One bulk copy per row -- cp.async.bulk completing on an
// mbarrier -- was measured first and was slower: 1 KB per copy is too little
// work per copy instruction, 6.1 ms against 1.2 ms on R-MAT scale 20, K = 128.)
//
// Work is cut along the path that walks A row by row, one step per stored entry
// and one per row end, into equal pieces; persistent warps draw pieces from a
// counter.  A hub row is therefore shared by many warps and a run of empty rows
// by several, with no separate long-row pass.  A row that lies inside one piece
// is written with plain stores; a row cut by a boundary is added with f64
// atomics (onto zeros written by the plan kernel when the call does not
// accumulate), so its summation order is not fixed and differences stay at
// rounding level.
//
// Bound: HBM.  Algorithmic bytes = 8(n+1) + 16 nnz + 8 ncols K + 8 nrows K.
#include "common.cuh"
#include "stream.cuh"

namespace cb200 {

static const int SB_WARPS = 16;                // warps per CTA, one CTA per SM
static const int SB_G = 4;                     // rows of B per stage (one copy group)
static const int SB_MAX_STAGES = 8;
static const int SB_RING_BYTES = 12 * 1024;    // per warp
static const int SB_SIDE_BYTES = 512;           // per warp: 32 column indices, 32 values of A, 32 row ends

// Blocks are equal pieces of the path that walks A row by row: one step per stored entry and one
// step per row end (a row costs about as much as an entry: its result is written, or zeros for an
// empty row).  One warp per block boundary b finds where the path stands after b*q steps: inside
// row block_row[b], at entry block_ent[b].  When the call does not accumulate, a row that a
// boundary cuts gets zeros here: its parts are added with atomics.
__global__ void __launch_bounds__(256)
spmm_stream_plan_kernel(int64_t nrows, int64_t nnz, int64_t q, int64_t nblocks, const int64_t *__restrict__ row_ids,
                        const int64_t *__restrict__ pos, double *__restrict__ c, int64_t ldc, int k, int accumulate,
                        int64_t *__restrict__ block_row, int64_t *__restrict__ block_ent)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = warp; b <= nblocks; b += nwarps) {
        int64_t d = b * q;
        if (d > nnz + nrows) d = nnz + nrows;
        // largest r in [0, nrows] with pos[r] + r <= d: the 32 lanes probe 32 points of the range per step
        int64_t lo = 0, hi = nrows;
        while (lo < hi) {
            const int64_t step = (hi - lo + 31) / 32;
            int64_t probe = lo + (lane + 1) * step;
            if (probe > hi) probe = hi;
            const int k = __popc(__ballot_sync(0xffffffffu, pos[probe] + probe <= d));   // the first k probes hold
            const int64_t fail_at = lo + (int64_t)(k + 1) * step;                             // probe k does not (if k < 32)
            if (k > 0) { lo += (int64_t)k * step; if (lo > hi) lo = hi; }
            if (k < 32) hi = (fail_at < hi ? fail_at : hi) - 1;                               // the answer lies before probe k
        }
        int64_t r = lo, e = d - lo;
        if (b > 0 && r < nrows && e >= pos[r + 1]) {   // the boundary is the end of row r: start at the next row
            e = pos[r + 1];
            r += 1;
        }
        if (lane == 0) {
            block_row[b] = r;
            block_ent[b] = e;
        }
        if (!accumulate && b > 0 && b < nblocks && r < nrows && e > pos[r]) {
            const int64_t out = row_ids ? row_ids[r] : r;
            double2 *crow = (double2 *)(c + out * ldc);
            for (int j = lane; j < k / 2; j += 32) crow[j] = make_double2(0.0, 0.0);
        }
    }
}

template <int NI, bool FULLK>
__global__ void __launch_bounds__(SB_WARPS * 32, 1)
spmm_stream_kernel(int64_t nrows, int64_t nnz, int64_t q, unsigned nblocks, const int64_t *__restrict__ row_ids,
                   const int64_t *__restrict__ pos, const int64_t *__restrict__ crd, const double *__restrict__ val,
                   const double *__restrict__ b, int64_t ldb, double *__restrict__ c, int64_t ldc, int k, int stages_arg,
                   int accumulate, WorkHeader *hdr, const int64_t *__restrict__ block_row,
                   const int64_t *__restrict__ block_ent)
{
    // per warp: a ring of `stages` stages of SB_G rows of B, then 32 column indices and 32 values of A
    extern __shared__ __align__(128) unsigned char sb_smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    // K = 64 NI is the common case: every size below is then a compile-time constant
    const int stages = FULLK ? SB_RING_BYTES / (SB_G * NI * 512) : stages_arg;
    const int k2 = FULLK ? NI * 32 : (k >> 1);          // double2 vectors per row
    const uint32_t rowbytes = FULLK ? (uint32_t)NI * 512u : (uint32_t)k * 8u;
    const uint32_t stagebytes = rowbytes * SB_G;
    const uint32_t warpbytes = (uint32_t)stages * stagebytes + SB_SIDE_BYTES;
    unsigned char *ring = sb_smem_raw + (size_t)warp * warpbytes;
    int32_t *cs = (int32_t *)(ring + (size_t)stages * stagebytes);
    double *vs = (double *)(cs + 32);
    int *ps = (int *)(vs + 32);                         // block-local end positions of 32 consecutive rows
    const uint32_t ring_s = sb_smem(ring) + (uint32_t)lane * 16u;
    const char *bl = (const char *)b + lane * 16;
    const int64_t ldb8 = ldb * 8;
    bool on[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) on[i] = FULLK || (lane + i * 32 < k2);

    uint32_t pofs = 0;               // byte offset of the stage the next issue fills
    uint32_t cofs = 0;               // byte offset of the stage the next wait reads
    const uint32_t ringbytes = (uint32_t)stages * stagebytes;

    while (true) {
        unsigned blk = 0;
        if (lane == 0) blk = atomicAdd(&hdr->pad[0], 1u);
        blk = __shfl_sync(0xffffffffu, blk, 0);
        if (blk >= nblocks) break;
        const int64_t n0 = block_ent[blk];
        const int cnt = (int)(block_ent[blk + 1] - n0);
        const int64_t rend = block_row[blk + 1];        // rows before rend end in this block
        const int ngroups = (cnt + SB_G - 1) / SB_G;
        const int64_t *crd0 = crd + n0;
        const double *val0 = val + n0;

        // rows: r is the row of the entry being consumed; its entries are [rs, re) in block-local positions
        int64_t r = block_row[blk];
        const int64_t far = (int64_t)cnt + 1;
        const int64_t d = pos[r] - n0;
        int rs = d < -1 ? -1 : (int)d;                  // -1: the row starts before the block
        int64_t rb = r;                                 // ps[i] = end of row rb + i; cnt + 1: it ends after the block
        auto load_ends = [&]() {
            __syncwarp();
            int64_t e = far;
            if (rb + lane < nrows) {
                e = pos[rb + lane + 1] - n0;
                if (e > far) e = far;
            }
            ps[lane] = (int)e;
            __syncwarp();
        };
        load_ends();
        int re = ps[0];

        int32_t cnext = (lane < cnt) ? (int32_t)ld_stream(crd0 + lane) : 0;
        double vnext = (lane < cnt) ? ld_stream(val0 + lane) : 0.0;

        double2 acc[NI];
#pragma unroll
        for (int i = 0; i < NI; i++) acc[i] = make_double2(0.0, 0.0);

        // write out the finished row r and clear the accumulators
        auto flush = [&](bool whole) {
            const int64_t out = row_ids ? row_ids[r] : r;
            double *crow = c + out * ldc;
            if (whole) {
                if (!accumulate || rs < re) {
#pragma unroll
                    for (int i = 0; i < NI; i++) {
                        const int j = lane + i * 32;
                        if (on[i]) {
                            double2 o = acc[i];
                            if (accumulate) {
                                const double2 old = __ldcs((const double2 *)crow + j);
                                o.x += old.x;
                                o.y += old.y;
                            }
                            __stcs((double2 *)crow + j, o);
                        }
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < NI; i++) {
                    const int j = lane + i * 32;
                    if (on[i]) {
                        atomicAdd(crow + 2 * j, acc[i].x);
                        atomicAdd(crow + 2 * j + 1, acc[i].y);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < NI; i++) acc[i] = make_double2(0.0, 0.0);
        };
        auto next_row = [&]() {
            flush(rs >= 0);
            r += 1;
            rs = re;
            if (r - rb == 32) {
                rb = r;
                load_ends();
            }
            re = ps[r - rb];
        };

        // every call commits one copy group (an empty one past the end of the block), so "all but
        // stages-1 groups have landed" always means the stage about to be read has landed
        auto issue = [&](int g) {
            if (g < ngroups) {
                const int off = (g * SB_G) & 31;
                if (off == 0) {
                    cs[lane] = cnext;
                    const int nb = g * SB_G + 32 + lane;
                    cnext = (nb < cnt) ? (int32_t)ld_stream(crd0 + nb) : 0;
                    __syncwarp();
                }
                const int4 c4 = *(const int4 *)(cs + off);          // broadcast read of four column indices
                const int cc[4] = {c4.x, c4.y, c4.z, c4.w};
                const uint32_t dst = ring_s + pofs;
                const int m = cnt - g * SB_G;
                if (m >= SB_G) {
#pragma unroll
                    for (int t = 0; t < SB_G; t++) {
                        const char *src = bl + (int64_t)cc[t] * ldb8;
#pragma unroll
                        for (int i = 0; i < NI; i++)
                            if (on[i]) sb_copy16(dst + (uint32_t)t * rowbytes + (uint32_t)i * 512u, src + i * 512);
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < SB_G; t++) {
                        if (t < m) {
                            const char *src = bl + (int64_t)cc[t] * ldb8;
#pragma unroll
                            for (int i = 0; i < NI; i++)
                                if (on[i]) sb_copy16(dst + (uint32_t)t * rowbytes + (uint32_t)i * 512u, src + i * 512);
                        }
                    }
                }
                pofs += stagebytes;
                if (pofs == ringbytes) pofs = 0;
            }
            sb_commit();
        };

        for (int g = 0; g < stages - 1; g++) issue(g);

        for (int g = 0; g < ngroups; g++) {
            const int off = (g * SB_G) & 31;
            if (off == 0) {
                vs[lane] = vnext;
                const int nb = g * SB_G + 32 + lane;
                vnext = (nb < cnt) ? ld_stream(val0 + nb) : 0.0;
            }
            issue(g + stages - 1);
            if (FULLK && NI == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");        // stages - 1
            else if (FULLK && NI == 1) asm volatile("cp.async.wait_group 5;" ::: "memory");
            else sb_wait_pending(stages - 1);
            __syncwarp();                               // the other lanes' copies of this stage have landed too
            const double2 *src = (const double2 *)(ring + cofs) + lane;
            double2 bv[SB_G][NI];
#pragma unroll
            for (int t = 0; t < SB_G; t++)
#pragma unroll
                for (int i = 0; i < NI; i++) bv[t][i] = on[i] ? src[t * k2 + i * 32] : make_double2(0.0, 0.0);
            const double2 v01 = *(const double2 *)(vs + off), v23 = *(const double2 *)(vs + off + 2);
            const double vv[4] = {v01.x, v01.y, v23.x, v23.y};
            const int j0 = g * SB_G;
            if (j0 + SB_G <= re && j0 + SB_G <= cnt) {  // the four entries belong to the row in progress
#pragma unroll
                for (int t = 0; t < SB_G; t++)
#pragma unroll
                    for (int i = 0; i < NI; i++) {
                        acc[i].x = fma(vv[t], bv[t][i].x, acc[i].x);
                        acc[i].y = fma(vv[t], bv[t][i].y, acc[i].y);
                    }
            } else {
#pragma unroll
                for (int t = 0; t < SB_G; t++) {
                    if (j0 + t < cnt) {
                        while (j0 + t >= re) next_row();
#pragma unroll
                        for (int i = 0; i < NI; i++) {
                            acc[i].x = fma(vv[t], bv[t][i].x, acc[i].x);
                            acc[i].y = fma(vv[t], bv[t][i].y, acc[i].y);
                        }
                    }
                }
            }
            cofs += stagebytes;
            if (cofs == ringbytes) cofs = 0;
            __syncwarp();                               // every lane has read the stage before it is refilled
        }

        // rows that end in this block (the one in progress, empty ones after it), then the part of
        // row rend this block holds, if the boundary cuts that row
        while (r < rend) next_row();
        if (rend < nrows && n0 + cnt > pos[rend]) flush(false);
    }
}

// Cuts the (entries + rows) path of a CSR matrix into pieces for `warps` persistent warps and runs the plan
// kernel.  c != null and accumulate == 0: rows cut by a boundary get zeros (k columns).  Returns 1, 0 when the
// piece count does not fit 32 bits, -1 on error.  The plan lives in the work-list scratch slot of the device.
int stream_plan(int64_t nrows, int64_t nnz, int64_t warps, const int64_t *row_ids, const int64_t *pos, double *c,
                int64_t ldc, int k, int accumulate, cudaStream_t st, StreamPlan *out)
{
    const int64_t steps = nnz + nrows;                 // path length: one step per entry, one per row end
    int64_t q = ceil_div(steps, warps * 8);
    if (q < 512) q = 512;
    const int64_t nblocks = ceil_div(steps, q);
    if (nblocks > 0x7ffffff0LL) return 0;
    void *wl = nullptr;
    if (scratch(SLOT_WORKLIST, sizeof(WorkHeader) + (size_t)(nblocks + 1) * 2 * sizeof(int64_t), &wl)) return -1;
    out->hdr = (WorkHeader *)wl;
    out->block_row = (int64_t *)((char *)wl + sizeof(WorkHeader));
    out->block_ent = out->block_row + (nblocks + 1);
    out->q = q;
    out->nblocks = nblocks;
    if (cudaMemsetAsync(out->hdr, 0, sizeof(WorkHeader), st) != cudaSuccess) {
        fail("clearing the block counter failed");
        return -1;
    }
    const int64_t pgrid = ceil_div((nblocks + 1) * 32, 256);
    spmm_stream_plan_kernel<<<(unsigned)pgrid, 256, 0, st>>>(nrows, nnz, q, nblocks, row_ids, pos, c, ldc, k,
                                                            c ? accumulate : 1, out->block_row, out->block_ent);
    return 1;
}

// Returns 1 when this path took the call, 0 when the shape is not one it handles, -1 on error.
int spmm_stream(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k, const int64_t *row_ids, const int64_t *pos,
                const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
                int accumulate, bool forced, cudaStream_t st)
{
    // 16-byte copies need aligned rows; the lane layout covers up to 256 columns
    if (k < 2 || k > 256 || (k & 1) || (ldb & 1) || (ldc & 1) || ((((uintptr_t)b | (uintptr_t)c) & 15) != 0)) return 0;
    if (nnz < (forced ? 1 : (1 << 16)) || nrows <= 0 || ncols > 0x7fffffffLL) return 0;   // column indices travel as int32
    const int rowbytes = (int)k * 8;
    int stages = SB_RING_BYTES / (SB_G * rowbytes);
    if (stages > SB_MAX_STAGES) stages = SB_MAX_STAGES;
    if (stages < 2) return 0;
    const size_t smem = (size_t)SB_WARPS * ((size_t)stages * SB_G * rowbytes + SB_SIDE_BYTES);

    StreamPlan plan;
    const int planned = stream_plan(nrows, nnz, (int64_t)sm_count() * SB_WARPS, row_ids, pos, c, ldc, (int)k, accumulate,
                                    st, &plan);
    if (planned <= 0) return planned;
    WorkHeader *hdr = plan.hdr;
    const int64_t *block_row = plan.block_row, *block_ent = plan.block_ent;
    const int64_t q = plan.q, nblocks = plan.nblocks;
    int64_t grid = ceil_div(nblocks, SB_WARPS);
    if (grid > sm_count()) grid = sm_count();
    const int ni = k <= 64 ? 1 : (k <= 128 ? 2 : 4);
#define SB_LAUNCH(NN, FK)                                                                                              \
    do {                                                                                                           \
        static bool attr_set[64] = {false};                                                                        \
        int d = 0;                                                                                                 \
        cudaGetDevice(&d);                                                                                         \
        if (d >= 0 && d < 64 && !attr_set[d]) {                                                                    \
            if (cudaFuncSetAttribute(spmm_stream_kernel<NN, FK>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                                     SB_WARPS * (SB_RING_BYTES + SB_SIDE_BYTES)) != cudaSuccess) {                    \
                fail("spmm: shared memory size refused");                                                          \
                return -1;                                                                                         \
            }                                                                                                      \
            attr_set[d] = true;                                                                                    \
        }                                                                                                          \
        spmm_stream_kernel<NN, FK><<<(unsigned)grid, SB_WARPS * 32, smem, st>>>(                                       \
            nrows, nnz, q, (unsigned)nblocks, row_ids, pos, crd, val, b, ldb, c, ldc, (int)k, stages, accumulate,  \
            hdr, block_row, block_ent);                                                                                       \
    } while (0)
    const bool fullk = (k == 64 * ni);
    if (ni == 1 && fullk) SB_LAUNCH(1, true);
    else if (ni == 1) SB_LAUNCH(1, false);
    else if (ni == 2 && fullk) SB_LAUNCH(2, true);
    else if (ni == 2) SB_LAUNCH(2, false);
    else if (fullk) SB_LAUNCH(4, true);
    else SB_LAUNCH(4, false);
#undef SB_LAUNCH
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fail("spmm: launch failed: %s", cudaGetErrorString(e));
        return -1;
    }
    return 1;
}

}  // namespace cb200
