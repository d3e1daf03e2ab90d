// The entry-stream SpMM with the rows of B staged by the TMA engine.
//
// Same decomposition as spmm_stream.cu (equal pieces of the entries + rows path of A, persistent warps,
// a ring of shared-memory stages per warp), but a stage is filled by BULK asynchronous copies instead of
// per-lane 16-byte cp.async: for each of the stage's rows one lane issues a single
// `cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes` of the whole row (K * 8 bytes), and
// the stage's mbarrier flips when all its bytes have landed.  That replaces 2 * SB_G copy instructions per
// lane per stage (K = 128) by one instruction for each of SB_G lanes, and the wait on copy groups by a wait
// on the barrier's phase.
//
// Every wait is bounded: a lane that does not see its stage's phase complete within the limit sets
// hdr->overflow = 2 in the work-list header, stops issuing and waiting for further stages, gives the copies
// already in flight the same bounded time to land, and leaves (the result is then incomplete; a correct run
// cannot get there, since a stage's expected byte count equals the bytes of the copies issued for it).
//
// A second form fills a stage with ONE instruction: the sm_100 tensor copy with four row coordinates,
// `cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4`, over a 2-D tensor map of this GPU's own B
// (box = one row of K doubles; the four rows named by the instruction land one after the other in shared
// memory, which is exactly a stage).  No cluster multicast anywhere.
//
// Selected with bits 24-25 of the SpMM variant = 3 (row-wise bulk copies) and bit 26 in addition (gather4);
// see the profiles for the measured differences to the cp.async kernel.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "stream.cuh"

namespace cb200 {

static const int ST_WARPS = 16;
static const int ST_G = 4;                      // rows of B per stage
static const int ST_RING_BYTES = 12 * 1024;     // per warp
static const int ST_SIDE_BYTES = 512 + 128;     // 32 column indices, 32 values, 32 row ends, up to 8 barriers; keeps every
                                                // warp's ring 128-byte aligned, which the tensor copy asks of its destination
static const unsigned ST_WAIT_LIMIT = 1u << 24; // polls of one barrier before giving up

__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint32_t bar, unsigned bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, unsigned parity)
{
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_row(uint32_t dst, const void *src, unsigned bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// four rows of the tensor behind `tmap`, columns from c0 on, rows r0..r3, into 4 consecutive rows at dst
__device__ __forceinline__ void gather4_rows(uint32_t dst, const CUtensorMap *tmap, int c0, int r0, int r1, int r2, int r3,
                                             uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes "
                 "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
                 ::"r"(dst), "l"(tmap), "r"(c0), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(bar) : "memory");
}

template <int NI, bool G4>
__global__ void __launch_bounds__(ST_WARPS * 32, 1)
spmm_stream_tma_kernel(const __grid_constant__ CUtensorMap tmap, int64_t nrows, int64_t nnz, unsigned nblocks,
                       const int64_t *__restrict__ row_ids,
                       const int64_t *__restrict__ pos, const int64_t *__restrict__ crd, const double *__restrict__ val,
                       const double *__restrict__ b, int64_t ldb, double *__restrict__ c, int64_t ldc, int k, int stages,
                       int accumulate, WorkHeader *hdr, const int64_t *__restrict__ block_row,
                       const int64_t *__restrict__ block_ent)
{
    extern __shared__ __align__(128) unsigned char st_smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int k2 = k >> 1;
    const uint32_t rowbytes = (uint32_t)k * 8u;
    const uint32_t stagebytes = rowbytes * ST_G;
    const uint32_t ringbytes = (uint32_t)stages * stagebytes;
    const uint32_t warpbytes = ringbytes + ST_SIDE_BYTES;
    unsigned char *ring = st_smem_raw + (size_t)warp * warpbytes;
    int32_t *cs = (int32_t *)(ring + ringbytes);
    double *vs = (double *)(cs + 32);
    int *ps = (int *)(vs + 32);
    const uint32_t bars = sb_smem(ps + 32);             // `stages` 8-byte barriers, 8-byte aligned
    const uint32_t ring_s = sb_smem(ring);
    bool on[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) on[i] = lane + i * 32 < k2;

    if (lane == 0)
        for (int s = 0; s < stages; s++) mbar_init(bars + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncwarp();

    unsigned fill = 0;      // stages filled so far by this warp (stage = fill % stages, phase parity = (fill / stages) & 1)
    unsigned used = 0;      // stages consumed so far
    bool dead = false;      // a wait ran out: stop issuing and waiting

    while (!dead) {
        unsigned blk = 0;
        if (lane == 0) blk = atomicAdd(&hdr->pad[0], 1u);
        blk = __shfl_sync(0xffffffffu, blk, 0);
        if (blk >= nblocks) break;
        const int64_t n0 = block_ent[blk];
        const int cnt = (int)(block_ent[blk + 1] - n0);
        const int64_t rend = block_row[blk + 1];
        const int ngroups = (cnt + ST_G - 1) / ST_G;
        const int64_t *crd0 = crd + n0;
        const double *val0 = val + n0;

        int64_t r = block_row[blk];
        const int64_t far = (int64_t)cnt + 1;
        const int64_t d = pos[r] - n0;
        int rs = d < -1 ? -1 : (int)d;
        int64_t rb = r;
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

        // fills the next stage of the ring with the rows of group g (nothing past the end of the piece)
        auto issue = [&](int g) {
            if (g >= ngroups) return;
            const int off = (g * ST_G) & 31;
            if (off == 0) {
                cs[lane] = cnext;
                const int nb = g * ST_G + 32 + lane;
                cnext = (nb < cnt) ? (int32_t)ld_stream(crd0 + nb) : 0;
                __syncwarp();
            }
            const int m = (cnt - g * ST_G) < ST_G ? (cnt - g * ST_G) : ST_G;
            const unsigned s = fill % (unsigned)stages;
            const uint32_t bar = bars + 8u * s;
            if (G4) {
                // one instruction for the stage; a stage at the end of a piece with fewer than four entries names
                // its last row again (the copies beyond m are not read)
                __syncwarp();                            // every lane is done reading the stage this one replaces
                if (lane == 0) {
                    const int4 c4 = *(const int4 *)(cs + off);
                    const int r0 = c4.x, r1 = m > 1 ? c4.y : r0, r2 = m > 2 ? c4.z : r1, r3 = m > 3 ? c4.w : r2;
                    mbar_expect(bar, stagebytes);
                    gather4_rows(ring_s + s * stagebytes, &tmap, 0, r0, r1, r2, r3, bar);
                }
            } else {
                if (lane == 0) mbar_expect(bar, (unsigned)m * rowbytes);
                __syncwarp();
                if (lane < m) {
                    const int col = cs[off + lane];
                    bulk_row(ring_s + s * stagebytes + (uint32_t)lane * rowbytes, (const char *)b + (int64_t)col * ldb * 8,
                             rowbytes, bar);
                }
            }
            fill++;
        };

        const unsigned fill0 = fill;                     // the piece's group g sits in stage number fill0 + g
        for (int g = 0; g < stages - 1; g++) issue(g);

        for (int g = 0; g < ngroups && !dead; g++) {
            const int off = (g * ST_G) & 31;
            if (off == 0) {
                vs[lane] = vnext;
                const int nb = g * ST_G + 32 + lane;
                vnext = (nb < cnt) ? ld_stream(val0 + nb) : 0.0;
            }
            issue(g + stages - 1);
            const unsigned s = used % (unsigned)stages, parity = (used / (unsigned)stages) & 1u;
            unsigned polls = 0;
            while (!mbar_try(bars + 8u * s, parity)) {
                if (++polls > ST_WAIT_LIMIT) { dead = true; break; }
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead) { if (lane == 0) hdr->overflow = 2; break; }
            used++;
            __syncwarp();
            const double2 *src = (const double2 *)(ring + s * stagebytes) + lane;
            double2 bv[ST_G][NI];
#pragma unroll
            for (int t = 0; t < ST_G; t++)
#pragma unroll
                for (int i = 0; i < NI; i++) bv[t][i] = on[i] ? src[t * k2 + i * 32] : make_double2(0.0, 0.0);
            const double2 v01 = *(const double2 *)(vs + off), v23 = *(const double2 *)(vs + off + 2);
            const double vv[4] = {v01.x, v01.y, v23.x, v23.y};
            const int j0 = g * ST_G;
            if (j0 + ST_G <= re && j0 + ST_G <= cnt) {
#pragma unroll
                for (int t = 0; t < ST_G; t++)
#pragma unroll
                    for (int i = 0; i < NI; i++) {
                        acc[i].x = fma(vv[t], bv[t][i].x, acc[i].x);
                        acc[i].y = fma(vv[t], bv[t][i].y, acc[i].y);
                    }
            } else {
#pragma unroll
                for (int t = 0; t < ST_G; t++) {
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
            __syncwarp();                               // every lane has read the stage before it is refilled
        }
        (void)fill0;
        if (dead) break;
        while (r < rend) next_row();
        if (rend < nrows && n0 + cnt > pos[rend]) flush(false);
    }
    // copies still in flight target this CTA's shared memory: wait for every stage that was filled and not
    // consumed (only after a wait ran out), within the same limit, before the CTA may exit
    while (used < fill) {
        const unsigned s = used % (unsigned)stages, parity = (used / (unsigned)stages) & 1u;
        unsigned polls = 0;
        while (!mbar_try(bars + 8u * s, parity) && ++polls <= ST_WAIT_LIMIT) {}
        used++;
    }
}

// 2-D tensor map of B for the gather4 form: dimension 0 = the K columns of a row, dimension 1 = the rows,
// box = one row.  cuTensorMapEncodeTiled is looked up through the runtime, so the library does not link libcuda.
static int make_row_map(const double *b, int64_t nrows_b, int64_t k, int64_t ldb, CUtensorMap *map)
{
    typedef CUresult (*Encode)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                               const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
            q != cudaDriverEntryPointSuccess)
            return fail("spmm: cuTensorMapEncodeTiled is not available from this driver");
        encode = (Encode)fn;
    }
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)nrows_b};
    const cuuint64_t strides[1] = {(cuuint64_t)ldb * 8};
    const cuuint32_t box[2] = {(cuuint32_t)k, 1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT64, 2, (void *)b, dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("spmm: cuTensorMapEncodeTiled refused the map of B (error %d)", (int)r);
    return 0;
}

// Returns 1 when this path took the call, 0 when the shape is not one it handles, -1 on error.
int spmm_stream_tma(int64_t nrows, int64_t ncols, int64_t nnz, int64_t k, const int64_t *row_ids, const int64_t *pos,
                    const int64_t *crd, const double *val, const double *b, int64_t ldb, double *c, int64_t ldc,
                    int accumulate, bool gather4, cudaStream_t st)
{
    // bulk copies need 16-byte aligned rows whose size is a multiple of 16 bytes
    if (k < 2 || k > 256 || (k & 1) || (ldb & 1) || (ldc & 1) || ((((uintptr_t)b | (uintptr_t)c) & 15) != 0)) return 0;
    if (nnz < 1 || nrows <= 0 || ncols > 0x7fffffffLL) return 0;
    const int rowbytes = (int)k * 8;
    int stages = ST_RING_BYTES / (ST_G * rowbytes);
    if (stages > 8) stages = 8;
    if (stages < 2) return 0;
    const size_t smem = (size_t)ST_WARPS * ((size_t)stages * ST_G * rowbytes + ST_SIDE_BYTES);
    alignas(64) CUtensorMap map;
    memset(&map, 0, sizeof(map));
    if (gather4) {
        // every stage must start on a 128-byte boundary of shared memory: rows of at least 32 bytes
        if ((ST_G * rowbytes) % 128 != 0 || ldb * 8 >= (1LL << 40)) return 0;
        if (make_row_map(b, ncols, k, ldb, &map)) return -1;
    }

    StreamPlan plan;
    const int planned = stream_plan(nrows, nnz, (int64_t)sm_count() * ST_WARPS, row_ids, pos, c, ldc, (int)k, accumulate,
                                    st, &plan);
    if (planned <= 0) return planned;
    int64_t grid = ceil_div(plan.nblocks, ST_WARPS);
    if (grid > sm_count()) grid = sm_count();
    const int ni = k <= 64 ? 1 : (k <= 128 ? 2 : 4);
#define ST_LAUNCH(NN, GG)                                                                                              \
    do {                                                                                                               \
        if (cudaFuncSetAttribute(spmm_stream_tma_kernel<NN, GG>, cudaFuncAttributeMaxDynamicSharedMemorySize,         \
                                 ST_WARPS * (ST_RING_BYTES + ST_SIDE_BYTES)) != cudaSuccess) {                         \
            fail("spmm: shared memory size refused");                                                                  \
            return -1;                                                                                                 \
        }                                                                                                              \
        spmm_stream_tma_kernel<NN, GG><<<(unsigned)grid, ST_WARPS * 32, smem, st>>>(                                   \
            map, nrows, nnz, (unsigned)plan.nblocks, row_ids, pos, crd, val, b, ldb, c, ldc, (int)k, stages,           \
            accumulate, plan.hdr, plan.block_row, plan.block_ent);                                                     \
    } while (0)
    if (gather4) {
        if (ni == 1) ST_LAUNCH(1, true);
        else if (ni == 2) ST_LAUNCH(2, true);
        else ST_LAUNCH(4, true);
    } else {
        if (ni == 1) ST_LAUNCH(1, false);
        else if (ni == 2) ST_LAUNCH(2, false);
        else ST_LAUNCH(4, false);
    }
#undef ST_LAUNCH
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        fail("spmm: launch failed: %s", cudaGetErrorString(e));
        return -1;
    }
    return 1;
}

}  // namespace cb200
