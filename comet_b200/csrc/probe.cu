// Measurement aid: the bare gather that SpMM and SDDMM are built around, with nothing else in the
// kernel -- for every stored entry, the row of the dense operand its column index names is read
// (128-bit loads) and folded into a running sum, eight rows in flight per warp.  No multiply by A's
// values, no row bookkeeping, one 8-byte store per warp at the end.  Its time over a benchmark's column
// stream is the ceiling a gather-per-entry kernel can reach on that stream: the L2 -> SM rate when the
// rows named fit L2 (`fold` > 0 maps every index into the first `fold` rows), the blend of L2 hits and
// DRAM misses otherwise.
#include "common.cuh"

namespace cb200 {

template <int NI>
__global__ void __launch_bounds__(256)
gather_probe_kernel(int64_t nnz, const int64_t *__restrict__ crd, const double *__restrict__ b, int64_t ldb, int k2,
                    int64_t fold, double *__restrict__ out)
{
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t per = (nnz + nwarps - 1) / nwarps;
    int64_t s = warp * per, e = s + per;
    if (e > nnz) e = nnz;
    double2 acc[NI];
#pragma unroll
    for (int i = 0; i < NI; i++) acc[i] = make_double2(0.0, 0.0);
    for (int64_t base = s; base < e; base += 32) {
        int64_t c = 0;
        if (base + lane < e) {
            c = ld_stream(crd + base + lane);
            if (fold > 0) c %= fold;
        }
        const int n = (e - base) < 32 ? (int)(e - base) : 32;
        for (int t0 = 0; t0 < n; t0 += 8) {
            double2 v[8][NI];
#pragma unroll
            for (int t = 0; t < 8; t++) {
                const int64_t cc = __shfl_sync(0xffffffffu, (long long)c, (t0 + t) & 31);
                const double2 *row = (const double2 *)(b + cc * ldb);
#pragma unroll
                for (int i = 0; i < NI; i++)
                    v[t][i] = (t0 + t < n && lane + i * 32 < k2) ? __ldg(row + lane + i * 32) : make_double2(0.0, 0.0);
            }
#pragma unroll
            for (int t = 0; t < 8; t++)
#pragma unroll
                for (int i = 0; i < NI; i++) { acc[i].x += v[t][i].x; acc[i].y += v[t][i].y; }
        }
    }
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < NI; i++) sum += acc[i].x + acc[i].y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) out[warp] = sum;
}

__global__ void noop_kernel() {}

}  // namespace cb200

// Measurement aid: an empty kernel on `stream`.  A CUDA graph of these, replayed, gives the floor any
// back-to-back sequence of small launches sits on (the benchmark prints it next to the SpMV figure).
extern "C" int32_t comet_b200_dev_noop(void *stream)
{
    using namespace cb200;
    noop_kernel<<<1, 32, 0, (cudaStream_t)stream>>>();
    CB_LAUNCH_CHECK();
    return 0;
}

extern "C" int32_t comet_b200_dev_gather_probe_f64_i64(int64_t nnz, const int64_t *crd, const double *b, int64_t ldb,
                                                       int64_t k, int64_t fold_rows, int32_t ctas_per_sm, double *out,
                                                       int64_t out_len, void *stream)
{
    using namespace cb200;
    clear_error();
    if (k < 2 || k > 256 || (k & 1) || (ldb & 1) || (((uintptr_t)b) & 15)) return fail("gather probe: K even, at most 256, B 16-byte aligned");
    if (ctas_per_sm < 1) ctas_per_sm = 8;
    const int64_t grid = (int64_t)sm_count() * ctas_per_sm;
    if (out_len < grid * 8) return fail("gather probe: out must hold %lld doubles", (long long)(grid * 8));
    if (nnz <= 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    const int k2 = (int)k / 2;
    if (k <= 64) gather_probe_kernel<1><<<(unsigned)grid, 256, 0, st>>>(nnz, crd, b, ldb, k2, fold_rows, out);
    else if (k <= 128) gather_probe_kernel<2><<<(unsigned)grid, 256, 0, st>>>(nnz, crd, b, ldb, k2, fold_rows, out);
    else gather_probe_kernel<4><<<(unsigned)grid, 256, 0, st>>>(nnz, crd, b, ldb, k2, fold_rows, out);
    CB_LAUNCH_CHECK();
    return 0;
}
