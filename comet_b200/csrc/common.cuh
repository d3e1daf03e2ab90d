// Shared host/device helpers of libcomet_b200 (sm_100a only).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/comet_b200.h"

namespace cb200 {

// ---------------------------------------------------------------------------
// Errors.  COMET's runtime reports a failure on stderr and exits
// (lib/ExecutionEngine/SparseUtils.cpp:158-168); that stays the default.  With
// COMET_B200_ON_ERROR=return (or comet_b200_set_error_mode(1)) the message is
// kept for comet_b200_last_error() and the call returns, so host-side fault
// tests can observe it.
// ---------------------------------------------------------------------------
int fail(const char *fmt, ...);   // always returns a non-zero status
void clear_error();

// With COMET_B200_TRACE set, phases of the host entry points are logged on stderr with a wall-clock
// stamp (milliseconds since the first line): where the time of an end-to-end call goes.
void trace(const char *fmt, ...);

#define CB_CUDA(expr)                                                               \
    do {                                                                            \
        cudaError_t e_ = (expr);                                                    \
        if (e_ != cudaSuccess)                                                      \
            return cb200::fail("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e_), \
                               __FILE__, __LINE__);                                 \
    } while (0)

#define CB_TRY(expr)                 \
    do {                             \
        int s_ = (expr);             \
        if (s_ != 0) return s_;      \
    } while (0)

#define CB_LAUNCH_CHECK() CB_CUDA(cudaGetLastError())

// ---------------------------------------------------------------------------
// Scratch memory.  One growing allocation per (device, slot); a slot keeps its
// buffer between calls so steady-state calls allocate nothing.
// ---------------------------------------------------------------------------
enum Slot {
    SLOT_WORKLIST = 0,   // long-row chunk lists + counters of the row-parallel kernels
    SLOT_NARROW_A,       // int32 copies of crd arrays
    SLOT_NARROW_B,
    SLOT_NARROW_M,
    SLOT_ROWINFO,        // per-row counts / upper bounds
    SLOT_BINS,           // row lists per bin
    SLOT_SCAN,           // block sums of the exclusive scan
    SLOT_BITMAP,         // per-CTA global bitmaps when a row of columns exceeds shared memory
    SLOT_POS,            // COO -> row pointer adapter
    SLOT_MISC,
    SLOT_TEAMS,          // team item list of the SpGEMM numeric pass
    SLOT_H2D_0, SLOT_H2D_1, SLOT_H2D_2, SLOT_H2D_3, SLOT_H2D_4, SLOT_H2D_5,
    SLOT_H2D_6, SLOT_H2D_7, SLOT_H2D_8, SLOT_H2D_9, SLOT_H2D_10, SLOT_H2D_11,
    SLOT_COUNT
};
int scratch(Slot slot, size_t bytes, void **ptr);   // status; *ptr valid until the slot grows
void scratch_release_all();

int sm_count();
cudaStream_t lib_stream();   // the library's own stream for the host-memref entry points
cudaStream_t aux_stream(int i);   // two more streams (i = 0, 1) for copies that overlap with compute

// ---------------------------------------------------------------------------
// Small shared kernels (util.cu)
// ---------------------------------------------------------------------------
int narrow_i64_to_i32(const int64_t *src, int32_t *dst, int64_t n, cudaStream_t st);
int narrow_any_i64_to_i32(const int64_t *src, int32_t *dst, int64_t n, cudaStream_t st);
int widen_i32_to_i64(const int32_t *src, int64_t *dst, int64_t n, cudaStream_t st);
int widen_f32_to_f64(const float *src, double *dst, int64_t n, cudaStream_t st);
int narrow_f64_to_f32(const double *src, float *dst, int64_t n, cudaStream_t st);
// out[0..n] = exclusive prefix sum of in[0..n-1], out[n] = total
int exclusive_scan_i64(const int64_t *in, int64_t *out, int64_t n, cudaStream_t st);
// sorted COO row coordinates -> row pointer; *sorted_flag_dev set to 0 if rows are not ascending
int coo_rows_to_pos(const int64_t *rows, int64_t nnz, int64_t nrows, int64_t *pos, int *flag_dev,
                    cudaStream_t st);

// *flag_dev (preset to 1 by the caller) becomes 0 if some idx[i] is outside [0, limit)
int check_index_range(const int64_t *idx, int64_t n, int64_t limit, int *flag_dev, cudaStream_t st);

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Work list of long-row chunks shared by the row-parallel kernels (SLOT_WORKLIST):
// a header followed by `count` entries.
struct Chunk {
    int64_t row;
    int64_t begin;
};
struct WorkHeader {
    unsigned int count;
    unsigned int overflow;
    unsigned int pad[2];
};

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
__device__ __forceinline__ double shfl_f64(double v, int src, int width)
{
    return __shfl_sync(0xffffffffu, v, src, width);
}
__device__ __forceinline__ int64_t shfl_i64(int64_t v, int src, int width)
{
    return __shfl_sync(0xffffffffu, (long long)v, src, width);
}
__device__ __forceinline__ int32_t shfl_idx(int32_t v, int src, int width)
{
    return __shfl_sync(0xffffffffu, v, src, width);
}
__device__ __forceinline__ int64_t shfl_idx(int64_t v, int src, int width)
{
    return __shfl_sync(0xffffffffu, (long long)v, src, width);
}
__device__ __forceinline__ double shfl_xor_f64(double v, int mask, int width)
{
    return __shfl_xor_sync(0xffffffffu, v, mask, width);
}
// streaming (read-once) loads that do not displace the gathered operand in L1
__device__ __forceinline__ double ld_stream(const double *p) { return __ldcs(p); }
__device__ __forceinline__ int64_t ld_stream(const int64_t *p)
{
    return (int64_t)__ldcs((const long long *)p);
}
__device__ __forceinline__ int32_t ld_stream(const int32_t *p) { return __ldcs(p); }
#endif

}  // namespace cb200
