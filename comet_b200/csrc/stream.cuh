// Shared by the entry-stream kernels (SpMM, SDDMM): asynchronous 16-byte copies into shared memory and the
// plan that cuts a CSR matrix into equal pieces of its (entries + rows) path.
#pragma once
#include "common.cuh"

namespace cb200 {

struct StreamPlan {
    WorkHeader *hdr;          // hdr->pad[0]: counter the persistent warps draw pieces from
    int64_t *block_row;       // piece b starts in row block_row[b] ...
    int64_t *block_ent;       // ... at entry block_ent[b]; both have nblocks + 1 entries
    int64_t q, nblocks;
};

int stream_plan(int64_t nrows, int64_t nnz, int64_t warps, const int64_t *row_ids, const int64_t *pos, double *c,
                int64_t ldc, int k, int accumulate, cudaStream_t st, StreamPlan *out);

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t sb_smem(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// 16 bytes global -> shared without passing through registers or L1
__device__ __forceinline__ void sb_copy16(uint32_t dst, const void *src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void sb_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// wait until at most `pending` of this thread's copy groups are still in flight
__device__ __forceinline__ void sb_wait_pending(int pending)
{
    switch (pending) {
    case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.wait_group 6;" ::: "memory"); break;
    default: asm volatile("cp.async.wait_group 7;" ::: "memory"); break;
    }
}
#endif

}  // namespace cb200
