// The library's per-device communicator and its collectives (comm.cu).
#pragma once
#include "common.cuh"

namespace cb200 {

struct Comm {
    void *comm = nullptr;    // ncclComm_t; for a one-rank "communicator" any non-null value
    int nranks = 0, rank = 0;
};

// The communicator bound to the current device, or null when comet_b200_comm_init has not been called.
Comm *comm_current();

// A replicated array of `total` bytes is exchanged as `nranks` equal slices of this many bytes
// (the last one padded): ceil(total / nranks) rounded up to 256.
size_t comm_slice_bytes(size_t total, int nranks);

// buf holds nranks slices of slice_bytes; this rank has filled slice number `rank`; on return (in
// stream order) all slices are filled.  A null or one-rank communicator is a no-op.
int comm_allgather_inplace(Comm *c, void *buf, size_t slice_bytes, cudaStream_t st);

// all[r] = rank r's *one (device memory).
int comm_allgather_i64(Comm *c, const int64_t *one, int64_t *all, cudaStream_t st);

int comm_allreduce_sum_i64(Comm *c, int64_t *buf, int64_t n, cudaStream_t st);

}  // namespace cb200
