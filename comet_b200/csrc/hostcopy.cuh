// Host <-> device copies of the host-memref entry points (hostcopy.cu): large copies on pageable host
// memory are staged through page-locked chunks by worker threads, everything else is a cudaMemcpyAsync.
#pragma once
#include "common.cuh"

namespace cb200 {

bool host_is_pageable(const void *p);

// Return when the host array has been read completely; complete on the device in stream order.
int h2d(void *dev, const void *host, size_t bytes, cudaStream_t st);
int h2d_2d(void *dev, size_t dev_pitch, const void *host, size_t host_pitch, size_t row_bytes, size_t rows,
           cudaStream_t st);

// Return when the copy has been enqueued; the host array is complete after copies_drain() AND a
// synchronisation of the stream (page-locked destinations are written by the DMA engine in stream order,
// pageable ones by worker threads that copies_drain waits for).
int d2h(void *host, const void *dev, size_t bytes, cudaStream_t st);
int d2h_2d(void *host, size_t host_pitch, const void *dev, size_t dev_pitch, size_t row_bytes, size_t rows,
           cudaStream_t st);
int copies_drain();

}  // namespace cb200
