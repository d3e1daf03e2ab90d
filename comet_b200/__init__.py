"""libcomet_b200: B200 (sm_100a) execution path for COMET's sparse tensor-algebra
operations, behind a C ABI that takes COMET's pos/crd/val memref descriptors.

    comet_b200.api      host arrays in / out through the memref entry points
    comet_b200.device   device-resident operands (torch tensors as plain memory)
    comet_b200.sharding row-block sharding over the GPUs of a node
    comet_b200.datasets seeded synthetic inputs of the benchmark configurations
    comet_b200.build    in-tree nvcc build of libcomet_b200.so
"""
from .api import (ANY_PAIR, MIN_FIRST, MIN_PLUS, MIN_SECOND, PLUS_FIRST, PLUS_PAIR, PLUS_SECOND, PLUS_TIMES, SparseTensor, dense_times_sparse, einsum, elews_csr_csr,  # noqa: F401
                  elews_sparse_dense, masked_pair_count, reduce_sum, sddmm, spgemm, spmm, spmv,
                  triangle_count)
