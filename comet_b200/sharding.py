"""Row-block sharding of the sparse operand across the GPUs of one node: one
process per GPU, ``torch.distributed`` for the few values that have to cross
(NCCL on GPUs, gloo in the CPU tests).

Output rows of every operation on this path are independent, so each rank owns
a contiguous block of rows of the left operand, chosen to balance the work
(stored entries, or products for SpGEMM / triangle counting), keeps the dense
operand or the right-hand matrix replicated in its own memory, and runs the
single-GPU kernels on its block.  Collectives only assemble results:
all-gather of dense row blocks, all-gather of per-shard nnz to place sparse
row blocks, all-reduce of the triangle count.
"""
import ctypes

import numpy as np
import torch
import torch.distributed as dist

from .api import SparseTensor, as_sparse


def slice_bytes(total_bytes, nranks):
    """Bytes of one slice when a replicated array is exchanged between ``nranks`` ranks: the same rule as
    ``comet_b200_comm_slice_bytes`` (ceil(total / nranks) rounded up to 256)."""
    nranks = max(int(nranks), 1)
    s = (int(total_bytes) + nranks - 1) // nranks
    return (s + 255) & ~255


def replica_slice(total_bytes, nranks, rank):
    """Byte range [lo, hi) of a replicated array that rank ``rank`` uploads itself."""
    s = slice_bytes(total_bytes, nranks)
    lo = min(s * rank, total_bytes)
    return lo, min(lo + s, total_bytes)


def init_library_comm(group=None):
    """Creates libcomet_b200's own communicator for the ranks of a torch.distributed group: rank 0 asks the
    library for a unique id, the id travels through torch.distributed, every rank calls
    comet_b200_comm_init with its CUDA device current.  Returns (nranks, rank)."""
    from . import _lib
    lib = _lib.load()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if lib.comet_b200_comm_nranks() == world:
        return world, rank
    ident = [None]
    if rank == 0 and world > 1:
        buf = ctypes.create_string_buffer(128)
        _lib.check(lib.comet_b200_comm_unique_id(buf, 128))
        ident = [buf.raw]
    if world > 1:
        dist.broadcast_object_list(ident, src=0, group=group)
        torch.cuda.synchronize()
    _lib.check(lib.comet_b200_comm_init(world, rank, ident[0]))
    return world, rank


def destroy_library_comm():
    from . import _lib
    _lib.check(_lib.load().comet_b200_comm_destroy())


def row_blocks(pos, nparts, weights=None):
    """Boundaries b[0..nparts] of contiguous row blocks with nearly equal weight.

    Default weight of a row is its stored-entry count (from ``pos``); pass
    per-row ``weights`` (e.g. product counts) to balance something else."""
    pos = np.asarray(pos, dtype=np.int64)
    nrows = pos.shape[0] - 1
    if weights is None:
        cum = pos - pos[0]
    else:
        w = np.asarray(weights)
        w = w.astype(np.float64) if w.dtype.kind == "f" else w.astype(np.int64)     # measured costs are fractional
        cum = np.concatenate([np.zeros(1, dtype=w.dtype), np.cumsum(w)])
    total = cum[-1]
    bounds = np.zeros(nparts + 1, dtype=np.int64)
    bounds[nparts] = nrows
    for p in range(1, nparts):
        target = (total * p) / nparts if cum.dtype.kind == "f" else (int(total) * p) // nparts
        bounds[p] = int(np.searchsorted(cum, target, side="left"))
    bounds = np.minimum(np.maximum.accumulate(bounds), nrows)
    return bounds


def product_weights(A, B):
    """Per-row work of A*B: sum over stored A[i,k] of the length of row k of B."""
    A, B = as_sparse(A), as_sparse(B)
    blen = np.diff(B.a2pos)
    per_entry = blen[A.a2crd]
    cum = np.concatenate([[0], np.cumsum(per_entry)])
    return cum[A.a2pos[1:]] - cum[A.a2pos[:-1]]


def take_rows(A, lo, hi):
    """CSR block of rows [lo, hi) with its own zero-based row pointer."""
    A = as_sparse(A)
    s, e = int(A.a2pos[lo]), int(A.a2pos[hi])
    return SparseTensor("CSR", hi - lo, A.ncols, np.array([hi - lo], dtype=np.int64),
                        np.array([-1], dtype=np.int64), A.a2pos[lo:hi + 1] - s, A.a2crd[s:e], A.val[s:e])


def _world(group):
    return dist.get_world_size(group) if dist.is_initialized() else 1


def all_gather_rows(block, bounds, group=None):
    """Concatenates per-rank row blocks (rank r holds rows bounds[r]:bounds[r+1]) on every rank.
    ``block`` is a [rows_r, ...] tensor; blocks are padded to the longest so that a plain
    all-gather can be used."""
    world = _world(group)
    if world == 1:
        return block
    counts = [int(bounds[r + 1] - bounds[r]) for r in range(world)]
    longest = max(counts)
    padded = block.new_zeros((longest,) + tuple(block.shape[1:]))
    padded[:block.shape[0]] = block
    out = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(out, padded, group=group)
    return torch.cat([out[r][:counts[r]] for r in range(world)], dim=0)


def global_row_pointer(local_pos, group=None):
    """Local zero-based row pointer of a sparse output block -> (global row pointer of the block,
    this rank's entry offset, total nnz).  One all-gather of a single int64 per rank."""
    world = _world(group)
    local_nnz = local_pos[-1:].clone()
    if world == 1:
        return local_pos, 0, int(local_nnz.item())
    parts = [torch.empty_like(local_nnz) for _ in range(world)]
    dist.all_gather(parts, local_nnz, group=group)
    sizes = [int(p.item()) for p in parts]
    rank = dist.get_rank(group)
    offset = sum(sizes[:rank])
    return local_pos + offset, offset, sum(sizes)


def all_reduce_sum(t, group=None):
    """In-place sum over ranks (the triangle count's last step)."""
    if _world(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t
