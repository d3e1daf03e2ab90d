"""One rank of the multi-GPU parity check (run under torch.distributed.run, one process per GPU).

Every rank takes a contiguous row block of the left operand, passes the right operand whole to the
sharded host entry points of the C ABI (each rank uploads one N-th of it, the slices cross NVLink
through the library's own NCCL communicator) and compares ITS block of the result with the CPU oracle
run on the same block.  A rank prints ``rank R ok`` and exits 0 only if every comparison holds."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

RTOL = 1e-12


def _orc(t):
    from oracle import oracle
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, np.asarray(t.a1pos, dtype=np.int64),
                               np.asarray(t.a1crd, dtype=np.int64), np.asarray(t.a2pos, dtype=np.int64),
                               np.asarray(t.a2crd, dtype=np.int64), t.val)


def _absd(t):
    from oracle import oracle
    o = _orc(t)
    return oracle.SparseArrays(o.format, o.nrows, o.ncols, o.a1pos, o.a1crd, o.a2pos, o.a2crd, np.abs(o.val))


def _close(got, ref, scale):
    bad = np.abs(np.asarray(got) - ref) > RTOL * np.maximum(np.abs(ref), scale)
    assert not bad.any(), "%d entries beyond 1e-12" % int(bad.sum())


def main():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    import comet_b200.api as api
    from comet_b200 import _lib, datasets, sharding
    from oracle import oracle

    n_r, r = sharding.init_library_comm()
    assert (n_r, r) == (world, rank)
    lib = _lib.load()
    assert lib.comet_b200_comm_nranks() == world and lib.comet_b200_comm_rank() == rank

    A = datasets.rmat_csr(11, 16, seed=3)
    bounds = sharding.row_blocks(A.a2pos, world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    blk = sharding.take_rows(A, lo, hi)

    # SpMM: the single-buffer path, then the column-panel pipeline (forced by a zero size threshold)
    for k, env in ((48, None), (128, "0")):
        if env is not None:
            os.environ["COMET_B200_SPMM_PANEL_MIN_BYTES"] = env
        B = datasets.dense_uniform((A.ncols, k), 5 + k)
        got = api.spmm(blk, B, sharded=True)
        _close(got, oracle.spmm(_orc(blk), B), oracle.spmm(_absd(blk), np.abs(B)))
        os.environ.pop("COMET_B200_SPMM_PANEL_MIN_BYTES", None)
    # 32-bit index arrays take the _i32 symbol
    got = api.spmm(blk.with_index_dtype(np.int32), B, sharded=True)
    _close(got, oracle.spmm(_orc(blk), B), oracle.spmm(_absd(blk), np.abs(B)))

    # SDDMM: S and X by row block, Y whole
    X, Y = datasets.dense_uniform((A.nrows, 64), 7), datasets.dense_uniform((A.ncols, 64), 8)
    got = api.sddmm(blk, X[lo:hi], Y, sharded=True)
    _close(got, oracle.sddmm(_orc(blk), X[lo:hi], Y), oracle.sddmm(_absd(blk), np.abs(X[lo:hi]), np.abs(Y)))

    # SpGEMM: block of C bit-exact in structure, and its place in the whole result
    whole = oracle.spgemm(_orc(A), _orc(A))
    C = api.spgemm(blk, A, sharded=True)
    ref = oracle.spgemm(_orc(blk), _orc(A))
    assert np.array_equal(C.a2pos, ref.a2pos) and np.array_equal(C.a2crd, ref.a2crd)
    _close(C.val, ref.val, oracle.spgemm(_absd(blk), _absd(A)).val)
    assert C.entry_offset == int(whole.a2pos[lo]) and C.total_nnz == int(whole.a2pos[-1])
    assert np.array_equal(C.a2crd, whole.a2crd[C.entry_offset:C.entry_offset + C.nnz])
    # masked, plus-pair, mask = the block itself
    Cm = api.spgemm(blk, A, blk, api.PLUS_PAIR, sharded=True)
    refm = oracle.spgemm(_orc(blk), _orc(A), _orc(blk), oracle.PLUS_PAIR)
    assert np.array_equal(Cm.a2pos, refm.a2pos) and np.array_equal(Cm.a2crd, refm.a2crd)
    assert np.array_equal(Cm.val, refm.val)

    # triangle count: every rank receives the count over all blocks
    L = datasets.config_triangles(scale=11, edge_factor=8)
    lb = sharding.row_blocks(L.a2pos, world, weights=sharding.product_weights(L, L))
    Lb = sharding.take_rows(L, int(lb[rank]), int(lb[rank + 1]))
    want = oracle.masked_pair_count(_orc(L), _orc(L), _orc(L))
    assert api.masked_pair_count(Lb, L, Lb, sharded=True) == want

    # a fault in ONE rank's operand (a column index one past the end, found by the host-side checks of
    # the library before any kernel runs) ends the call on EVERY rank with an error instead of leaving
    # the others waiting in the exchange; the communicator stays usable
    bad = api.SparseTensor(blk.format, blk.nrows, blk.ncols, blk.a1pos, blk.a1crd, blk.a2pos,
                           blk.a2crd.copy(), blk.val)
    if rank == world - 1 and bad.nnz:
        bad.a2crd[bad.nnz // 2] = bad.ncols
    for call in (lambda: api.spmm(bad, B, sharded=True), lambda: api.spgemm(bad, A, sharded=True),
                 lambda: api.masked_pair_count(bad, A, bad, sharded=True),
                 lambda: api.sddmm(bad, X[lo:hi], Y, sharded=True)):
        try:
            call()
        except _lib.CometB200Error as e:
            assert ("outside" in str(e)) == (rank == world - 1), str(e)
        else:
            raise AssertionError("rank %d: the faulty call was not refused" % rank)
    got = api.spmm(blk, B, sharded=True)
    _close(got, oracle.spmm(_orc(blk), B), oracle.spmm(_absd(blk), np.abs(B)))

    torch.cuda.synchronize()
    dist.barrier()
    sharding.destroy_library_comm()
    dist.destroy_process_group()
    print("rank %d ok" % rank, flush=True)


if __name__ == "__main__":
    main()
