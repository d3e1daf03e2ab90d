"""CPU tests of the host-side logic: synthetic inputs and row-block sharding,
including a world_size-2 gloo run in which the per-rank compute is the oracle
(there is no GPU here) so that only partitioning and collectives are under test."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from comet_b200 import datasets, sharding
from oracle import oracle


def test_rmat_is_deduplicated_sorted_and_seeded():
    A = datasets.rmat_csr(10, 8, seed=0)
    B = datasets.rmat_csr(10, 8, seed=0)
    assert np.array_equal(A.a2crd, B.a2crd) and np.array_equal(A.val, B.val)
    rows = np.repeat(np.arange(A.nrows), np.diff(A.a2pos))
    keys = rows * A.ncols + A.a2crd
    assert np.all(np.diff(keys) > 0)                 # strictly ascending => sorted, no duplicates
    assert not np.any(rows == A.a2crd)               # self-loops dropped
    assert A.val.min() >= 0.5 and A.val.max() <= 1.5
    L = datasets.config_triangles(scale=9, edge_factor=8)
    lr = np.repeat(np.arange(L.nrows), np.diff(L.a2pos))
    assert np.all(lr > L.a2crd) and np.all(L.val == 1.0)


def test_uniform_rows_and_mtx_round_trip(tmp_path):
    A, x = datasets.config_spmv(n=256, per_row=16)
    assert A.nnz == 256 * 16 and np.all(np.diff(A.a2pos) == 16)
    cols = A.a2crd.reshape(256, 16)
    assert np.all(np.diff(cols, axis=1) > 0)
    path = tmp_path / "a.mtx"
    datasets.write_mtx(str(path), A)
    R = oracle.read_mtx(str(path), "CSR")
    assert np.array_equal(R.a2pos, A.a2pos) and np.array_equal(R.a2crd, A.a2crd)
    assert np.array_equal(R.val, A.val)              # %.17g round-trips float64 exactly


def test_row_blocks_balance_and_cover():
    A = datasets.rmat_csr(12, 16, seed=1)
    for parts in (1, 2, 4, 8):
        b = sharding.row_blocks(A.a2pos, parts)
        assert b[0] == 0 and b[-1] == A.nrows and np.all(np.diff(b) >= 0)
        per = np.diff(A.a2pos[b])
        assert per.sum() == A.nnz
        assert per.max() <= A.nnz / parts + np.diff(A.a2pos).max()
    w = sharding.product_weights(A, A)
    b = sharding.row_blocks(A.a2pos, 4, weights=w)
    cw = np.concatenate([[0], np.cumsum(w)])
    per = np.diff(cw[b])
    assert per.sum() == w.sum() and per.max() <= w.sum() / 4 + w.max()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A = datasets.rmat_csr(9, 8, seed=3)
        x = datasets.dense_uniform(A.ncols, 5)
        b = sharding.row_blocks(A.a2pos, world)
        mine = sharding.take_rows(A, int(b[rank]), int(b[rank + 1]))
        oa = oracle.SparseArrays("CSR", mine.nrows, mine.ncols, mine.a1pos, mine.a1crd, mine.a2pos,
                                 mine.a2crd, mine.val)
        # SpMV: all-gather of y blocks
        y_block = torch.from_numpy(oracle.spmv(oa, x))
        y = sharding.all_gather_rows(y_block, b).numpy()
        full = oracle.SparseArrays("CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val)
        ok_spmv = np.array_equal(y, oracle.spmv(full, x))
        # SpGEMM: per-shard nnz -> global row pointer
        Cb = oracle.spgemm(oa, full)
        gpos, off, total = sharding.global_row_pointer(torch.from_numpy(Cb.a2pos))
        C = oracle.spgemm(full, full)
        ok_pos = np.array_equal(gpos.numpy(), C.a2pos[b[rank]:b[rank + 1] + 1]) and total == C.nnz
        ok_crd = np.array_equal(Cb.a2crd, C.a2crd[off:off + Cb.nnz])
        # triangle count: all-reduce of per-block counts
        L = datasets.config_triangles(scale=8, edge_factor=8)
        ol = oracle.SparseArrays("CSR", L.nrows, L.ncols, L.a1pos, L.a1crd, L.a2pos, L.a2crd, L.val)
        lb = sharding.row_blocks(L.a2pos, world, weights=sharding.product_weights(L, L))
        cnt = torch.tensor([oracle.masked_pair_count(ol, ol, ol, int(lb[rank]), int(lb[rank + 1]))])
        sharding.all_reduce_sum(cnt)
        ok_tc = int(cnt.item()) == oracle.masked_pair_count(ol, ol, ol)
        q.put((rank, ok_spmv, ok_pos, ok_crd, ok_tc))
    finally:
        dist.destroy_process_group()


def test_sharded_collectives_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, *oks in results:
        assert all(oks), (rank, oks)


# ---------------------------------------------------------------------------
# The call sequence of the sharded host entry points, replayed on CPU ranks (gloo): every rank uploads
# only its slice of the replicated operand, the slices are all-gathered, each rank works on its row
# block, per-rank entry counts are all-gathered and the count is all-reduced.  The slice arithmetic is
# the library's own (comet_b200_comm_slice_bytes is a pure function and needs no device).
# ---------------------------------------------------------------------------
def test_slice_rule_matches_the_library_and_covers_the_array():
    from comet_b200 import _lib
    lib = _lib.load()
    rng = np.random.default_rng(0)
    for total in [0, 1, 255, 256, 257, 4096, 10 ** 6 + 3, 1073741824, 8589934591] + list(rng.integers(1, 1 << 34, 50)):
        for n in range(1, 9):
            s = sharding.slice_bytes(total, n)
            assert s == lib.comet_b200_comm_slice_bytes(int(total), n)
            assert s % 256 == 0 and s * n >= total
            ranges = [sharding.replica_slice(int(total), n, r) for r in range(n)]
            assert ranges[0][0] == 0 and ranges[-1][1] == total
            assert all(ranges[r][1] == ranges[r + 1][0] or ranges[r + 1][0] == total for r in range(n - 1))


def _replica_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A = datasets.rmat_csr(9, 8, seed=4)
        B = datasets.dense_uniform((A.ncols, 10), 6)             # 40 KB: slices end inside a row
        raw = np.frombuffer(B.tobytes(), dtype=np.uint8)
        s = sharding.slice_bytes(raw.nbytes, world)
        lo, hi = sharding.replica_slice(raw.nbytes, world, rank)
        mine = torch.zeros(s, dtype=torch.uint8)                  # what this rank sends through its own link
        mine[:hi - lo] = torch.from_numpy(raw[lo:hi].copy())
        parts = [torch.empty(s, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, mine)                              # ncclAllGather in the library
        Bfull = np.frombuffer(torch.cat(parts).numpy()[:raw.nbytes].tobytes(), dtype=np.float64).reshape(B.shape)
        ok_rep = np.array_equal(Bfull, B)
        b = sharding.row_blocks(A.a2pos, world)
        blk = sharding.take_rows(A, int(b[rank]), int(b[rank + 1]))
        ob = oracle.SparseArrays("CSR", blk.nrows, blk.ncols, blk.a1pos, blk.a1crd, blk.a2pos, blk.a2crd, blk.val)
        full = oracle.SparseArrays("CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val)
        Cb = torch.from_numpy(oracle.spmm(ob, Bfull))
        C = sharding.all_gather_rows(Cb, b).numpy()
        ok_spmm = np.array_equal(C, oracle.spmm(full, B))
        # the agreement step: one rank reports a fault, every rank sees it
        flag = torch.tensor([1 if rank == world - 1 else 0])
        dist.all_reduce(flag)
        q.put((rank, ok_rep, ok_spmm, int(flag.item()) == 1))
    finally:
        dist.destroy_process_group()


def test_replicated_operand_by_slices_world2_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_replica_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, *oks in results:
        assert all(oks), (rank, oks)
