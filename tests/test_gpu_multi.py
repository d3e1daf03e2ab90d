"""The sharded entry points of the C ABI: on one GPU with a one-rank communicator (they must then
give what the plain entry points give), and on two GPUs as two processes with the library's NCCL
communicator (skipped where fewer than two GPUs are visible)."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_one_rank_communicator_gives_the_plain_results():
    import comet_b200.api as api
    from comet_b200 import _lib, datasets, sharding
    lib = _lib.load()
    # without a communicator the sharded calls are refused
    A = datasets.rmat_csr(10, 8, seed=1)
    B = datasets.dense_uniform((A.ncols, 64), 2)
    if lib.comet_b200_comm_nranks() == 0:
        with pytest.raises(_lib.CometB200Error, match="no communicator"):
            api.spmm(A, B, sharded=True)
    assert sharding.init_library_comm() == (1, 0)
    try:
        assert np.array_equal(api.spmm(A, B, sharded=True), api.spmm(A, B))
        X = datasets.dense_uniform((A.nrows, 64), 3)
        assert np.array_equal(api.sddmm(A, X, B, sharded=True), api.sddmm(A, X, B))
        C, R = api.spgemm(A, A, sharded=True), api.spgemm(A, A)
        assert np.array_equal(C.a2pos, R.a2pos) and np.array_equal(C.a2crd, R.a2crd)
        assert C.entry_offset == 0 and C.total_nnz == R.nnz
        L = datasets.config_triangles(scale=10, edge_factor=8)
        assert api.masked_pair_count(L, L, L, sharded=True) == api.masked_pair_count(L, L, L)
    finally:
        sharding.destroy_library_comm()
    assert lib.comet_b200_comm_nranks() == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_sharded_entry_points_on_two_gpus():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    env["COMET_B200_ON_ERROR"] = "return"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout, r.stdout[-4000:]
