"""Host arrays as COMET's generated code holds them: plain malloc'ed (pageable) memory.  Large copies
between such arrays and the device are staged by the library through page-locked chunks on worker
threads; these tests push operands and results of several chunks through that path -- contiguous,
strided (column windows of wider matrices), 32-bit indices -- and compare with the CPU oracle, and
run the same calls with the staging switched off and with page-locked arrays."""
import numpy as np
import pytest
import torch

import comet_b200.api as api
from comet_b200 import _lib, datasets
from oracle import oracle

pytestmark = pytest.mark.gpu

RTOL = 1e-12


def _orc(t, absval=False):
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd,
                               np.abs(t.val) if absval else t.val)


def _close(got, ref, scale):
    bad = np.abs(np.asarray(got) - ref) > RTOL * np.maximum(np.abs(ref), scale)
    assert not bad.any(), "%d entries beyond 1e-12" % int(bad.sum())


def _spmm_window(A, wide_b, col0, k, out, out0):
    lib = _lib.load()
    pk = api._Packer()
    fn, _, (A_,) = api._entry(lib, "spmm", api.as_sparse(A))
    fn(*pk.sparse(A_), *pk.m2(wide_b[:, col0:col0 + k]), *pk.m2(out[:, out0:out0 + k]), 0, 0)
    _lib.check()


@pytest.mark.parametrize("mode", ["staged", "driver", "page-locked"])
@pytest.mark.parametrize("panels", [True, False])
def test_spmm_through_pageable_host_arrays(monkeypatch, mode, panels):
    monkeypatch.setenv("COMET_B200_STAGE_MIN_BYTES", str(1 << 20))
    A = datasets.rmat_csr(15, 8, seed=2)                       # 32768 rows: B and C are 33.5 MB each at K = 128
    k = 128
    wide = datasets.dense_uniform((A.ncols, k + 10), 3)        # B is a column window: rows 1104 bytes apart
    out = np.full((A.nrows, k + 6), -7.0)
    if mode == "page-locked":
        wide = torch.from_numpy(wide).pin_memory().numpy()
        out = torch.from_numpy(out).pin_memory().numpy()
    if mode == "driver":
        monkeypatch.setenv("COMET_B200_STAGED_COPIES", "0")
    monkeypatch.setenv("COMET_B200_SPMM_PANEL_MIN_BYTES", "0" if panels else "1e18")
    if panels:
        monkeypatch.setenv("COMET_B200_SPMM_PANEL", "32")       # asked for by name: kept even for pageable operands
    _spmm_window(A, wide, 5, k, out, 3)
    B = np.ascontiguousarray(wide[:, 5:5 + k])
    _close(out[:, 3:3 + k], oracle.spmm(_orc(A), B), oracle.spmm(_orc(A, True), np.abs(B)))
    assert np.all(out[:, :3] == -7.0) and np.all(out[:, 3 + k:] == -7.0)          # padding untouched


def test_small_chunks_and_every_staged_direction(monkeypatch):
    """Staging from 4 KB on, so that even the index arrays and short results go through the chunks: SpMV,
    SDDMM, a sparse product with 32-bit indices (narrowed on the device, then staged down) and the count."""
    monkeypatch.setenv("COMET_B200_STAGE_MIN_BYTES", "4096")
    A = datasets.rmat_csr(13, 16, seed=5)
    x = datasets.dense_uniform(A.ncols, 1)
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), oracle.spmv(_orc(A, True), np.abs(x)))
    X, Y = datasets.dense_uniform((A.nrows, 64), 2), datasets.dense_uniform((A.ncols, 64), 3)
    _close(api.sddmm(A, X, Y), oracle.sddmm(_orc(A), X, Y), oracle.sddmm(_orc(A, True), np.abs(X), np.abs(Y)))
    for dt in (np.int64, np.int32):
        C = api.spgemm(A.with_index_dtype(dt), A.with_index_dtype(dt))
        R = oracle.spgemm(_orc(A), _orc(A))
        assert C.a2crd.dtype == dt and C.nnz * 8 > (4 << 20)       # several chunks per result array
        assert np.array_equal(C.a2pos, R.a2pos) and np.array_equal(C.a2crd, R.a2crd)
        _close(C.val, R.val, oracle.spgemm(_orc(A, True), _orc(A, True)).val)
    L = datasets.config_triangles(scale=12, edge_factor=8)
    assert api.triangle_count(L) == oracle.masked_pair_count(_orc(L), _orc(L), _orc(L))
