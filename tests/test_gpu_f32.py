"""float values.  COMET instantiates its kernels and runtime symbols for f32 as well as f64
(lib/ExecutionEngine/SparseUtils.cpp:2354-2400); the _f32_ entry points take float memrefs, compute in
double on the device and round once.  They are compared with the single-precision build of the CPU
oracle (the same loop nests with float mulf / addf) at 1e-5 relative to sum(|terms|), and with the
double result rounded to float, which they must equal exactly where no atomics reorder the sum."""
import numpy as np
import pytest

import comet_b200.api as api
from comet_b200 import datasets
from oracle import oracle

pytestmark = pytest.mark.gpu

RTOL32 = 1e-5


def _f32(A):
    return api.SparseTensor(A.format, A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val.astype(np.float32))


def _orc(t, absval=False):
    v = np.abs(t.val) if absval else t.val
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, np.asarray(t.a1pos, dtype=np.int64),
                               np.asarray(t.a1crd, dtype=np.int64), np.asarray(t.a2pos, dtype=np.int64),
                               np.asarray(t.a2crd, dtype=np.int64), v)


def _close32(got, ref, scale):
    got = np.asarray(got)
    assert got.dtype == np.float32
    bad = np.abs(got.astype(np.float64) - ref.astype(np.float64)) > RTOL32 * np.maximum(np.abs(ref), scale)
    assert not bad.any(), int(bad.sum())


@pytest.mark.parametrize("idx", [np.int64, np.int32])
def test_float_entry_points_against_the_single_precision_oracle(idx):
    A = _f32(datasets.rmat_csr(11, 8, seed=7)).with_index_dtype(idx)
    n = A.nrows
    x = datasets.dense_uniform(n, 1).astype(np.float32)
    y = api.spmv(A, x)
    _close32(y, oracle.spmv_f32(_orc(A), x), oracle.spmv_f32(_orc(A, True), np.abs(x)))
    # the float result is the double result of the same float inputs, rounded once (SpMV sums in a fixed order)
    y64 = api.spmv(api.SparseTensor(A.format, n, n, A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val.astype(np.float64)),
                   x.astype(np.float64))
    assert np.array_equal(y, y64.astype(np.float32))

    B = datasets.dense_uniform((n, 64), 2).astype(np.float32)
    _close32(api.spmm(A, B), oracle.spmm_f32(_orc(A), B), oracle.spmm_f32(_orc(A, True), np.abs(B)))
    C0 = datasets.dense_uniform((n, 64), 3).astype(np.float32)
    ref = oracle.spmm_f32(_orc(A), B) + C0
    _close32(api.spmm(A, B, C0), ref, oracle.spmm_f32(_orc(A, True), np.abs(B)) + np.abs(C0))

    X, Y = datasets.dense_uniform((n, 32), 4).astype(np.float32), datasets.dense_uniform((n, 32), 5).astype(np.float32)
    _close32(api.sddmm(A, X, Y), oracle.sddmm_f32(_orc(A), X, Y), oracle.sddmm_f32(_orc(A, True), np.abs(X), np.abs(Y)))

    C = api.spgemm(A, A)
    R = oracle.spgemm_f32(_orc(A), _orc(A))
    assert C.val.dtype == np.float32 and C.a2crd.dtype == idx
    assert np.array_equal(C.a2pos, R.a2pos) and np.array_equal(C.a2crd, R.a2crd)
    _close32(C.val, R.val, oracle.spgemm_f32(_orc(A, True), _orc(A, True)).val)


def test_value_widths_of_a_handle_must_match():
    from comet_b200 import _lib
    lib = _lib.load()
    A = _f32(datasets.rmat_csr(8, 4, seed=1))
    pk = api._Packer()
    cpos = np.zeros(A.nrows + 1, dtype=np.int64)
    sizes = np.zeros(11, dtype=np.int64)
    h = lib.comet_b200_spgemm_symbolic_f32_i64(*pk.sparse(A), *pk.sparse(A), *pk.sparse(A), 0, 0, *pk.m1(cpos), *pk.m1(sizes))
    _lib.check()
    crd, val = np.zeros(int(sizes[8]), dtype=np.int64), np.zeros(int(sizes[8]), dtype=np.float64)
    lib.comet_b200_spgemm_numeric_f64_i64(h, *pk.m1(crd), *pk.m1(val))
    with pytest.raises(_lib.CometB200Error, match="another index or value width"):
        _lib.check()
