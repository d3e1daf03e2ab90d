"""cometpy's calling convention: the `_mlir_ciface_comet_b200_*` symbols take what cometpy passes to a
kernel it has compiled (frontends/numpy-scipy/cometpy/MLIRGen/lowering.py:212-360) -- a pointer per
result, a dense array as one memref pointer, a scipy CSR matrix as seven arguments -- and fill the
result descriptors with arrays the caller wraps WITHOUT a copy (lowering.py:433-448).  The ctypes
classes below restate the field layout of MLIRGen/utils.py:5-48; arguments are packed and results
unpacked the way lowering.py does it, for scipy's default int32 index arrays and for int64 ones."""
import ctypes
from ctypes import POINTER, Structure, byref, c_double, c_int32, c_int64

import numpy as np
import pytest
import scipy.sparse as sp

from comet_b200 import _lib, datasets
from oracle import oracle

pytestmark = pytest.mark.gpu

RTOL = 1e-12


def _memref(ctype, rank=1):
    class M(Structure):          # ('mem_aligned', 'mem', 'offset', 'dim', 'stride') as in utils.py:5-21
        _fields_ = [("mem_aligned", POINTER(ctype)), ("mem", POINTER(ctype)), ("offset", c_int64),
                    ("dim", c_int64 * rank), ("stride", c_int64 * rank)]
    return M


MemI64, MemI32, MemF64, MemF64x2 = _memref(c_int64), _memref(c_int32), _memref(c_double), _memref(c_double, 2)


def _out_csr(mem_idx):
    class OutCsr(Structure):     # utils.py:26-27 / :38-39
        _fields_ = [("dims_sizes", MemI64), ("insert_1", c_int64), ("A1pos", mem_idx), ("insert_2", c_int64),
                    ("A2pos", mem_idx), ("A2crd", mem_idx), ("Aval", MemF64)]
    return OutCsr


def _from_array(a):
    """memref_from_np_array of lowering.py: the descriptor points at the array's own buffer."""
    cls = {np.dtype(np.int64): MemI64, np.dtype(np.int32): MemI32, np.dtype(np.float64): MemF64}[a.dtype] \
        if a.ndim == 1 else MemF64x2
    m = cls()
    ptr = a.ctypes.data_as(type(m.mem))
    m.mem_aligned, m.mem, m.offset = ptr, ptr, 0
    for i in range(a.ndim):
        m.dim[i] = a.shape[i]
        m.stride[i] = a.strides[i] // a.itemsize
    return m


def _csr_args(m, keep):
    """The seven arguments a scipy CSR matrix becomes (lowering.py:298-321)."""
    dims = np.array(m.shape, dtype=np.int64)
    a1pos = np.array([m.shape[0]], dtype=m.indptr.dtype)
    mems = [_from_array(dims), _from_array(a1pos), _from_array(m.indptr), _from_array(m.indices), _from_array(m.data)]
    keep += [dims, a1pos] + mems
    return [byref(mems[0]), 0, byref(mems[1]), 0, byref(mems[2]), byref(mems[3]), byref(mems[4])]


def _wrap(mem, n):
    return np.ctypeslib.as_array(mem.mem, [n]) if n else np.zeros(0)


def _orc(m, absval=False):
    return oracle.SparseArrays("CSR", m.shape[0], m.shape[1], np.array([m.shape[0]]), np.array([-1]),
                               m.indptr.astype(np.int64), m.indices.astype(np.int64), np.abs(m.data) if absval else m.data)


def _close(got, ref, scale):
    assert np.all(np.abs(np.asarray(got) - ref) <= RTOL * np.maximum(np.abs(ref), scale))


@pytest.mark.parametrize("idx", [np.int32, np.int64])
def test_kernels_called_the_way_cometpy_calls_them(idx):
    lib = _lib.load()
    w = "i32" if idx == np.int32 else "i64"
    fn = lambda name: getattr(lib, "_mlir_ciface_comet_b200_%s_csr_f64_%s" % (name, w))
    A = datasets.rmat_csr(10, 8, seed=1).to_scipy().tocsr()
    A.sort_indices()
    A.indptr, A.indices = A.indptr.astype(idx), A.indices.astype(idx)
    n = A.shape[0]
    keep = []
    OutCsr = _out_csr(MemI32 if idx == np.int32 else MemI64)

    # A @ x: dense result descriptor filled by the callee, wrapped without a copy
    x = datasets.dense_uniform(n, 2)
    y = MemF64()
    mx = _from_array(x)
    fn("spmv")(byref(y), *_csr_args(A, keep), byref(mx))
    _lib.check()
    yv = np.ctypeslib.as_array(y.mem, [n])
    _close(yv, oracle.spmv(_orc(A), x), oracle.spmv(_orc(A, True), np.abs(x)))
    lib.comet_b200_ciface_free(ctypes.cast(y.mem, ctypes.c_void_p))

    # A @ B
    B = datasets.dense_uniform((n, 24), 3)
    C = MemF64x2()
    mB = _from_array(B)
    fn("spmm")(byref(C), *_csr_args(A, keep), byref(mB))
    _lib.check()
    Cv = np.ctypeslib.as_array(C.mem, [C.dim[0], C.dim[1]])
    assert Cv.shape == (n, 24) and C.stride[0] == 24 and C.stride[1] == 1
    _close(Cv, oracle.spmm(_orc(A), B), oracle.spmm(_orc(A, True), np.abs(B)))

    # A @ A (sparse): CSR result struct, arrays wrapped as scipy does (csr_array(..., copy=False))
    out = OutCsr()
    fn("spgemm")(byref(out), *_csr_args(A, keep), *_csr_args(A, keep), 0)
    _lib.check()
    R = oracle.spgemm(_orc(A), _orc(A))
    assert (out.dims_sizes.mem[0], out.dims_sizes.mem[1]) == (n, n) and out.A1pos.mem[0] == n
    pos = np.ctypeslib.as_array(out.A2pos.mem, [out.A2pos.dim[0]])
    crd, val = _wrap(out.A2crd, out.A2crd.dim[0]), _wrap(out.Aval, out.Aval.dim[0])
    assert pos.dtype == idx and crd.dtype == idx
    got = sp.csr_array((val, crd, pos), shape=(n, n), copy=False)
    assert np.array_equal(got.indptr, R.a2pos) and np.array_equal(got.indices, R.a2crd)
    _close(got.data, R.val, oracle.spgemm(_orc(A, True), _orc(A, True)).val)

    # einsum('ij,jk->ik', L, L, mask=L, semiring='+,pair') and its sum (the triangle count)
    L = datasets.config_triangles(scale=10, edge_factor=8).to_scipy().tocsr()
    L.indptr, L.indices = L.indptr.astype(idx), L.indices.astype(idx)
    want = oracle.masked_pair_count(_orc(L), _orc(L), _orc(L))
    outm = OutCsr()
    fn("spgemm_masked")(byref(outm), *_csr_args(L, keep), *_csr_args(L, keep), *_csr_args(L, keep), 1)
    _lib.check()
    assert int(round(_wrap(outm.Aval, outm.Aval.dim[0]).sum())) == want
    cnt = fn("masked_count")
    assert cnt(*_csr_args(L, keep), *_csr_args(L, keep), *_csr_args(L, keep)) == float(want)
    _lib.check()

    # S.multiply(X @ Y.T) on S's pattern
    X, Y = datasets.dense_uniform((n, 16), 4), datasets.dense_uniform((n, 16), 5)
    o = OutCsr()
    mX, mY = _from_array(X), _from_array(Y)
    fn("sddmm")(byref(o), *_csr_args(A, keep), byref(mX), byref(mY))
    _lib.check()
    assert np.array_equal(np.ctypeslib.as_array(o.A2pos.mem, [n + 1]), A.indptr)
    assert np.array_equal(_wrap(o.A2crd, o.A2crd.dim[0]), A.indices)
    _close(_wrap(o.Aval, o.Aval.dim[0]), oracle.sddmm(_orc(A), X, Y), oracle.sddmm(_orc(A, True), np.abs(X), np.abs(Y)))
