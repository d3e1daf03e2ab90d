"""Host-side mirror of the operations COMET's front ends reach the sparse hot
path with, executed through the C ABI of ``libcomet_b200`` (layer 1: host
memref descriptors, the same calls a COMET lowering would emit).

Operands are packed the way cometpy packs them for ``_mlir_ciface_`` calls
(frontends/numpy-scipy/cometpy/MLIRGen/lowering.py:283-360): a dims array, then
per dimension pos / crd arrays, then values; values are float64, index arrays
int64 or int32 (scipy's default), which selects the _i64 or _i32 entry points.  Sparse operands may be

  * any object with ``format`` ('CSR' | 'DCSR' | 'COO'), ``nrows``, ``ncols`` and
    the COMET arrays ``a1pos, a1crd, a2pos, a2crd, val`` (what COMET's reader
    produces, lib/ExecutionEngine/SparseUtils.cpp:1643-1751), or
  * a scipy.sparse CSR / COO matrix (what cometpy accepts, CSC rejected).

Function names follow the cometpy surface: ``A @ x`` -> spmv/spmm,
``A.multiply(B)`` -> elews_mul, ``einsum('ij,jk->ik', A, B, mask=M,
mask_type='push', semiring='+,pair')`` -> spgemm
(frontends/numpy-scipy/cometpy/comet.py:1014-1088, 1210-1319).
"""
import ctypes

import numpy as np

from . import _lib
from ._lib import MemRef1D, MemRef2D

PLUS_TIMES, PLUS_PAIR, PLUS_FIRST, PLUS_SECOND, MIN_PLUS, MIN_FIRST, MIN_SECOND, ANY_PAIR = range(8)
MASK_NONE = 0
MASK_PUSH = 1

_FMT = {"CSR": (0, 1), "DCSR": (1, 1), "COO": (2, 3)}
# DSL / cometpy spellings (frontends/comet_dsl/mlir/MLIRGen.cpp:102-145) and the IR attribute strings
_SEMIRINGS = {"+,*": PLUS_TIMES, "plusxy_times": PLUS_TIMES, "+,pair": PLUS_PAIR, "plusxy_pairxy": PLUS_PAIR,
              "+,first": PLUS_FIRST, "plusxy_first": PLUS_FIRST, "+,second": PLUS_SECOND,
              "plusxy_second": PLUS_SECOND, "min,+": MIN_PLUS, "minxy_plusxy": MIN_PLUS,
              "min,first": MIN_FIRST, "minxy_first": MIN_FIRST, "min,second": MIN_SECOND,
              "minxy_second": MIN_SECOND, "any,pair": ANY_PAIR, "any_pairxy": ANY_PAIR}
_SEMIRINGS.update({c: c for c in range(8)})
_DENSE_OUTPUT_SEMIRINGS = (PLUS_TIMES, PLUS_PAIR)


class SparseTensor:
    """COMET's per-dimension arrays for one sparse matrix (int64 / float64)."""

    def __init__(self, fmt, nrows, ncols, a1pos, a1crd, a2pos, a2crd, val):
        self.format = fmt
        self.nrows, self.ncols = int(nrows), int(ncols)
        self.a1pos, self.a1crd, self.a2pos, self.a2crd, self.val = a1pos, a1crd, a2pos, a2crd, val

    @property
    def nnz(self):
        return int(self.val.shape[0])

    @property
    def shape(self):
        return (self.nrows, self.ncols)

    @property
    def index_dtype(self):
        return np.asarray(self.a2crd).dtype

    def with_index_dtype(self, dt):
        if self.index_dtype == dt:
            return self
        return SparseTensor(self.format, self.nrows, self.ncols, _idx(self.a1pos, dt), _idx(self.a1crd, dt),
                            _idx(self.a2pos, dt), _idx(self.a2crd, dt), self.val)

    def to_scipy(self):
        import scipy.sparse as sp
        if self.format == "CSR":
            return sp.csr_matrix((self.val, self.a2crd, self.a2pos), shape=self.shape)
        if self.format == "COO":
            return sp.coo_matrix((self.val, (self.a1crd, self.a2crd)), shape=self.shape)
        raise ValueError("to_scipy: unsupported format " + self.format)


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _idx(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def _index_dtype(*arrays):
    """int32 when every index array is int32 (scipy's default), else int64 -- the
    rule cometpy applies to pick the index type of a sparse tensor
    (frontends/numpy-scipy/cometpy/comet.py:198-218)."""
    return np.int32 if all(np.asarray(a).dtype == np.int32 for a in arrays) else np.int64


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def _vals(a):
    """Values as the library takes them: float32 arrays stay float32 (they select the _f32_ entry points,
    as cometpy's element type does), everything else becomes float64."""
    a = np.asarray(a)
    return np.ascontiguousarray(a, dtype=np.float32 if a.dtype == np.float32 else np.float64)


def as_sparse(m):
    """scipy CSR/COO or a COMET-array object -> SparseTensor (index width kept, values float64)."""
    if isinstance(m, SparseTensor):
        return m
    if hasattr(m, "a2crd") and hasattr(m, "format") and isinstance(m.format, str) and m.format.isupper():
        dt = _index_dtype(m.a1pos, m.a1crd, m.a2pos, m.a2crd)
        return SparseTensor(m.format, m.nrows, m.ncols, _idx(m.a1pos, dt), _idx(m.a1crd, dt), _idx(m.a2pos, dt),
                            _idx(m.a2crd, dt), _vals(m.val))
    fmt = getattr(m, "format", None)
    if fmt == "csr":
        dt = _index_dtype(m.indptr, m.indices)
        return SparseTensor("CSR", m.shape[0], m.shape[1], np.array([m.shape[0]], dtype=dt),
                            np.array([-1], dtype=dt), _idx(m.indptr, dt), _idx(m.indices, dt), _vals(m.data))
    if fmt == "coo":
        dt = _index_dtype(m.row, m.col)
        return SparseTensor("COO", m.shape[0], m.shape[1], np.array([0, m.nnz], dtype=dt),
                            _idx(m.row, dt), np.array([-1], dtype=dt), _idx(m.col, dt), _vals(m.data))
    raise TypeError("unsupported sparse operand: %r (CSR and COO are accepted, like cometpy)" % type(m))


class _Packer:
    """Builds the (rank, descriptor*) argument pairs and keeps the arrays alive."""

    def __init__(self):
        self.keep = []

    def m1(self, arr):
        arr = np.ascontiguousarray(arr)
        d = MemRef1D()
        d.allocated = d.aligned = arr.ctypes.data
        d.offset = 0
        d.sizes[0] = arr.shape[0]
        d.strides[0] = 1
        self.keep += [arr, d]
        return [1, ctypes.addressof(d)]

    def m2(self, arr, transposed_view=False):
        d = MemRef2D()
        d.allocated = d.aligned = arr.ctypes.data
        d.offset = 0
        if transposed_view:       # present row-major [n, k] as a {k, n} memref with strides {1, ld}
            d.sizes[0], d.sizes[1] = arr.shape[1], arr.shape[0]
            d.strides[0], d.strides[1] = 1, arr.strides[0] // arr.itemsize
        else:
            d.sizes[0], d.sizes[1] = arr.shape
            d.strides[0], d.strides[1] = arr.strides[0] // arr.itemsize, arr.strides[1] // arr.itemsize
        self.keep += [arr, d]
        return [2, ctypes.addressof(d)]

    def sparse(self, t):
        f1, f2 = _FMT[t.format]
        empty = np.zeros(0, dtype=t.index_dtype)
        dims = np.array([t.nrows, t.ncols], dtype=np.int64)
        args = [f1, -1, f2, -1]
        args += self.m1(t.a1pos) + self.m1(t.a1crd) + self.m1(empty) + self.m1(empty)
        args += self.m1(t.a2pos) + self.m1(t.a2crd) + self.m1(empty) + self.m1(empty)
        args += self.m1(t.val) + self.m1(dims)
        return args


_F32_OPS = ("spmv", "spmm", "sddmm", "spgemm_symbolic", "spgemm_numeric")


def _entry(lib, name, *tensors, dense=()):
    """The entry point of the operands' common index width and value type, and the sparse operands
    converted to that index width (mixed widths are promoted to int64, like cometpy does).  float32 is
    chosen only when every sparse and dense operand is float32 and the operation has an _f32_ form."""
    dt = np.int32 if all(t.index_dtype == np.int32 for t in tensors) else np.int64
    f32 = (name in _F32_OPS and all(np.asarray(t.val).dtype == np.float32 for t in tensors)
           and all(np.asarray(d).dtype == np.float32 for d in dense))
    fn = getattr(lib, "comet_b200_%s_%s_%s" % (name, "f32" if f32 else "f64", "i32" if dt == np.int32 else "i64"))
    fn.value_dtype = np.float32 if f32 else np.float64
    out = []
    for t in tensors:
        t = t.with_index_dtype(dt)
        if np.asarray(t.val).dtype != fn.value_dtype:
            t = SparseTensor(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd,
                             np.ascontiguousarray(t.val, dtype=fn.value_dtype))
        out.append(t)
    return fn, dt, out


def _semiring(s):
    if s is None:
        return PLUS_TIMES
    key = s.replace(" ", "") if isinstance(s, str) else s
    if key not in _SEMIRINGS:
        raise ValueError("unsupported semiring %r" % (s,))
    return _SEMIRINGS[key]


def _dense_semiring(s):
    code = _semiring(s)
    if code not in _DENSE_OUTPUT_SEMIRINGS:
        raise ValueError("unsupported semiring %r for a dense result (plus-times and plus-pair are handled)" % (s,))
    return code


def spmv(A, x, y0=None, semiring=PLUS_TIMES):
    """y = y0 + A @ x  (ta.mul, sparse x dense vector)."""
    A = as_sparse(A)
    lib = _lib.load()
    pk = _Packer()
    fn, _, (A,) = _entry(lib, "spmv", A, dense=(x,) if y0 is None else (x, y0))
    vt = fn.value_dtype
    x = np.ascontiguousarray(x, dtype=vt)
    y = np.zeros(A.nrows, dtype=vt) if y0 is None else np.array(y0, dtype=vt)
    fn(*pk.sparse(A), *pk.m1(x), *pk.m1(y), _dense_semiring(semiring), 0 if y0 is None else 1)
    _lib.check()
    return y


def _name(op, sharded):
    """``sharded``: the collective form of the call, under the communicator set up by
    ``sharding.init_library_comm``: the left operand, mask and result are this rank's row block, the right
    operand is the whole matrix (identical on every rank)."""
    return op + "_sharded" if sharded else op


def spmm(A, B, C0=None, semiring=PLUS_TIMES, sharded=False):
    """C = C0 + A @ B  (ta.mul, sparse x dense matrix), B row-major."""
    A = as_sparse(A)
    lib = _lib.load()
    pk = _Packer()
    fn, _, (A,) = _entry(lib, _name("spmm", sharded), A, dense=(B,) if C0 is None else (B, C0))
    vt = fn.value_dtype
    B = np.ascontiguousarray(B, dtype=vt)
    C = np.zeros((A.nrows, B.shape[1]), dtype=vt) if C0 is None else np.array(C0, dtype=vt, order="C")
    fn(*pk.sparse(A), *pk.m2(B), *pk.m2(C), _dense_semiring(semiring), 0 if C0 is None else 1)
    _lib.check()
    return C


def dense_times_sparse(A, B, C0=None, semiring=PLUS_TIMES):
    """C = C0 + A @ B with dense A (vector or row-major matrix) and sparse B (CSR, DCSR or COO):
    the `dense @ sparse` forms of cometpy."""
    B = as_sparse(B)
    lib = _lib.load()
    pk = _Packer()
    A = _f64(A)
    vec = A.ndim == 1
    shape = (B.ncols,) if vec else (A.shape[0], B.ncols)
    C = np.zeros(shape) if C0 is None else _f64(C0).reshape(shape).copy()
    fn, _, (B,) = _entry(lib, "dense_times_sparse", B)
    pack = pk.m1 if vec else pk.m2
    fn(*pack(A), *pk.sparse(B), *pack(C), _dense_semiring(semiring), 0 if C0 is None else 1)
    _lib.check()
    return C


def sddmm(S, X, Y, y_is_kj=False, sharded=False):
    """values of S .* (X @ Y^T) on S's pattern.  Y is [cols, K] row-major, or the
    [K, cols] operand D[k,j] of the reference's sddmm.ta when ``y_is_kj``."""
    S = as_sparse(S)
    lib = _lib.load()
    pk = _Packer()
    fn, _, (S,) = _entry(lib, _name("sddmm", sharded), S, dense=(X, Y))
    vt = fn.value_dtype
    X, Y = np.ascontiguousarray(X, dtype=vt), np.ascontiguousarray(Y, dtype=vt)
    out = SparseTensor("CSR", S.nrows, S.ncols, np.zeros_like(S.a1pos), np.zeros_like(S.a1crd),
                       np.zeros_like(S.a2pos), np.zeros_like(S.a2crd), np.zeros(S.nnz, dtype=vt))
    d_args = pk.m2(Y) if y_is_kj else pk.m2(Y, transposed_view=True)
    fn(*pk.sparse(S), *pk.m2(X), *d_args, *pk.sparse(out))
    _lib.check()
    assert np.array_equal(out.a2pos, S.a2pos) and np.array_equal(out.a2crd, S.a2crd)
    return out.val


def elews_sparse_dense(A, B):
    """values of A .* B on A's pattern (A CSR or COO, B dense)."""
    A = as_sparse(A)
    lib = _lib.load()
    pk = _Packer()
    B = _f64(B)
    out = SparseTensor(A.format, A.nrows, A.ncols, np.zeros_like(A.a1pos), np.zeros_like(A.a1crd),
                       np.zeros_like(A.a2pos), np.zeros_like(A.a2crd), np.zeros(A.nnz))
    fn, _, _unused = _entry(lib, "elews_mul_sparse_dense", A)
    fn(*pk.sparse(A), *pk.m2(B), *pk.sparse(out))
    _lib.check()
    return out.val


def elews_sparse_dense_to_dense(A, B, C0=None):
    """Dense C with A.val * B at A's stored positions (A CSR, DCSR or COO), C0 (default zeros) elsewhere."""
    A = as_sparse(A)
    lib = _lib.load()
    pk = _Packer()
    B = _f64(B)
    C = np.zeros((A.nrows, A.ncols)) if C0 is None else _f64(C0).copy()
    fn, _, (A,) = _entry(lib, "elews_mul_sparse_dense_to_dense", A)
    fn(*pk.sparse(A), *pk.m2(B), *pk.m2(C))
    _lib.check()
    return C


def _finish_sparse_out(lib, handle, nrows, ncols, cpos, sizes, vt=np.float64):
    _lib.check()
    nnz = int(sizes[8])
    dt = cpos.dtype
    ccrd = np.zeros(nnz, dtype=dt)
    cval = np.zeros(nnz, dtype=vt)
    pk = _Packer()
    fn = getattr(lib, "comet_b200_spgemm_numeric_%s_%s" % ("f32" if vt == np.float32 else "f64",
                                                           "i32" if dt == np.int32 else "i64"))
    fn(handle, *pk.m1(ccrd), *pk.m1(cval))
    _lib.check()
    return SparseTensor("CSR", nrows, ncols, np.array([nrows], dtype=dt), np.array([-1], dtype=dt), cpos, ccrd,
                        cval)


def spgemm(A, B, M=None, semiring=PLUS_TIMES, sharded=False):
    """C = A @ B, or C<M,push> = A @ B, all CSR; returns a CSR SparseTensor.  With ``sharded`` the
    result is this rank's row block and carries ``entry_offset`` / ``total_nnz`` (its place in the whole C)."""
    A, B = as_sparse(A), as_sparse(B)
    Mt = as_sparse(M) if M is not None else A
    lib = _lib.load()
    pk = _Packer()
    fn, dt, (A, B, Mt) = _entry(lib, _name("spgemm_symbolic", sharded), A, B, Mt)
    cpos = np.zeros(A.nrows + 1, dtype=dt)
    sizes = np.zeros(13, dtype=np.int64)
    handle = fn(*pk.sparse(A), *pk.sparse(B), *pk.sparse(Mt), MASK_PUSH if M is not None else MASK_NONE,
                _semiring(semiring), *pk.m1(cpos), *pk.m1(sizes))
    C = _finish_sparse_out(lib, handle, A.nrows, B.ncols, cpos, sizes, fn.value_dtype)
    if sharded:
        C.entry_offset, C.total_nnz = int(sizes[11]), int(sizes[12])
    return C


def elews_csr_csr(A, B):
    """C = A .* B with both operands CSR."""
    A, B = as_sparse(A), as_sparse(B)
    lib = _lib.load()
    pk = _Packer()
    fn, dt, (A, B) = _entry(lib, "elews_mul_sparse_sparse_symbolic", A, B)
    cpos = np.zeros(A.nrows + 1, dtype=dt)
    sizes = np.zeros(11, dtype=np.int64)
    handle = fn(*pk.sparse(A), *pk.sparse(B), *pk.m1(cpos), *pk.m1(sizes))
    return _finish_sparse_out(lib, handle, A.nrows, A.ncols, cpos, sizes)


def masked_pair_count(A, B, M, sharded=False):
    """SUM(C<M,push> = A @ B) under plus-pair as an exact integer (with ``sharded``: over all ranks' blocks)."""
    A, B, M = as_sparse(A), as_sparse(B), as_sparse(M)
    lib = _lib.load()
    pk = _Packer()
    out = np.zeros(1, dtype=np.int64)
    fn, _, (A, B, M) = _entry(lib, _name("masked_spgemm_count", sharded), A, B, M)
    fn(*pk.sparse(A), *pk.sparse(B), *pk.sparse(M), MASK_PUSH, PLUS_PAIR, *pk.m1(out))
    _lib.check()
    return int(out[0])


def triangle_count(L):
    """Sandia LL: sum((L @ L) .* L) for the strict lower triangle L of a symmetric graph
    (test/integration/kernels/triangleCount_SandiaLL_wMasking.ta)."""
    return masked_pair_count(L, L, L)


def transpose(A):
    """Transpose of a CSR or COO matrix in the same format, through the entry point that stands in
    for the reference runtime's transpose_2D_f64_i64 (lib/ExecutionEngine/TransposeUtils.cpp:1439)."""
    A = as_sparse(A)
    if A.format not in ("CSR", "COO"):
        raise ValueError("transpose: CSR and COO are handled")
    lib = _lib.load()
    dt = A.index_dtype if A.index_dtype == np.int32 else np.dtype(np.int64)
    A = A.with_index_dtype(dt)
    fn = getattr(lib, "comet_b200_transpose_2D_f64_%s" % ("i32" if dt == np.int32 else "i64"))
    pk = _Packer()
    nnz = A.nnz
    if A.format == "CSR":
        b1pos, b1crd = np.zeros(1, dtype=dt), np.zeros(1, dtype=dt)
        b2pos = np.zeros(A.ncols + 1, dtype=dt)
    else:
        b1pos, b1crd = np.zeros(2, dtype=dt), np.zeros(nnz, dtype=dt)
        b2pos = np.zeros(1, dtype=dt)
    b2crd, bval = np.zeros(nnz, dtype=dt), np.zeros(nnz)
    sizes = np.array([A.nrows, A.ncols] + [0] * 9, dtype=dt)
    empty = np.zeros(0, dtype=dt)
    f1, f2 = _FMT[A.format]

    def block(a1pos, a1crd, a2pos, a2crd, val):
        return ([f1, -1, f2, -1] + pk.m1(a1pos) + pk.m1(a1crd) + pk.m1(empty) + pk.m1(empty) + pk.m1(a2pos) +
                pk.m1(a2crd) + pk.m1(empty) + pk.m1(empty) + pk.m1(val))

    fn(*block(A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val), *block(b1pos, b1crd, b2pos, b2crd, bval), *pk.m1(sizes))
    _lib.check()
    return SparseTensor(A.format, int(sizes[0]), int(sizes[1]), b1pos, b1crd, b2pos, b2crd, bval)


def read_mtx(path, fmt="CSR", read_mode=1, index_dtype=np.int64, file_id=0):
    """MatrixMarket file -> COMET arrays through the two reader entry points (sizes, then fill), the way
    generated code calls read_input_sizes_2D_f64 / read_input_2D_f64_i64
    (lib/Conversion/TensorAlgebraToSCF/TensorDeclLowering.cpp:937-1052).  The sort runs on the device."""
    import os
    lib = _lib.load()
    os.environ["SPARSE_FILE_NAME%d" % file_id] = os.fspath(path)
    f1, f2 = _FMT[fmt]
    pk = _Packer()
    sizes = np.zeros(11, dtype=np.int64)
    lib.comet_b200_read_input_sizes_2D_f64(file_id, f1, -1, f2, -1, *pk.m1(sizes), int(read_mode))
    _lib.check()
    dt = np.dtype(index_dtype)
    arrs = [np.zeros(max(int(sizes[i]), 1), dtype=dt) for i in (0, 1, 4, 5)]
    val = np.zeros(max(int(sizes[8]), 1))
    empty = np.zeros(0, dtype=dt)
    fn = lib.comet_b200_read_input_2D_f64_i32 if dt == np.int32 else lib.comet_b200_read_input_2D_f64_i64
    fn(file_id, f1, -1, f2, -1, *pk.m1(arrs[0]), *pk.m1(arrs[1]), *pk.m1(empty), *pk.m1(empty), *pk.m1(arrs[2]),
       *pk.m1(arrs[3]), *pk.m1(empty), *pk.m1(empty), *pk.m1(val), int(read_mode))
    _lib.check()
    return SparseTensor(fmt, int(sizes[9]), int(sizes[10]), arrs[0][:int(sizes[0])], arrs[1][:int(sizes[1])],
                        arrs[2][:int(sizes[4])], arrs[3][:int(sizes[5])], val[:int(sizes[8])])


def from_coordinates(rows, cols, vals, shape):
    """CSR from coordinate entries in any order, sorted on the device the way the reference reader sorts
    them on the host (by row, then column; entries with equal coordinates stay in input order and are
    kept, lib/ExecutionEngine/SparseUtils.cpp:360-533)."""
    import torch
    lib = _lib.load()
    nrows, ncols = int(shape[0]), int(shape[1])
    r = torch.from_numpy(_i64(rows)).cuda()
    c = torch.from_numpy(_i64(cols)).cuda()
    v = torch.from_numpy(_f64(vals)).cuda()
    nnz = int(r.shape[0])
    pos = torch.empty(nrows + 1, dtype=torch.int64, device="cuda")
    crd = torch.empty(nnz, dtype=torch.int64, device="cuda")
    val = torch.empty(nnz, dtype=torch.float64, device="cuda")
    st = lib.comet_b200_dev_coo_to_csr_f64_i64(nrows, ncols, nnz, r.data_ptr(), c.data_ptr(), v.data_ptr(),
                                               pos.data_ptr(), crd.data_ptr(), val.data_ptr(),
                                               torch.cuda.current_stream().cuda_stream)
    _lib.check(st)
    torch.cuda.synchronize()
    return SparseTensor("CSR", nrows, ncols, np.array([nrows], dtype=np.int64), np.array([-1], dtype=np.int64),
                        pos.cpu().numpy(), crd.cpu().numpy(), val.cpu().numpy())


def reduce_sum(vals):
    """ta.reduce over stored values.  Not part of the device path: the values are
    host memrefs after every call, and COMET's generated loop sums them there
    (lib/Conversion/TensorAlgebraToSCF/TensorAlgebraToSCF.cpp:483-517)."""
    s = 0.0
    for v in np.asarray(vals, dtype=np.float64).ravel():
        s = s + float(v)
    return s


def einsum(subscripts, A, B, mask=None, mask_type="push", semiring="+,*"):
    """The cometpy einsum forms that reach the sparse hot path
    (frontends/numpy-scipy/cometpy/comet.py:1210-1319): 'ij,jk->ik' with a sparse
    first operand and a dense or sparse second one, and 'ij,j->i'."""
    spec = subscripts.replace(" ", "")
    lhs, out = spec.split("->")
    a, b = lhs.split(",")
    if not (a[-1] == b[0]):
        raise ValueError("unsupported einsum " + subscripts)
    if mask is not None and mask_type != "push":
        raise ValueError("only the push mask is handled")
    sr = _semiring(semiring)
    sparse_a = hasattr(A, "format") or hasattr(A, "a2crd")
    sparse_b = hasattr(B, "format") or hasattr(B, "a2crd")
    if not sparse_a and sparse_b:
        ok = (len(a) == 1 and len(b) == 2 and a == b[0] and out == b[1]) or \
             (len(a) == 2 and len(b) == 2 and out == a[0] + b[1])
        if not ok:
            raise ValueError("unsupported einsum " + subscripts)
        return dense_times_sparse(A, B, semiring=sr)
    if len(b) == 1 and out == a[0]:
        return spmv(A, B, semiring=sr)
    if len(b) == 2 and out == a[0] + b[1]:
        if sparse_b:
            return spgemm(A, B, mask, sr)
        return spmm(A, B, semiring=sr)
    raise ValueError("unsupported einsum " + subscripts)
