"""ctypes front end of the CPU oracle (TEST INFRASTRUCTURE, not product code).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the shipped library never does.  Every function here forwards to
``libcomet_oracle.so`` (built from ``comet_oracle.c`` by ``oracle/Makefile``),
whose header cites the COMET source lines each loop nest restates.

All index arrays are int64, all values float64, matching COMET's CPU path
(frontends/comet_dsl/comet.cpp:817-823 picks i64 indices for the CPU target).
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcomet_oracle.so")

PLUS_TIMES, PLUS_PAIR, PLUS_FIRST, PLUS_SECOND, MIN_PLUS, MIN_FIRST, MIN_SECOND, ANY_PAIR = range(8)

# runtime format codes: include/comet/ExecutionEngine/RunnerUtils.h:71-77
DENSE, CU, CN, S = 0, 1, 2, 3
FORMATS = {"CSR": (DENSE, CU), "DCSR": (CU, CU), "COO": (CN, S)}

_LIB32_PATH = os.path.join(_HERE, "libcomet_oracle_f32.so")   # the same loops with float values

_lib = None
_lib32 = None


def build(force=False):
    """Compile the oracle with gcc (no GPU needed)."""
    src = os.path.join(_HERE, "comet_oracle.c")
    stale = lambda p: not os.path.exists(p) or os.path.getmtime(p) < os.path.getmtime(src)
    if force or stale(_LIB_PATH) or stale(_LIB32_PATH):
        subprocess.check_call(["make", "-C", _HERE, "-B", "all"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_reader_open.restype = ctypes.c_void_p
        _lib.oracle_reader_open.argtypes = [ctypes.c_char_p]
        _lib.oracle_reader_close.argtypes = [ctypes.c_void_p]
        _lib.oracle_spgemm_symbolic.restype = ctypes.c_int64
        _lib.oracle_elews_csr_csr.restype = ctypes.c_int64
        _lib.oracle_masked_pair_count.restype = ctypes.c_int64
        _lib.oracle_masked_pair_count_rowparallel.restype = ctypes.c_int64
        _lib.oracle_spgemm_rowparallel.restype = ctypes.c_int64
        _lib.oracle_reduce_sum.restype = ctypes.c_double
    return _lib


def num_threads():
    return int(lib().oracle_num_threads())


def use_all_cores():
    """Launchers such as torch.distributed.run export OMP_NUM_THREADS=1; the CPU baseline is meant
    to use every core of the host, so set the team size explicitly."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


def _f64(a):
    return np.ascontiguousarray(a, dtype=np.float64)


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _l(v):
    return ctypes.c_int64(int(v))


class SparseArrays:
    """The per-dimension arrays COMET keeps for one sparse matrix, with the
    shapes read_input_sizes_2D reports (lib/ExecutionEngine/SparseUtils.cpp:1643-1751)."""

    def __init__(self, fmt, nrows, ncols, a1pos, a1crd, a2pos, a2crd, val):
        self.format = fmt
        self.nrows, self.ncols = int(nrows), int(ncols)
        self.a1pos, self.a1crd, self.a2pos, self.a2crd, self.val = a1pos, a1crd, a2pos, a2crd, val

    @property
    def nnz(self):
        return int(self.val.shape[0])


def read_mtx(path, fmt="CSR", read_mode=1):
    """MatrixMarket file -> COMET arrays, following the reference reader."""
    L = lib()
    h = L.oracle_reader_open(os.fsencode(path))
    if not h:
        raise IOError("oracle: cannot read " + str(path))
    try:
        f1, f2 = FORMATS[fmt]
        sizes = np.zeros(11, dtype=np.int64)
        if L.oracle_reader_sizes(ctypes.c_void_p(h), f1, f2, int(read_mode), _p(sizes)) != 0:
            raise ValueError("oracle: unsupported format " + fmt)
        a1pos = np.zeros(max(int(sizes[0]), 1), dtype=np.int64)
        a1crd = np.zeros(max(int(sizes[1]), 1), dtype=np.int64)
        a2pos = np.zeros(max(int(sizes[4]), 1), dtype=np.int64)
        a2crd = np.zeros(max(int(sizes[5]), 1), dtype=np.int64)
        val = np.zeros(max(int(sizes[8]), 1), dtype=np.float64)
        L.oracle_reader_fill(ctypes.c_void_p(h), f1, f2, int(read_mode), _p(a1pos), _p(a1crd),
                             _p(a2pos), _p(a2crd), _p(val))
        return SparseArrays(fmt, sizes[9], sizes[10], a1pos[:int(sizes[0])], a1crd[:int(sizes[1])],
                            a2pos[:int(sizes[4])], a2crd[:int(sizes[5])], val[:int(sizes[8])])
    finally:
        L.oracle_reader_close(ctypes.c_void_p(h))


# --- dense-output products --------------------------------------------------

def spmv(A, x, y0=None, semiring=PLUS_TIMES):
    x = _f64(x)
    y = np.zeros(A.nrows) if y0 is None else _f64(y0).copy()
    L = lib()
    if A.format == "CSR":
        L.oracle_spmv_csr(_l(A.nrows), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)), _p(_f64(A.val)),
                          _p(x), _p(y), int(semiring))
    elif A.format == "DCSR":
        L.oracle_spmv_dcsr(_p(_i64(A.a1pos)), _p(_i64(A.a1crd)), _p(_i64(A.a2pos)),
                           _p(_i64(A.a2crd)), _p(_f64(A.val)), _p(x), _p(y), int(semiring))
    elif A.format == "COO":
        L.oracle_spmv_coo(_p(_i64(A.a1pos)), _p(_i64(A.a1crd)), _p(_i64(A.a2crd)),
                          _p(_f64(A.val)), _p(x), _p(y), int(semiring))
    else:
        raise ValueError(A.format)
    return y


def spmm(A, B, C0=None, semiring=PLUS_TIMES):
    B = _f64(B)
    k = B.shape[1]
    C = np.zeros((A.nrows, k)) if C0 is None else _f64(C0).copy()
    L = lib()
    if A.format == "CSR":
        L.oracle_spmm_csr(_l(A.nrows), _l(k), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)),
                          _p(_f64(A.val)), _p(B), _l(k), _p(C), _l(k), int(semiring))
    elif A.format == "DCSR":
        L.oracle_spmm_dcsr(_l(k), _p(_i64(A.a1pos)), _p(_i64(A.a1crd)), _p(_i64(A.a2pos)),
                           _p(_i64(A.a2crd)), _p(_f64(A.val)), _p(B), _l(k), _p(C), _l(k),
                           int(semiring))
    elif A.format == "COO":
        L.oracle_spmm_coo(_l(k), _p(_i64(A.a1pos)), _p(_i64(A.a1crd)), _p(_i64(A.a2crd)),
                          _p(_f64(A.val)), _p(B), _l(k), _p(C), _l(k), int(semiring))
    else:
        raise ValueError(A.format)
    return C


def dense_times_sparse(A, B, C0=None, semiring=PLUS_TIMES):
    """C = C0 + A @ B with dense A (vector or matrix) and sparse B (CSR / DCSR / COO)."""
    A = _f64(A)
    vec = A.ndim == 1
    A2 = A.reshape(1, -1) if vec else A
    m = A2.shape[0]
    C = np.zeros((m, B.ncols)) if C0 is None else _f64(C0).reshape(m, B.ncols).copy()
    if B.format == "CSR":
        nst, rows, pos = B.nrows, None, _i64(B.a2pos)
    elif B.format == "DCSR":
        nst, rows, pos = int(B.a1pos[1]), _i64(B.a1crd), _i64(B.a2pos)
    else:
        nst, rows, pos = B.nnz, _i64(B.a1crd), None
    lib().oracle_dense_times_sparse(_l(m), _l(nst), _p(rows), _p(pos), _p(_i64(B.a2crd)), _p(_f64(B.val)),
                                    _p(A2), _l(A2.shape[1]), _p(C), _l(B.ncols), int(semiring))
    return C[0] if vec else C


def sddmm(S, X, Y, y_is_kj=False):
    """out.val = S.val * (X @ Y^T sampled on S).  ``Y`` is (ncols, K) row-major,
    or (K, ncols) row-major when ``y_is_kj`` (the D[k,j] operand of sddmm.ta)."""
    X, Y = _f64(X), _f64(Y)
    k = X.shape[1]
    out = np.zeros(S.nnz)
    if y_is_kj:
        ys_k, ys_j = Y.shape[1], 1
    else:
        ys_k, ys_j = 1, Y.shape[1]
    lib().oracle_sddmm_csr(_l(S.nrows), _l(k), _p(_i64(S.a2pos)), _p(_i64(S.a2crd)),
                           _p(_f64(S.val)), _p(X), _l(k), _p(Y), _l(ys_k), _l(ys_j), _p(out))
    return out


def elews_sparse_dense(A, B):
    B = _f64(B)
    out = np.zeros(A.nnz)
    if A.format == "CSR":
        lib().oracle_elews_csr_dense(_l(A.nrows), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)),
                                     _p(_f64(A.val)), _p(B), _l(B.shape[1]), _p(out))
    elif A.format == "COO":
        lib().oracle_elews_coo_dense(_l(A.nnz), _p(_i64(A.a1crd)), _p(_i64(A.a2crd)),
                                     _p(_f64(A.val)), _p(B), _l(B.shape[1]), _p(out))
    else:
        raise ValueError(A.format)
    return out


def transpose(A):
    """Transpose of a CSR or COO matrix in the same format: the entries ordered by (column, row) of
    the input, the CSR -> COO -> sort -> CSR route of transpose_2D
    (lib/ExecutionEngine/TransposeUtils.cpp:738-812; COO: :625-697).  Entries with equal coordinates
    keep their input order."""
    if A.format == "CSR":
        rows = np.repeat(np.arange(A.nrows, dtype=np.int64), np.diff(_i64(A.a2pos)))
    elif A.format == "COO":
        rows = _i64(A.a1crd)
    else:
        raise ValueError("transpose: CSR and COO")
    cols = _i64(A.a2crd)
    order = np.lexsort((rows, cols))                     # stable: by column, then row, then position
    if A.format == "COO":
        return SparseArrays("COO", A.ncols, A.nrows, np.array([0, A.nnz], dtype=np.int64), cols[order],
                            np.array([-1], dtype=np.int64), rows[order], A.val[order])
    pos = np.zeros(A.ncols + 1, dtype=np.int64)
    np.cumsum(np.bincount(cols, minlength=A.ncols), out=pos[1:])
    return SparseArrays("CSR", A.ncols, A.nrows, np.array([A.ncols], dtype=np.int64), np.array([-1], dtype=np.int64),
                        pos, rows[order], A.val[order])


def elews_sparse_dense_to_dense(A, B, C0=None):
    """Dense result of ta.elews_mul with one sparse operand: products at the stored positions
    (lib/Conversion/IndexTreeToSCF/IndexTreeToSCF.cpp:1247-1284 with the "noop" reduce)."""
    B = _f64(B)
    C = np.zeros((A.nrows, A.ncols)) if C0 is None else _f64(C0).copy()
    if A.format == "COO":
        rows = _i64(A.a1crd)
    elif A.format == "DCSR":
        rows = np.repeat(_i64(A.a1crd)[:int(A.a1pos[1])], np.diff(_i64(A.a2pos)))
    else:
        rows = np.repeat(np.arange(A.nrows), np.diff(_i64(A.a2pos)))
    cols = _i64(A.a2crd)
    for p in range(A.nnz):          # sequential like the reference: a repeated coordinate keeps the last product
        C[rows[p], cols[p]] = A.val[p] * B[rows[p], cols[p]]
    return C


def elews_csr_csr(A, B):
    L = lib()
    cpos = np.zeros(A.nrows + 1, dtype=np.int64)
    args = (_l(A.nrows), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)), _p(_f64(A.val)),
            _p(_i64(B.a2pos)), _p(_i64(B.a2crd)), _p(_f64(B.val)))
    nnz = L.oracle_elews_csr_csr(*args, _p(cpos), None, None)
    ccrd = np.zeros(max(nnz, 1), dtype=np.int64)
    cval = np.zeros(max(nnz, 1))
    L.oracle_elews_csr_csr(*args, _p(cpos), _p(ccrd), _p(cval))
    return SparseArrays("CSR", A.nrows, A.ncols, np.array([A.nrows], dtype=np.int64),
                        np.array([-1], dtype=np.int64), cpos, ccrd[:nnz], cval[:nnz])


# --- sparse-output products -------------------------------------------------

def spgemm(A, B, M=None, semiring=PLUS_TIMES):
    """C = A*B (optionally C<M,push>), CSR operands, Gustavson with workspace."""
    L = lib()
    apos, acrd, aval = _i64(A.a2pos), _i64(A.a2crd), _f64(A.val)
    bpos, bcrd, bval = _i64(B.a2pos), _i64(B.a2crd), _f64(B.val)
    mpos = _i64(M.a2pos) if M is not None else None
    mcrd = _i64(M.a2crd) if M is not None else None
    cpos = np.zeros(A.nrows + 1, dtype=np.int64)
    nnz = L.oracle_spgemm_symbolic(_l(A.nrows), _l(B.ncols), _p(apos), _p(acrd), _p(bpos),
                                   _p(bcrd), _p(mpos), _p(mcrd), _p(cpos))
    ccrd = np.zeros(max(nnz, 1), dtype=np.int64)
    cval = np.zeros(max(nnz, 1))
    L.oracle_spgemm_numeric(_l(A.nrows), _l(B.ncols), _p(apos), _p(acrd), _p(aval), _p(bpos),
                            _p(bcrd), _p(bval), _p(mpos), _p(mcrd), int(semiring), _p(cpos),
                            _p(ccrd), _p(cval))
    return SparseArrays("CSR", A.nrows, B.ncols, np.array([A.nrows], dtype=np.int64),
                        np.array([-1], dtype=np.int64), cpos, ccrd[:nnz], cval[:nnz])


def spgemm_rowparallel(A, B, semiring=PLUS_TIMES):
    """C = A*B with the rows of A handed to OpenMP threads, a workspace per thread.  NOT COMET's schedule
    (its sparse-output loops are sequential); same result as ``spgemm``.  For the benchmark's second CPU figure."""
    L = lib()
    apos, acrd, aval = _i64(A.a2pos), _i64(A.a2crd), _f64(A.val)
    bpos, bcrd, bval = _i64(B.a2pos), _i64(B.a2crd), _f64(B.val)
    cpos = np.zeros(A.nrows + 1, dtype=np.int64)
    args = (_l(A.nrows), _l(B.ncols), _p(apos), _p(acrd), _p(aval), _p(bpos), _p(bcrd), _p(bval), int(semiring))
    nnz = L.oracle_spgemm_rowparallel(*args, _p(cpos), None, None)
    ccrd = np.zeros(max(nnz, 1), dtype=np.int64)
    cval = np.zeros(max(nnz, 1))
    L.oracle_spgemm_rowparallel(*args, _p(cpos), _p(ccrd), _p(cval))
    return SparseArrays("CSR", A.nrows, B.ncols, np.array([A.nrows], dtype=np.int64),
                        np.array([-1], dtype=np.int64), cpos, ccrd[:nnz], cval[:nnz])


def masked_pair_count_rowparallel(A, B, M, row_lo=0, row_hi=None):
    """``masked_pair_count`` with the rows handed to OpenMP threads (NOT COMET's schedule); same count."""
    row_hi = A.nrows if row_hi is None else row_hi
    return int(lib().oracle_masked_pair_count_rowparallel(
        _l(row_lo), _l(row_hi), _l(B.ncols), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)),
        _p(_i64(B.a2pos)), _p(_i64(B.a2crd)), _p(_i64(M.a2pos)), _p(_i64(M.a2crd))))


def reduce_sum(vals):
    vals = _f64(vals)
    return float(lib().oracle_reduce_sum(_l(vals.shape[0]), _p(vals)))


def masked_pair_count(A, B, M, row_lo=0, row_hi=None):
    """SUM(C<M,push> = A*B) under plus-pair over rows [row_lo, row_hi)."""
    row_hi = A.nrows if row_hi is None else row_hi
    return int(lib().oracle_masked_pair_count(
        _l(row_lo), _l(row_hi), _l(B.ncols), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)),
        _p(_i64(B.a2pos)), _p(_i64(B.a2crd)), _p(_i64(M.a2pos)), _p(_i64(M.a2crd))))


def from_scipy_csr(m):
    """scipy CSR -> SparseArrays with int64 indices (no sorting, no dedup)."""
    return SparseArrays("CSR", m.shape[0], m.shape[1], np.array([m.shape[0]], dtype=np.int64),
                        np.array([-1], dtype=np.int64), _i64(m.indptr), _i64(m.indices),
                        _f64(m.data))


def print_memref(a):
    """Text that comet_print_memref_{i64,f64} writes for a 1-D array
    (lib/ExecutionEngine/StatUtils.cpp:90-140, RunnerUtils.h:232-266):
    'data = ' then values at ostream default precision, each followed by ','."""
    a = np.asarray(a).reshape(-1)
    if a.dtype.kind in "iu":
        body = "".join("%d," % int(v) for v in a)
    else:
        body = "".join("%g," % float(v) for v in a)
    return "data = \n" + body + "\n"


# --- single precision: the same loop nests compiled with float values (libcomet_oracle_f32.so) -----------

def lib32():
    global _lib32
    if _lib32 is None:
        if not os.path.exists(_LIB32_PATH):
            build(force=True)
        _lib32 = ctypes.CDLL(_LIB32_PATH)
        _lib32.oracle_spgemm_symbolic.restype = ctypes.c_int64
    return _lib32


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def spmv_f32(A, x):
    x = _f32(x)
    y = np.zeros(A.nrows, dtype=np.float32)
    lib32().oracle_spmv_csr(_l(A.nrows), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)), _p(_f32(A.val)), _p(x), _p(y), 0)
    return y


def spmm_f32(A, B):
    B = _f32(B)
    k = B.shape[1]
    C = np.zeros((A.nrows, k), dtype=np.float32)
    lib32().oracle_spmm_csr(_l(A.nrows), _l(k), _p(_i64(A.a2pos)), _p(_i64(A.a2crd)), _p(_f32(A.val)), _p(B),
                            _l(k), _p(C), _l(k), 0)
    return C


def sddmm_f32(S, X, Y):
    X, Y = _f32(X), _f32(Y)
    k = X.shape[1]
    out = np.zeros(S.nnz, dtype=np.float32)
    lib32().oracle_sddmm_csr(_l(S.nrows), _l(k), _p(_i64(S.a2pos)), _p(_i64(S.a2crd)), _p(_f32(S.val)), _p(X),
                             _l(k), _p(Y), _l(1), _l(k), _p(out))
    return out


def spgemm_f32(A, B):
    L = lib32()
    apos, acrd, aval = _i64(A.a2pos), _i64(A.a2crd), _f32(A.val)
    bpos, bcrd, bval = _i64(B.a2pos), _i64(B.a2crd), _f32(B.val)
    cpos = np.zeros(A.nrows + 1, dtype=np.int64)
    nnz = L.oracle_spgemm_symbolic(_l(A.nrows), _l(B.ncols), _p(apos), _p(acrd), _p(bpos), _p(bcrd), None, None,
                                   _p(cpos))
    ccrd = np.zeros(max(nnz, 1), dtype=np.int64)
    cval = np.zeros(max(nnz, 1), dtype=np.float32)
    L.oracle_spgemm_numeric(_l(A.nrows), _l(B.ncols), _p(apos), _p(acrd), _p(aval), _p(bpos), _p(bcrd), _p(bval),
                            None, None, 0, _p(cpos), _p(ccrd), _p(cval))
    return SparseArrays("CSR", A.nrows, B.ncols, np.array([A.nrows], dtype=np.int64),
                        np.array([-1], dtype=np.int64), cpos, ccrd[:nnz], cval[:nnz])
