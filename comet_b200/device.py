"""Device-resident operands: calls layer 2 of the C ABI (``comet_b200_dev_*``) on
torch CUDA tensors.  torch supplies device memory and streams only; every
computation is done by the kernels of ``libcomet_b200``.

Used by the benchmark (inputs already in HBM when the clock starts), by the
multi-GPU sharding layer and by the device-level parity tests.
"""
import ctypes

import numpy as np
import torch

from . import _lib
from .api import PLUS_PAIR, PLUS_TIMES, as_sparse  # noqa: F401


class DeviceCSR:
    """A CSR (or DCSR when ``row_ids`` is set) matrix in device memory, int64 / float64."""

    def __init__(self, nrows, ncols, pos, crd, val, row_ids=None):
        self.nrows, self.ncols = int(nrows), int(ncols)
        self.pos, self.crd, self.val, self.row_ids = pos, crd, val, row_ids
        self.nnz = int(crd.shape[0])

    @property
    def nstored(self):
        return int(self.pos.shape[0]) - 1


def to_device(A, device="cuda", pin=False):
    """Host COMET arrays / scipy matrix -> DeviceCSR (COO is not taken here)."""
    A = as_sparse(A)
    if A.format == "COO":
        raise ValueError("to_device: pass CSR or DCSR (the host entry points convert COO)")

    def up(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        if pin:
            t = t.pin_memory()
        return t.to(device, non_blocking=pin)

    i64 = lambda a: np.asarray(a, dtype=np.int64)       # the device entry points take int64 indices
    row_ids = up(i64(A.a1crd[:int(A.a1pos[1])])) if A.format == "DCSR" else None
    return DeviceCSR(A.nrows, A.ncols, up(i64(A.a2pos)), up(i64(A.a2crd)), up(A.val), row_ids)


def _p(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _check_cuda(*ts):
    for t in ts:
        if t is not None and (not t.is_cuda or not t.is_contiguous()):
            raise ValueError("device entry points need contiguous CUDA tensors")


def spmv(A, x, y=None, semiring=PLUS_TIMES, accumulate=False):
    _check_cuda(A.pos, A.crd, A.val, x, y)
    if y is None:
        y = torch.zeros(A.nrows, dtype=torch.float64, device=x.device)
    lib = _lib.load()
    st = lib.comet_b200_dev_spmv_f64_i64(A.nstored, A.nnz, _p(A.row_ids), _p(A.pos), _p(A.crd),
                                         _p(A.val), _p(x), _p(y), semiring, int(accumulate), _stream())
    _lib.check(st)
    return y


def spmm(A, B, C=None, semiring=PLUS_TIMES, accumulate=False, variant=0):
    """B may be a column slice of a wider row-major array (unit column stride); its row stride is passed on."""
    _check_cuda(A.pos, A.crd, A.val, C)
    if not B.is_cuda or B.dim() != 2 or B.stride(1) != 1:
        raise ValueError("B must be a CUDA matrix with unit column stride")
    k = B.shape[1]
    if C is None:
        C = torch.empty((A.nrows, k), dtype=torch.float64, device=B.device)
        if A.row_ids is not None:
            C.zero_()
    lib = _lib.load()
    st = lib.comet_b200_dev_spmm_f64_i64(A.nstored, A.ncols, A.nnz, k, _p(A.row_ids), _p(A.pos),
                                         _p(A.crd), _p(A.val), _p(B), B.stride(0), _p(C), C.stride(0),
                                         semiring, int(accumulate), int(variant), _stream())
    _lib.check(st)
    return C


def sddmm(S, X, Y, out=None):
    """Y is [ncols, K] row-major."""
    _check_cuda(S.pos, S.crd, S.val, X, Y, out)
    if out is None:
        out = torch.empty(S.nnz, dtype=torch.float64, device=X.device)
    lib = _lib.load()
    st = lib.comet_b200_dev_sddmm_f64_i64(S.nrows, S.nnz, X.shape[1], _p(S.pos), _p(S.crd), _p(S.val),
                                          _p(X), X.stride(0), _p(Y), Y.stride(0), _p(out), _stream())
    _lib.check(st)
    return out


class SpgemmResult:
    def __init__(self, nrows, ncols, pos, crd, val):
        self.nrows, self.ncols, self.pos, self.crd, self.val = nrows, ncols, pos, crd, val
        self.nnz = int(crd.shape[0])


def spgemm_symbolic(A, B, M=None, semiring=PLUS_TIMES):
    """Returns (handle, cpos tensor, nnz)."""
    _check_cuda(A.pos, A.crd, A.val, B.pos, B.crd, B.val)
    lib = _lib.load()
    cpos = torch.empty(A.nrows + 1, dtype=torch.int64, device=A.pos.device)
    nnz = ctypes.c_int64(0)
    handle = ctypes.c_int64(0)
    st = lib.comet_b200_dev_spgemm_symbolic_f64_i64(
        A.nrows, B.ncols, B.nnz, _p(A.pos), _p(A.crd), _p(A.val), _p(B.pos), _p(B.crd), _p(B.val),
        _p(M.pos if M is not None else None), _p(M.crd if M is not None else None), semiring, _p(cpos),
        ctypes.byref(nnz), ctypes.byref(handle), _stream())
    _lib.check(st)
    return handle.value, cpos, nnz.value


def spgemm_numeric(handle, nnz, device, keep=False, crd=None, val=None):
    lib = _lib.load()
    if crd is None:
        crd = torch.empty(max(nnz, 1), dtype=torch.int64, device=device)[:nnz]
        val = torch.empty(max(nnz, 1), dtype=torch.float64, device=device)[:nnz]
    st = lib.comet_b200_dev_spgemm_numeric_f64_i64(handle, _p(crd), _p(val), int(keep), _stream())
    _lib.check(st)
    return crd, val


def spgemm(A, B, M=None, semiring=PLUS_TIMES):
    handle, cpos, nnz = spgemm_symbolic(A, B, M, semiring)
    crd, val = spgemm_numeric(handle, nnz, A.pos.device)
    return SpgemmResult(A.nrows, B.ncols, cpos, crd, val)


def masked_pair_count(A, B, M, row_lo=0, row_hi=None, out=None):
    """Device int64 scalar tensor: products of rows [row_lo, row_hi) of A that land on M's pattern."""
    _check_cuda(A.pos, A.crd, B.pos, B.crd, M.pos, M.crd)
    row_hi = A.nrows if row_hi is None else row_hi
    if out is None:
        out = torch.zeros(1, dtype=torch.int64, device=A.pos.device)
    lib = _lib.load()
    st = lib.comet_b200_dev_masked_spgemm_count_f64_i64(
        row_lo, row_hi, B.ncols, A.nnz, B.nnz, M.nnz, _p(A.pos), _p(A.crd), _p(B.pos), _p(B.crd),
        _p(M.pos), _p(M.crd), _p(out), _stream())
    _lib.check(st)
    return out
