"""The allocation-free SpMM entry point (comet_b200_dev_spmm_noalloc_f64_i64).

It serves callers that cannot allocate device memory inside an operation (a
fixed memory budget, a loop that must never stall on the allocator, a runtime
that owns the heap): its long-row work list sits in a fixed array inside the
library instead of growable scratch.  The test calls it through the C ABI twice
in a row -- each later call meets the list the one before left behind -- and
compares each result with the CPU oracle and with the regular entry point on
the same device arrays.
This file sorts last so that a run stopping at the first failure has already
run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-12


def _inputs():
    import scipy.sparse as sp
    rng = np.random.default_rng(42)
    n = 4000
    lens = rng.integers(0, 10, n)
    lens[[0, 17, n - 1]] = [3000, 1500, 700]        # rows that go through the work list
    rows = np.repeat(np.arange(n), lens)
    cols = np.concatenate([np.sort(rng.choice(n, l, replace=False)) for l in lens])
    vals = rng.uniform(-1, 1, rows.shape[0])
    m = sp.csr_matrix((vals, (rows, cols)), shape=(n, n))
    m.sort_indices()
    return m, [rng.uniform(-1, 1, (n, k)) for k in (128, 64, 256)]


def _oracle_spmm(m, B, C0=None, semiring=0):
    """The CPU restatement of COMET's loop nest (the checker every other parity test uses)."""
    from comet_b200 import api
    from oracle import oracle
    t = api.as_sparse(m)
    A = oracle.SparseArrays("CSR", t.nrows, t.ncols, t.a1pos.astype(np.int64), t.a1crd.astype(np.int64),
                            t.a2pos.astype(np.int64), t.a2crd.astype(np.int64), t.val)
    return oracle.spmm(A, B, C0, semiring=semiring)


def _within(got, ref, scale):
    err = np.abs(got - ref)
    bound = RTOL * np.maximum(np.abs(ref), scale)
    return bool((err <= bound).all())


def test_noalloc_spmm_matches_regular_entry_point_twice():
    import torch
    from comet_b200 import _lib, device as dev

    lib = _lib.load()
    m, Bs = _inputs()
    A = dev.to_device(m)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(dB, out, semiring=0, accumulate=0):
        st = lib.comet_b200_dev_spmm_noalloc_f64_i64(A.nrows, A.nnz, dB.shape[1], None, p(A.pos), p(A.crd), p(A.val),
                                                     p(dB), dB.stride(0), p(out), out.stride(0), semiring,
                                                     accumulate, stream)
        _lib.check(st)
        torch.cuda.synchronize()
        return out.cpu().numpy()

    for B in Bs:                                      # calls in a row share the built-in list
        dB = torch.from_numpy(B).cuda()
        k = B.shape[1]
        ref = _oracle_spmm(m, B)                      # CPU oracle: an independent implementation
        scale = _oracle_spmm(abs(m), np.abs(B))       # sum of |terms| bounds the reordering error
        got = call(dB, torch.full((A.nrows, k), float("nan"), dtype=torch.float64, device="cuda"))
        assert _within(got, ref, scale)
        # ... and the regular entry point on the same device arrays gives the same result
        assert _within(got, dev.spmm(A, dB).cpu().numpy(), scale)
        # accumulate into existing values as well
        base = np.random.default_rng(1).uniform(-1, 1, (A.nrows, k))
        got2 = call(dB, torch.from_numpy(base).cuda(), accumulate=1)
        assert _within(got2, _oracle_spmm(m, B, base), scale + np.abs(base))
    # plus-pair: every column of row i holds the number of entries row i stores (exact)
    dB = torch.from_numpy(Bs[0]).cuda()
    got = call(dB, torch.empty((A.nrows, 128), dtype=torch.float64, device="cuda"), semiring=1)
    assert np.array_equal(got, _oracle_spmm(m, Bs[0], semiring=1))
    assert np.array_equal(got[:, 0], np.diff(m.indptr).astype(np.float64))


def test_noalloc_spmm_refuses_sizes_beyond_its_list():
    import torch
    from comet_b200 import _lib, device as dev

    lib = _lib.load()
    m, Bs = _inputs()
    A = dev.to_device(m)
    dB = torch.from_numpy(Bs[0]).cuda()
    C = torch.zeros((A.nrows, 128), dtype=torch.float64, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the size check comes before any launch, so a claimed nnz beyond the limit is refused untouched
    st = lib.comet_b200_dev_spmm_noalloc_f64_i64(A.nrows, 10 ** 9, 128, None, p(A.pos), p(A.crd), p(A.val),
                                                 p(dB), dB.stride(0), p(C), C.stride(0), 0, 0, stream)
    assert st != 0
    with pytest.raises(_lib.CometB200Error, match="built-in list holds"):
        _lib.check(st)
    # odd K is outside what the allocation-free variant takes
    st = lib.comet_b200_dev_spmm_noalloc_f64_i64(A.nrows, A.nnz, 127, None, p(A.pos), p(A.crd), p(A.val),
                                                 p(dB), dB.stride(0), p(C), C.stride(0), 0, 0, stream)
    assert st != 0
    torch.cuda.synchronize()
    assert float(C.abs().sum()) == 0.0
