"""Operands that hold the same coordinate more than once.

COMET's MatrixMarket reader keeps repeated coordinates: it sorts the entries by
(row, col) with a stable sort and never sums them
(lib/ExecutionEngine/SparseUtils.cpp:360-367), so a CSR operand can carry equal
column indices at adjacent positions of a row.  The generated loops then treat
every stored position as its own entry: a repeated entry of A or B contributes
once per occurrence, a repeated entry of a push mask sets the same bit twice.
These tests feed such operands to every CUDA kernel of the path and compare
with the CPU oracle, which walks positions exactly like the generated loops."""
import numpy as np
import pytest
import torch

import comet_b200.api as api
import comet_b200.device as dev
from comet_b200 import datasets
from oracle import oracle

pytestmark = pytest.mark.gpu

RTOL = 1e-12


def _orc(t):
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, t.val)


def _abs(t):
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, np.abs(t.val))


def _close(got, ref, scale):
    got, ref, scale = np.asarray(got), np.asarray(ref), np.asarray(scale)
    assert got.shape == ref.shape
    bad = np.abs(got - ref) > RTOL * np.maximum(np.abs(ref), scale)
    assert not bad.any(), "%d entries beyond 1e-12" % int(bad.sum())


def dup_csr(nrows, ncols, lens, seed, spread=None, values="signed"):
    """CSR in reader order with repeated coordinates: every row draws its columns WITH replacement
    from a window of `spread` columns (narrow windows force many repeats) and is sorted ascending,
    equal columns adjacent, each with its own value."""
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, dtype=np.int64)
    pos = np.zeros(nrows + 1, dtype=np.int64)
    np.cumsum(lens, out=pos[1:])
    crd = np.empty(int(pos[-1]), dtype=np.int64)
    for r in range(nrows):
        n = int(lens[r])
        if n == 0:
            continue
        w = ncols if spread is None else max(1, min(ncols, spread if np.isscalar(spread) else int(spread[r])))
        lo = int(rng.integers(0, ncols - w + 1))
        crd[pos[r]:pos[r + 1]] = np.sort(lo + rng.integers(0, w, n), kind="stable")
    val = np.ones(crd.shape[0]) if values == "ones" else rng.uniform(-1, 1, crd.shape[0])
    return api.SparseTensor("CSR", nrows, ncols, np.array([nrows], dtype=np.int64), np.array([-1], dtype=np.int64),
                            pos, crd, val)


def _has_dups(A):
    same = A.a2crd[1:] == A.a2crd[:-1]
    row_of = np.searchsorted(A.a2pos, np.arange(A.nnz), side="right")
    return bool(np.any(same & (row_of[1:] == row_of[:-1])))


def _lens(n, seed, hubs=()):
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, 14, n)
    lens[rng.integers(0, n, n // 6)] = 0
    for r, l in hubs:
        lens[r] = l
    return lens


def test_spmv_with_repeated_coordinates():
    n = 4000
    A = dup_csr(n, n, _lens(n, 1, hubs=[(7, 3000), (n - 2, 600)]), seed=2, spread=40)
    assert _has_dups(A)
    x = datasets.dense_uniform(n, 3)
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), oracle.spmv(_abs(A), np.abs(x)))
    assert np.array_equal(api.spmv(A, x, semiring=api.PLUS_PAIR), np.diff(A.a2pos).astype(np.float64))


def test_spmv_chunk_list_path_with_repeated_coordinates():
    n = 1 << 16                                     # 2^20 stored entries: long rows go to the chunk list
    lens = np.full(n, 17)
    lens[[5, 999, n - 1]] = [9000, 70, 5000]
    lens[100:4000] = 14
    A = dup_csr(n, n, lens, seed=4, spread=64)
    assert A.nnz >= 1 << 20 and _has_dups(A)
    x = datasets.dense_uniform(n, 5)
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), oracle.spmv(_abs(A), np.abs(x)))


@pytest.mark.parametrize("variant", [1 << 24, 2 << 24, 3 << 24])     # entry stream, row panels, TMA-staged stream
@pytest.mark.parametrize("k", [128, 16])
def test_spmm_with_repeated_coordinates(variant, k):
    n = 3000
    A = dup_csr(n, n, _lens(n, 6, hubs=[(0, 2600), (1500, 900)]), seed=7, spread=50)
    assert _has_dups(A)
    B = datasets.dense_uniform((n, k), 8)
    C0 = datasets.dense_uniform((n, k), 9)
    scale = oracle.spmm(_abs(A), np.abs(B), np.abs(C0))
    dA, dB = dev.to_device(A), torch.from_numpy(B).cuda()
    _close(dev.spmm(dA, dB, variant=variant).cpu().numpy(), oracle.spmm(_orc(A), B), scale)
    C = dev.spmm(dA, dB, torch.from_numpy(C0).cuda(), accumulate=True, variant=variant)
    _close(C.cpu().numpy(), oracle.spmm(_orc(A), B, C0), scale)


def test_sddmm_with_repeated_coordinates():
    n, k = 2500, 64
    S = dup_csr(n, n, _lens(n, 10, hubs=[(3, 1800)]), seed=11, spread=30)
    X, Y = datasets.dense_uniform((n, k), 12), datasets.dense_uniform((n, k), 13)
    got = api.sddmm(S, X, Y)
    ref = oracle.sddmm(_orc(S), X, Y)
    _close(got, ref, oracle.sddmm(_abs(S), np.abs(X), np.abs(Y)))


def _check_spgemm(A, B, M=None, semiring=api.PLUS_TIMES):
    got = api.spgemm(A, B, M, semiring)
    ref = oracle.spgemm(_orc(A), _orc(B), _orc(M) if M is not None else None, semiring)
    assert np.array_equal(got.a2pos, ref.a2pos)
    assert np.array_equal(got.a2crd, ref.a2crd)
    if semiring == api.PLUS_PAIR:
        assert np.array_equal(got.val, ref.val)
    else:
        _close(got.val, ref.val, oracle.spgemm(_abs(A), _abs(B), _orc(M) if M is not None else None, semiring).val)
    return got


@pytest.mark.parametrize("semiring", [api.PLUS_TIMES, api.PLUS_PAIR])
def test_spgemm_hash_and_bitmap_bins_with_repeated_coordinates(semiring):
    """Short rows take the shared-memory hash, rows whose bound exceeds 256 distinct columns the bitmap;
    both operands repeat coordinates, so a product's column can recur inside one B row and one B row
    can be named twice by a row of A."""
    n = 3000
    A = dup_csr(n, n, _lens(n, 20, hubs=[(1, 700), (2, 1400), (n - 1, 300)]), seed=21, spread=60)
    B = dup_csr(n, n, _lens(n, 22, hubs=[(10, 1200), (11, 1200)]), seed=23, spread=200)
    assert _has_dups(A) and _has_dups(B)
    C = _check_spgemm(A, B, semiring=semiring)
    assert C.nnz > 0 and not _has_dups(C)            # output coordinates are distinct per row


@pytest.mark.parametrize("semiring", [api.PLUS_TIMES, api.PLUS_PAIR])
def test_masked_spgemm_with_repeated_mask_coordinates(semiring):
    n = 2000
    A = dup_csr(n, n, _lens(n, 30, hubs=[(4, 900)]), seed=31, spread=80)
    B = dup_csr(n, n, _lens(n, 32, hubs=[(40, 1500)]), seed=33, spread=300)
    M = dup_csr(n, n, _lens(n, 34, hubs=[(4, 1000), (5, 400)]), seed=35, spread=500)
    assert _has_dups(M)
    C = _check_spgemm(A, B, M, semiring)
    assert not _has_dups(C)


def test_masked_count_with_repeated_coordinates_in_every_operand():
    n = 2500
    A = dup_csr(n, n, _lens(n, 40, hubs=[(8, 2300), (9, 150)]), seed=41, spread=90, values="ones")
    B = dup_csr(n, n, _lens(n, 42, hubs=[(60, 800)]), seed=43, spread=400, values="ones")
    # warp bin (<= 128 mask entries), CTA bin (<= 2048) and the long bin, all with repeats
    M = dup_csr(n, n, _lens(n, 44, hubs=[(8, 5000), (9, 1500), (70, 120)]), seed=45, spread=700, values="ones")
    assert _has_dups(A) and _has_dups(B) and _has_dups(M)
    want = oracle.masked_pair_count(_orc(A), _orc(B), _orc(M))
    assert want > 0
    assert api.masked_pair_count(A, B, M) == want


@pytest.mark.parametrize("a_len", [100, 5000])       # one slice of A's row, several slices
def test_masked_count_mask_segment_boundary_between_two_copies(a_len):
    """A mask row longer than one 4096-entry segment whose entries 4095 and 4096 (and again 8191 and
    8192) are the same coordinate: the two copies fall into different segments of the counting kernel
    and must still count as one mask bit."""
    n = 12000
    mrow = np.sort(np.random.default_rng(50).choice(n, 9000, replace=False))
    mrow = np.concatenate([mrow[:4096], mrow[4095:8191], mrow[8190:]])        # positions 4095|4096 and 8191|8192
    assert mrow[4095] == mrow[4096] and mrow[8191] == mrow[8192] and np.all(np.diff(mrow) >= 0)
    row = 17
    mlens = np.zeros(n, dtype=np.int64)
    mlens[row] = mrow.shape[0]
    M = dup_csr(n, n, mlens, seed=51, values="ones")
    M.a2crd[:] = mrow
    alens = np.zeros(n, dtype=np.int64)
    alens[row] = a_len
    A = dup_csr(n, n, alens, seed=52, values="ones")
    # every row of B that A names holds the two boundary coordinates, so a double count would show
    blens = np.full(n, 6)
    B = dup_csr(n, n, blens, seed=53, values="ones")
    for k in np.unique(A.a2crd):
        s = B.a2pos[k]
        B.a2crd[s:s + 6] = np.sort(np.array([mrow[4095], mrow[8191], mrow[0], mrow[-1], mrow[100], mrow[5000]]))
    want = oracle.masked_pair_count(_orc(A), _orc(B), _orc(M))
    assert want == 6 * a_len
    assert api.masked_pair_count(A, B, M) == want
    # the same through the device entry point over a row range that holds the row
    dA, dB, dM = dev.to_device(A), dev.to_device(B), dev.to_device(M)
    assert int(dev.masked_pair_count(dA, dB, dM, 10, 30).item()) == want


# ---------------------------------------------------------------------------
# A coordinate outside the matrix is refused before any kernel gathers through it.  The only bad value
# used here is crd == ncols (one past the end), never anything further out.
# ---------------------------------------------------------------------------
def _one_past_the_end(A):
    bad = api.SparseTensor(A.format, A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd.copy(), A.val)
    bad.a2crd[A.nnz // 2] = A.ncols
    return bad


def test_coordinate_one_past_the_end_is_refused_by_every_host_entry_point():
    from comet_b200 import _lib
    k = 8
    A = datasets.rmat_csr(9, 8, seed=3)
    n = A.nrows
    bad = _one_past_the_end(A)
    x = datasets.dense_uniform(n, 1)
    B = datasets.dense_uniform((n, k), 2)
    calls = [
        lambda: api.spmv(bad, x),
        lambda: api.spmm(bad, B),
        lambda: api.sddmm(bad, B, B),
        lambda: api.spgemm(bad, A),
        lambda: api.spgemm(A, bad),
        lambda: api.spgemm(A, A, bad, api.PLUS_PAIR),
        lambda: api.masked_pair_count(bad, A, A),
        lambda: api.masked_pair_count(A, A, bad),
        lambda: api.elews_sparse_dense(bad, np.ones((n, n))),
    ]
    for call in calls:
        with pytest.raises(_lib.CometB200Error, match="outside the"):
            call()
    # the library is still usable afterwards
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), oracle.spmv(_abs(A), np.abs(x)))
