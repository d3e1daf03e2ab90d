"""Parity of the CUDA path with the CPU oracle on seeded inputs: structure
(pos, crd) and integer results bit-exact, float64 values within 1e-12 relative
(the tolerance the path is specified to; differences come from summation order).

For sums of signed terms the error of any summation order is bounded by
eps * n * sum(|terms|), so values are compared relative to max(|ref|, sum(|terms|)):
an entry that cancels to nearly zero is not held to 1e-12 of its tiny result."""
import numpy as np
import pytest
import scipy.sparse as sp
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
    err = np.abs(got - ref)
    bound = RTOL * np.maximum(np.abs(ref), scale)
    bad = err > bound
    assert not bad.any(), "max rel err %.3e at %d entries" % (float((err / np.maximum(bound, 1e-300)).max() * RTOL), int(bad.sum()))


def _skewed(n=3000, seed=0):
    """CSR with empty rows, short rows, and a few rows far longer than any lane group or chunk."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, 12, n)
    lens[rng.integers(0, n, n // 5)] = 0
    lens[[1, n // 2, n - 1]] = [min(2500, n - 7), min(700, n // 2), min(1301, n // 3)]
    rows = np.repeat(np.arange(n), lens)
    cols = np.concatenate([np.sort(rng.choice(n, l, replace=False)) for l in lens])
    vals = rng.uniform(-1, 1, rows.shape[0])
    m = sp.csr_matrix((vals, (rows, cols)), shape=(n, n))
    m.sort_indices()
    return api.as_sparse(m)


@pytest.mark.parametrize("make", [lambda: datasets.config_spmv(n=2048, per_row=16)[0],
                                  lambda: datasets.rmat_csr(12, 16, seed=2), _skewed])
def test_spmv_parity(make):
    A = make()
    x = datasets.dense_uniform(A.ncols, 11)
    y0 = datasets.dense_uniform(A.nrows, 12)
    ref = oracle.spmv(_orc(A), x, y0)
    scale = oracle.spmv(_abs(A), np.abs(x), np.abs(y0))
    _close(api.spmv(A, x, y0), ref, scale)
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), scale)
    # plus-pair: exact small integers
    assert np.array_equal(api.spmv(A, x, semiring=api.PLUS_PAIR), oracle.spmv(_orc(A), x, semiring=oracle.PLUS_PAIR))


@pytest.mark.parametrize("k", [128, 64, 32, 6, 5, 1])
def test_spmm_parity(k):
    A = _skewed(2000, seed=k)
    B = datasets.dense_uniform((A.ncols, k), 3)
    C0 = datasets.dense_uniform((A.nrows, k), 4)
    ref = oracle.spmm(_orc(A), B, C0)
    scale = oracle.spmm(_abs(A), np.abs(B), np.abs(C0))
    _close(api.spmm(A, B, C0), ref, scale)
    _close(api.spmm(A, B), oracle.spmm(_orc(A), B), scale)


def test_spmm_rmat_and_panel_variants():
    A, B = datasets.config_spmm(scale=13, edge_factor=16, k=128)
    ref = oracle.spmm(_orc(A), B)
    scale = oracle.spmm(_abs(A), np.abs(B))
    dA = dev.to_device(A)
    dB = torch.from_numpy(B).cuda()
    for variant in (0, 64, 32, 16, 32 | (8 << 16), 128 | (16 << 16)):
        C = dev.spmm(dA, dB, variant=variant)
        _close(C.cpu().numpy(), ref, scale)
    # plus-pair counts entries per row in every column
    Cp = dev.spmm(dA, dB, semiring=api.PLUS_PAIR).cpu().numpy()
    assert np.array_equal(Cp, np.repeat(np.diff(A.a2pos)[:, None], 128, axis=1).astype(np.float64))


def _gappy(n=6000, seed=5):
    """Leading, trailing and long runs of empty rows, single-entry rows and one row far longer than a block."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(0, 5, n)
    lens[:70] = 0
    lens[-130:] = 0
    lens[2000:3400] = 0
    lens[rng.integers(0, n, n // 2)] = 0
    lens[1234] = 4000
    rows = np.repeat(np.arange(n), lens)
    cols = rng.integers(0, n, rows.shape[0])
    m = sp.csr_matrix((rng.uniform(-1, 1, rows.shape[0]), (rows, cols)), shape=(n, n))
    m.sum_duplicates()
    m.sort_indices()
    return api.as_sparse(m)


@pytest.mark.parametrize("k", [128, 64, 96, 16, 2, 256])
@pytest.mark.parametrize("make", [_gappy, _skewed])
@pytest.mark.parametrize("family", [1, 3, 7])
def test_spmm_entry_stream_path(make, k, family):
    """The entry-stream kernels (asked for by bits 24-26 of the variant: 1 = rows of B staged with cp.async,
    the default from 64 columns on; 3 = staged by TMA bulk copies completing on mbarriers; 7 = staged by one
    tile::gather4 tensor copy per four rows): rows cut by block boundaries, empty rows at every position, both
    store modes."""
    A = make()
    B = datasets.dense_uniform((A.ncols, k), 3)
    C0 = datasets.dense_uniform((A.nrows, k), 4)
    scale = oracle.spmm(_abs(A), np.abs(B), np.abs(C0))
    dA = dev.to_device(A)
    dB = torch.from_numpy(B).cuda()
    C = dev.spmm(dA, dB, variant=family << 24)
    _close(C.cpu().numpy(), oracle.spmm(_orc(A), B), scale)
    C = dev.spmm(dA, dB, torch.from_numpy(C0).cuda(), accumulate=True, variant=family << 24)
    _close(C.cpu().numpy(), oracle.spmm(_orc(A), B, C0), scale)


@pytest.mark.parametrize("family", [3, 7])
def test_spmm_tma_staging_on_a_power_law_matrix(family):
    A, B = datasets.config_spmm(scale=14, edge_factor=16, k=128)
    dA, dB = dev.to_device(A), torch.from_numpy(B).cuda()
    C = dev.spmm(dA, dB, variant=family << 24)
    _close(C.cpu().numpy(), oracle.spmm(_orc(A), B), oracle.spmm(_abs(A), np.abs(B)))


def test_spmm_gather4_staging_with_a_padded_leading_dimension():
    """B is a view of a wider array: the tensor map's row stride is the leading dimension, not K."""
    A = _skewed(3000, seed=12)
    wide = datasets.dense_uniform((A.ncols, 80), 5)
    dwide = torch.from_numpy(wide).cuda()
    C = dev.spmm(dev.to_device(A), dwide[:, :64], variant=7 << 24)
    B = np.ascontiguousarray(wide[:, :64])
    _close(C.cpu().numpy(), oracle.spmm(_orc(A), B), oracle.spmm(_abs(A), np.abs(B)))


def test_spmm_entry_stream_path_dcsr(tmp_path):
    A = _gappy(seed=6)
    path = tmp_path / "a.mtx"
    datasets.write_mtx(str(path), A)
    D = oracle.read_mtx(str(path), "DCSR")
    B = datasets.dense_uniform((D.ncols, 64), 3)
    C = dev.spmm(dev.to_device(D), torch.from_numpy(B).cuda(), variant=1 << 24)
    _close(C.cpu().numpy(), oracle.spmm(D, B), oracle.spmm(_abs(D), np.abs(B)))


@pytest.mark.parametrize("fmt", ["DCSR", "COO"])
def test_dcsr_and_coo_operands(fmt, tmp_path):
    A = _skewed(500, seed=9)
    path = tmp_path / "a.mtx"
    datasets.write_mtx(str(path), A)
    T = oracle.read_mtx(str(path), fmt)
    x = datasets.dense_uniform(A.ncols, 1)
    B = datasets.dense_uniform((A.ncols, 8), 2)
    y0 = datasets.dense_uniform(A.nrows, 5)
    _close(api.spmv(T, x, y0), oracle.spmv(T, x, y0), oracle.spmv(_abs(T), np.abs(x), np.abs(y0)))
    _close(api.spmm(T, B), oracle.spmm(T, B), oracle.spmm(_abs(T), np.abs(B)))


def test_unsorted_coo_is_rejected():
    from comet_b200._lib import CometB200Error
    m = sp.coo_matrix((np.ones(3), (np.array([2, 0, 1]), np.array([0, 1, 2]))), shape=(3, 3))
    with pytest.raises(CometB200Error, match="ascending"):
        api.spmv(m, np.ones(3))


@pytest.mark.parametrize("k", [64, 128, 16, 10, 7])
def test_sddmm_parity(k):
    S = _skewed(1500, seed=k)
    X = datasets.dense_uniform((S.nrows, k), 1)
    Y = datasets.dense_uniform((S.ncols, k), 2)
    ref = oracle.sddmm(_orc(S), X, Y)
    scale = oracle.sddmm(_abs(S), np.abs(X), np.abs(Y))
    _close(api.sddmm(S, X, Y), ref, scale)
    # the D[k, j] operand layout of the reference's sddmm.ta
    _close(api.sddmm(S, X, np.ascontiguousarray(Y.T), y_is_kj=True), ref, scale)


def test_sddmm_rmat():
    S, X, Y = datasets.config_sddmm(scale=12, edge_factor=32, k=64)
    _close(api.sddmm(S, X, Y), oracle.sddmm(_orc(S), X, Y), oracle.sddmm(_abs(S), np.abs(X), np.abs(Y)))


def test_elementwise():
    A = _skewed(800, seed=4)
    B = datasets.dense_uniform((A.nrows, A.ncols), 6)
    assert np.array_equal(api.elews_sparse_dense(A, B), oracle.elews_sparse_dense(_orc(A), B))
    A2 = _skewed(800, seed=5)
    got, ref = api.elews_csr_csr(A, A2), oracle.elews_csr_csr(_orc(A), _orc(A2))
    assert np.array_equal(got.a2pos, ref.a2pos) and np.array_equal(got.a2crd, ref.a2crd)
    assert np.array_equal(got.val, ref.val)


def _check_spgemm(A, B, M=None, semiring=api.PLUS_TIMES):
    got = api.spgemm(A, B, M, semiring)
    ref = oracle.spgemm(_orc(A), _orc(B), _orc(M) if M is not None else None, semiring)
    assert np.array_equal(got.a2pos, ref.a2pos)
    assert np.array_equal(got.a2crd, ref.a2crd)
    if semiring == api.PLUS_PAIR:
        assert np.array_equal(got.val, ref.val)
    else:
        scale = oracle.spgemm(_abs(A), _abs(B), _orc(M) if M is not None else None, semiring).val
        _close(got.val, ref.val, scale)
    return got


@pytest.mark.parametrize("scale,ef", [(8, 4), (11, 8), (13, 16)])
def test_spgemm_rmat_parity(scale, ef):
    A = datasets.config_spgemm(scale=scale, edge_factor=ef)
    C = _check_spgemm(A, A)
    assert C.nnz > 0
    _check_spgemm(A, A, semiring=api.PLUS_PAIR)


def test_spgemm_rectangular_empty_and_long_rows():
    rng = np.random.default_rng(0)
    A = sp.random(300, 5000, density=0.02, random_state=rng, format="csr")
    B = sp.random(5000, 70000, density=0.002, random_state=rng, format="csr")   # rows of C far beyond the hash bin
    A.sort_indices(); B.sort_indices()
    A, B = api.as_sparse(A), api.as_sparse(B)
    A.val[:] = rng.uniform(-1, 1, A.nnz)
    _check_spgemm(A, B)
    Z = api.as_sparse(sp.csr_matrix((300, 5000)))
    got = api.spgemm(Z, B)
    assert got.nnz == 0 and np.all(got.a2pos == 0)


@pytest.mark.parametrize("semiring", [api.PLUS_TIMES, api.MIN_PLUS])
def test_spgemm_teams_and_long_rows_of_b(monkeypatch, semiring):
    """Rows whose output is large are accumulated by a team of CTAs (forced here by a tiny budget), and
    rows of B above 1024 entries are walked by the whole CTA: row 1500 of A names 1200 such rows, more
    than the per-CTA list of long rows holds, so the rescan path runs too."""
    rng = np.random.default_rng(3)
    n, nlong, width = 4096, 1200, 1030
    rows, cols = [], []
    for i in range(nlong):                               # long rows, pointing at short ones
        rows.append(np.full(width, i)); cols.append(nlong + np.sort(rng.choice(n - nlong, width, replace=False)))
    for i in range(nlong, n):
        c = np.arange(nlong) if i == 1500 else np.sort(rng.choice(n, 3, replace=False))
        rows.append(np.full(c.shape[0], i)); cols.append(c)
    rows, cols = np.concatenate(rows), np.concatenate(cols)
    m = sp.csr_matrix((rng.uniform(-1, 1, rows.shape[0]), (rows, cols)), shape=(n, n))
    m.sort_indices()
    A = api.as_sparse(m)
    for budget in ("0.01", "60"):
        monkeypatch.setenv("COMET_B200_SPGEMM_TEAM_MB", budget)
        _check_spgemm(A, A, semiring=semiring)
    R = datasets.rmat_csr(12, 16, seed=4)
    monkeypatch.setenv("COMET_B200_SPGEMM_TEAM_MB", "0.01")
    _check_spgemm(R, R, semiring=semiring)
    _check_spgemm(R, R, datasets.rmat_csr(12, 32, seed=5), semiring)


def test_spgemm_many_columns_uses_global_bitmaps():
    rng = np.random.default_rng(1)
    n = 1_200_000                                    # bitmap + ranks no longer fit shared memory
    A = sp.random(64, 2000, density=0.2, random_state=rng, format="csr")
    B = sp.random(2000, n, density=2e-4, random_state=rng, format="csr")
    A.sort_indices(); B.sort_indices()
    _check_spgemm(api.as_sparse(A), api.as_sparse(B))


@pytest.mark.parametrize("scale", [9, 12])
def test_masked_spgemm_and_triangle_count(scale):
    L = datasets.config_triangles(scale=scale, edge_factor=8)
    C = _check_spgemm(L, L, L, api.PLUS_PAIR)
    want = oracle.masked_pair_count(_orc(L), _orc(L), _orc(L))
    assert int(round(api.reduce_sum(C.val))) == want
    assert api.triangle_count(L) == want
    # cross-check with scipy on the smaller case
    if scale == 9:
        m = L.to_scipy()
        assert want == int((m @ m).multiply(m).sum())
    # masked plus-times, mask different from the operands
    A = datasets.rmat_csr(scale, 8, seed=5)
    M = datasets.rmat_csr(scale, 16, seed=6)
    _check_spgemm(A, A, M)
    assert api.masked_pair_count(A, A, M) == oracle.masked_pair_count(_orc(A), _orc(A), _orc(M))


def test_device_layer_row_ranges_and_repeat_calls():
    L = datasets.config_triangles(scale=11, edge_factor=8)
    dL = dev.to_device(L)
    ol = _orc(L)
    half = L.nrows // 3
    a = int(dev.masked_pair_count(dL, dL, dL, 0, half).item())
    b = int(dev.masked_pair_count(dL, dL, dL, half, L.nrows).item())
    assert a == oracle.masked_pair_count(ol, ol, ol, 0, half)
    assert a + b == oracle.masked_pair_count(ol, ol, ol)
    # numeric phase repeated on a kept handle gives the same structure
    A = datasets.config_spgemm(scale=10, edge_factor=8)
    dA = dev.to_device(A)
    h, cpos, nnz = dev.spgemm_symbolic(dA, dA)
    crd1, val1 = dev.spgemm_numeric(h, nnz, "cuda", keep=True)
    crd2, val2 = dev.spgemm_numeric(h, nnz, "cuda", keep=False)
    assert torch.equal(crd1, crd2)
    ref = oracle.spgemm(_orc(A), _orc(A))
    assert np.array_equal(cpos.cpu().numpy(), ref.a2pos) and np.array_equal(crd1.cpu().numpy(), ref.a2crd)
    _close(val2.cpu().numpy(), ref.val, ref.val)


def test_einsum_surface_matches_cometpy_forms():
    A = datasets.rmat_csr(9, 8, seed=1).to_scipy()
    x = datasets.dense_uniform(A.shape[1], 2)
    B = datasets.dense_uniform((A.shape[1], 4), 3)
    np.testing.assert_allclose(api.einsum("ij,j->i", A, x), A @ x, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(api.einsum("ij,jk->ik", A, B), A @ B, rtol=1e-12, atol=1e-13)
    C = api.einsum("ij,jk->ik", A, A, mask=A, mask_type="push", semiring="+,pair")
    want = (A.astype(bool).astype(float) @ A.astype(bool).astype(float)).multiply(A.astype(bool)).tocsr()
    want.sort_indices(); want.eliminate_zeros()
    got = C.to_scipy(); got.eliminate_zeros()
    assert (abs(got - want)).nnz == 0


def test_int32_index_entry_points_match_int64():
    """scipy's default int32 index arrays go through the _f64_i32 symbols (indices widened on the
    device) and give the same results, with int32 structure arrays coming back."""
    A64 = datasets.rmat_csr(11, 8, seed=7)
    A32 = A64.with_index_dtype(np.int32)
    assert A32.index_dtype == np.int32
    x = datasets.dense_uniform(A64.ncols, 1)
    B = datasets.dense_uniform((A64.ncols, 16), 2)
    assert np.array_equal(api.spmv(A32, x), api.spmv(A64, x))
    np.testing.assert_allclose(api.spmm(A32, B), api.spmm(A64, B), rtol=1e-13, atol=1e-13)
    X = datasets.dense_uniform((A64.nrows, 8), 3)
    Y = datasets.dense_uniform((A64.ncols, 8), 4)
    assert np.array_equal(api.sddmm(A32, X, Y), api.sddmm(A64, X, Y))
    D = datasets.dense_uniform((A64.nrows, A64.ncols), 5)
    assert np.array_equal(api.elews_sparse_dense(A32, D), api.elews_sparse_dense(A64, D))
    C32, C64 = api.spgemm(A32, A32), api.spgemm(A64, A64)
    assert C32.a2pos.dtype == np.int32 and C32.a2crd.dtype == np.int32
    assert np.array_equal(C32.a2pos, C64.a2pos) and np.array_equal(C32.a2crd, C64.a2crd)
    np.testing.assert_allclose(C32.val, C64.val, rtol=1e-13)
    M32 = api.spgemm(A32, A32, A32, api.PLUS_PAIR)
    ref = oracle.spgemm(_orc(A64), _orc(A64), _orc(A64), oracle.PLUS_PAIR)
    assert np.array_equal(M32.a2pos, ref.a2pos) and np.array_equal(M32.a2crd, ref.a2crd)
    E32 = api.elews_csr_csr(A32, A32)
    assert E32.a2crd.dtype == np.int32 and np.array_equal(E32.a2crd, A64.a2crd)
    L = datasets.config_triangles(scale=10, edge_factor=8)
    assert api.triangle_count(L.with_index_dtype(np.int32)) == api.triangle_count(L)
    # mixed widths are promoted to int64
    assert api.spgemm(A32, A64).a2crd.dtype == np.int64
    # COO and DCSR operands with int32 indices
    import scipy.sparse as sp
    coo = A64.to_scipy().tocoo()
    assert coo.row.dtype == np.int32
    np.testing.assert_allclose(api.spmv(coo, x), api.spmv(A64, x), rtol=1e-13, atol=1e-13)


def test_empty_and_degenerate_inputs():
    """Zero rows, zero stored entries, all-empty rows, a single entry: nothing is launched out of
    bounds and outputs follow the accumulate semantics."""
    import scipy.sparse as sp
    Z = api.as_sparse(sp.csr_matrix((50, 40)))                     # no stored entries
    x = np.ones(40)
    assert np.array_equal(api.spmv(Z, x), np.zeros(50))
    y0 = np.arange(50, dtype=np.float64)
    assert np.array_equal(api.spmv(Z, x, y0), y0)                  # accumulate keeps the old values
    assert np.array_equal(api.spmm(Z, np.ones((40, 6))), np.zeros((50, 6)))
    assert api.sddmm(Z, np.ones((50, 4)), np.ones((40, 4))).shape == (0,)
    assert api.spgemm(Z, api.as_sparse(sp.csr_matrix((40, 30)))).nnz == 0
    assert api.masked_pair_count(Z, api.as_sparse(sp.csr_matrix((40, 40))), Z) == 0
    E = api.as_sparse(sp.csr_matrix((0, 7)))                       # no rows at all
    assert api.spmv(E, np.ones(7)).shape == (0,)
    one = api.as_sparse(sp.csr_matrix(([2.5], ([3], [1])), shape=(5, 4)))
    assert np.array_equal(api.spmv(one, np.array([1.0, 2.0, 3.0, 4.0])), [0, 0, 0, 5.0, 0])
    C = api.spgemm(one, api.as_sparse(sp.csr_matrix(([4.0], ([1], [2])), shape=(4, 6))))
    assert C.nnz == 1 and C.a2crd[0] == 2 and C.val[0] == 10.0 and list(C.a2pos) == [0, 0, 0, 0, 1, 1]


def test_handles_are_single_use_and_checked():
    from comet_b200._lib import CometB200Error
    A = datasets.rmat_csr(8, 4, seed=2)
    dA = dev.to_device(A)
    h, cpos, nnz = dev.spgemm_symbolic(dA, dA)
    dev.spgemm_numeric(h, nnz, "cuda")
    with pytest.raises(CometB200Error, match="unknown handle"):
        dev.spgemm_numeric(h, nnz, "cuda")                          # released by the first numeric call
    h2, _, _ = dev.spgemm_symbolic(dA, dA)
    from comet_b200 import _lib
    _lib.load().comet_b200_handle_destroy(h2)                       # dropping without numeric is allowed
    with pytest.raises(CometB200Error, match="unknown handle"):
        dev.spgemm_numeric(h2, nnz, "cuda")


def test_unaligned_device_arrays_take_the_scalar_paths():
    """Views that start 8 bytes into an allocation break the 16-byte alignment the vector loads want;
    SpMV and SpMM fall back to scalar loads, operations that cannot say so."""
    from comet_b200._lib import CometB200Error
    A = datasets.rmat_csr(9, 8, seed=4)
    x = datasets.dense_uniform(A.ncols, 1)
    pad = lambda a: torch.from_numpy(np.concatenate([np.zeros(1, dtype=a.dtype), a])).cuda()[1:]
    dA = dev.DeviceCSR(A.nrows, A.ncols, torch.from_numpy(A.a2pos).cuda(), pad(A.a2crd), pad(A.val))
    assert dA.crd.data_ptr() % 16 == 8
    want = oracle.spmv(_orc(A), x)
    np.testing.assert_allclose(dev.spmv(dA, torch.from_numpy(x).cuda()).cpu().numpy(), want, rtol=1e-12, atol=1e-13)
    B = datasets.dense_uniform((A.ncols, 8), 2)
    np.testing.assert_allclose(dev.spmm(dA, torch.from_numpy(B).cuda()).cpu().numpy(), oracle.spmm(_orc(A), B),
                               rtol=1e-12, atol=1e-13)
    with pytest.raises(CometB200Error, match="aligned"):
        dev.spgemm_symbolic(dA, dA)


def test_spmm_host_entry_point_panel_pipeline(monkeypatch):
    """Large SpMM calls through the host entry point are cut into column panels so that the upload of
    B, the multiplication and the download of C overlap; force that path on a small input, with a
    dense width that is not a multiple of the panel."""
    A = _skewed(1200, seed=11)
    for k, panel in ((10, 4), (64, 32), (6, 2)):
        B = datasets.dense_uniform((A.ncols, k), k)
        ref = oracle.spmm(_orc(A), B)
        scale = oracle.spmm(_abs(A), np.abs(B))
        monkeypatch.setenv("COMET_B200_SPMM_PANEL", str(panel))
        monkeypatch.setenv("COMET_B200_SPMM_PANEL_MIN_BYTES", "0")
        got = api.spmm(A, B)
        monkeypatch.delenv("COMET_B200_SPMM_PANEL")
        monkeypatch.delenv("COMET_B200_SPMM_PANEL_MIN_BYTES")
        _close(got, ref, scale)
        # strided (non-contiguous) host operands: a column window of wider matrices
        wide = datasets.dense_uniform((A.ncols, k + 6), 99)
        monkeypatch.setenv("COMET_B200_SPMM_PANEL", str(panel))
        monkeypatch.setenv("COMET_B200_SPMM_PANEL_MIN_BYTES", "0")
        lib_b = wide[:, 3:3 + k]
        pk = api._Packer()
        out = np.full((A.nrows, k + 4), -7.0)
        from comet_b200 import _lib
        lib = _lib.load()
        fn, _, (A_,) = api._entry(lib, "spmm", api.as_sparse(A))      # entry point of A's index width
        fn(*pk.sparse(A_), *pk.m2(lib_b), *pk.m2(out[:, 2:2 + k]), 0, 0)
        _lib.check()
        monkeypatch.delenv("COMET_B200_SPMM_PANEL")
        monkeypatch.delenv("COMET_B200_SPMM_PANEL_MIN_BYTES")
        _close(out[:, 2:2 + k], oracle.spmm(_orc(A), np.ascontiguousarray(lib_b)),
               oracle.spmm(_abs(A), np.abs(np.ascontiguousarray(lib_b))))
        assert np.all(out[:, :2] == -7.0) and np.all(out[:, 2 + k:] == -7.0)      # padding untouched


def test_spmv_large_power_law_uses_the_chunk_list():
    """Above 2^20 stored entries long rows are cut into chunks handled by a second launch."""
    A = datasets.rmat_csr(17, 16, seed=3)
    assert A.nnz > (1 << 20) and np.diff(A.a2pos).max() > 2048
    x = datasets.dense_uniform(A.ncols, 1)
    y0 = datasets.dense_uniform(A.nrows, 2)
    scale = oracle.spmv(_abs(A), np.abs(x), np.abs(y0))
    _close(api.spmv(A, x), oracle.spmv(_orc(A), x), scale)
    _close(api.spmv(A, x, y0), oracle.spmv(_orc(A), x, y0), scale)
    assert np.array_equal(api.spmv(A, x, semiring=api.PLUS_PAIR), np.diff(A.a2pos).astype(np.float64))


@pytest.mark.parametrize("semiring", ["+,first", "+,second", "min,+", "min,first", "min,second", "any,pair"])
def test_spgemm_further_semirings(semiring):
    """The other semirings COMET tests on CSR x CSR: structure identical, min / any results exact,
    plus results within tolerance; rows short enough for the hash path and long enough for the bitmap path."""
    code = api._semiring(semiring)
    A = datasets.rmat_csr(11, 8, seed=21)
    A.val[:] = datasets.dense_uniform(A.nnz, 22, -2.0, 3.0)
    got = api.spgemm(A, A, None, semiring)
    ref = oracle.spgemm(_orc(A), _orc(A), None, code)
    assert np.array_equal(got.a2pos, ref.a2pos) and np.array_equal(got.a2crd, ref.a2crd)
    if semiring.startswith("+"):
        _close(got.val, ref.val, oracle.spgemm(_abs(A), _abs(A), None, code).val)
    else:
        assert np.array_equal(got.val, ref.val)
    # with a push mask as well
    M = datasets.rmat_csr(11, 16, seed=23)
    gm = api.spgemm(A, A, M, semiring)
    rm = oracle.spgemm(_orc(A), _orc(A), _orc(M), code)
    assert np.array_equal(gm.a2pos, rm.a2pos) and np.array_equal(gm.a2crd, rm.a2crd)
    if semiring.startswith("+"):
        _close(gm.val, rm.val, oracle.spgemm(_abs(A), _abs(A), _orc(M), code).val)
    else:
        assert np.array_equal(gm.val, rm.val)


@pytest.mark.parametrize("fmt", ["CSR", "DCSR", "COO"])
def test_dense_times_sparse(fmt, tmp_path):
    Bm = _skewed(400, seed=31)
    path = tmp_path / "b.mtx"
    datasets.write_mtx(str(path), Bm)
    B = oracle.read_mtx(str(path), fmt)
    x = datasets.dense_uniform(B.nrows, 1)
    A = datasets.dense_uniform((13, B.nrows), 2)
    absB = _abs(B)
    _close(api.dense_times_sparse(x, B), oracle.dense_times_sparse(x, B), oracle.dense_times_sparse(np.abs(x), absB))
    C0 = datasets.dense_uniform((13, B.ncols), 3)
    _close(api.dense_times_sparse(A, B, C0), oracle.dense_times_sparse(A, B, C0),
           oracle.dense_times_sparse(np.abs(A), absB, np.abs(C0)))
    _close(api.einsum("ij,jk->ik", A, B), oracle.dense_times_sparse(A, B), oracle.dense_times_sparse(np.abs(A), absB))
    assert np.array_equal(api.dense_times_sparse(x, B, semiring=api.PLUS_PAIR),
                          oracle.dense_times_sparse(x, B, semiring=oracle.PLUS_PAIR))


@pytest.mark.parametrize("m", [32, 33, 130])
def test_dense_times_sparse_many_rows(m, monkeypatch):
    """From 32 rows of the dense operand on (B in CSR) the product is formed as C^T = B^T A^T by the SpMM
    kernels; odd row counts are padded to an even width.  Held to the oracle, and to the atomics kernel."""
    B = _skewed(3000, seed=41)
    A = datasets.dense_uniform((m, B.nrows), 2)
    C0 = datasets.dense_uniform((m, B.ncols), 3)
    absB = _abs(B)
    want = oracle.dense_times_sparse(A, _orc(B))
    scale = oracle.dense_times_sparse(np.abs(A), absB, np.abs(C0))
    got = api.dense_times_sparse(A, B)
    _close(got, want, scale)
    _close(api.dense_times_sparse(A, B, C0), oracle.dense_times_sparse(A, _orc(B), C0), scale)
    assert np.array_equal(api.dense_times_sparse(A, B, semiring=api.PLUS_PAIR),
                          oracle.dense_times_sparse(A, _orc(B), semiring=oracle.PLUS_PAIR))
    monkeypatch.setenv("COMET_B200_DENSE_SPARSE_ATOMICS", "1")
    _close(api.dense_times_sparse(A, B), got, scale)


@pytest.mark.parametrize("fmt", ["CSR", "DCSR", "COO"])
def test_elews_sparse_dense_to_dense(fmt, tmp_path):
    Am = _skewed(500, seed=41)
    path = tmp_path / "a.mtx"
    datasets.write_mtx(str(path), Am)
    A = oracle.read_mtx(str(path), fmt)
    B = datasets.dense_uniform((A.nrows, A.ncols), 4)
    C0 = datasets.dense_uniform((A.nrows, A.ncols), 5)
    # a product is one IEEE multiply: the results are bit-identical, untouched entries included
    assert np.array_equal(api.elews_sparse_dense_to_dense(A, B), oracle.elews_sparse_dense_to_dense(A, B))
    assert np.array_equal(api.elews_sparse_dense_to_dense(A, B, C0), oracle.elews_sparse_dense_to_dense(A, B, C0))
    A32 = api.as_sparse(A).with_index_dtype(np.int32)
    assert np.array_equal(api.elews_sparse_dense_to_dense(A32, B), oracle.elews_sparse_dense_to_dense(A, B))


def test_device_coo_to_csr_reproduces_the_reader_goldens(golden, mtx_dir):
    """The reader sorts the parsed entries on the host; the device sort must give the same CSR arrays.
    Every CSR reader test of the reference is replayed: the entries (as the reader keeps them, read mode
    applied) are shuffled, sorted on the device, printed and compared with the CHECK lines."""
    import os
    rng = np.random.default_rng(11)
    n = 0
    for name, case in golden["cases"].items():
        if case["kind"] != "reader":
            continue
        (tname, r), = case["reads"].items()
        if case["tensors"][tname]["format"] != "CSR":
            continue
        path = os.path.join(mtx_dir, case["files"][r["file_id"]])
        coo = oracle.read_mtx(path, "COO", r["read_mode"])
        perm = rng.permutation(coo.nnz)
        got = api.from_coordinates(np.asarray(coo.a1crd)[perm], np.asarray(coo.a2crd)[perm], coo.val[perm],
                                   (coo.nrows, coo.ncols))
        text = "".join(oracle.print_memref(a) for a in (got.a1pos, got.a1crd, got.a2pos, got.a2crd, got.val))
        want = oracle.read_mtx(path, "CSR", r["read_mode"])
        assert text == "".join(oracle.print_memref(a) for a in (want.a1pos, want.a1crd, want.a2pos, want.a2crd, want.val))
        assert [l for l in text.splitlines() if l.strip() and not l.startswith("data")] == \
               [c for c in case["checks"] if not c.startswith("data")]
        n += 1
    assert n >= 5
    # equal coordinates keep their input order (values tell them apart)
    rows = np.array([2, 0, 2, 1, 2, 0]); cols = np.array([1, 3, 1, 0, 1, 3]); vals = np.arange(6.0)
    got = api.from_coordinates(rows, cols, vals, (3, 4))
    assert got.a2pos.tolist() == [0, 2, 3, 6] and got.a2crd.tolist() == [3, 3, 0, 1, 1, 1]
    assert got.val.tolist() == [1.0, 5.0, 3.0, 0.0, 2.0, 4.0]


@pytest.mark.parametrize("index_dtype", [np.int64, np.int32])
def test_sparse_transpose(index_dtype, tmp_path):
    A = _skewed(1500, seed=13).with_index_dtype(index_dtype)
    T = api.transpose(A)
    ref = oracle.transpose(_orc(A))
    assert (T.nrows, T.ncols) == (ref.nrows, ref.ncols)
    assert T.a2pos.dtype == index_dtype and T.a2crd.dtype == index_dtype
    assert np.array_equal(T.a2pos, ref.a2pos) and np.array_equal(T.a2crd, ref.a2crd) and np.array_equal(T.val, ref.val)
    want = A.to_scipy().T.tocsr()
    want.sort_indices()
    assert np.array_equal(T.a2pos, want.indptr) and np.array_equal(T.a2crd, want.indices)
    # rectangular, with empty rows and columns; twice transposed is the matrix itself
    R = api.as_sparse(sp.random(300, 7000, density=0.001, random_state=np.random.default_rng(5), format="csr"))
    RT = api.transpose(R)
    assert (RT.nrows, RT.ncols) == (7000, 300)
    RTT = api.transpose(RT)
    assert np.array_equal(RTT.a2pos, R.a2pos) and np.array_equal(RTT.a2crd, R.a2crd) and np.array_equal(RTT.val, R.val)
    # COO -> COO
    path = tmp_path / "a.mtx"
    datasets.write_mtx(str(path), A)
    C = oracle.read_mtx(str(path), "COO")
    TC = api.transpose(C)
    rc = oracle.transpose(C)
    assert np.array_equal(TC.a1crd, rc.a1crd) and np.array_equal(TC.a2crd, rc.a2crd) and np.array_equal(TC.val, rc.val)
    assert TC.a1pos.tolist() == [0, C.nnz]


def _same_arrays(got, ref):
    for name in ("a1pos", "a1crd", "a2pos", "a2crd", "val"):
        assert np.array_equal(np.asarray(getattr(got, name)), np.asarray(getattr(ref, name))), name
    assert (got.nrows, got.ncols) == (ref.nrows, ref.ncols)


def test_reader_entry_points_reproduce_the_reader_goldens(golden, mtx_dir, tmp_path):
    """read_input_sizes_2D / read_input_2D stand-ins (sort on the device): every reader test of the
    reference prints the same lines, and all formats / read modes agree with the oracle's reader."""
    import os
    n = 0
    for name, case in golden["cases"].items():
        if case["kind"] != "reader":
            continue
        (tname, r), = case["reads"].items()
        fmt = case["tensors"][tname]["format"]
        path = os.path.join(mtx_dir, case["files"][r["file_id"]])
        got = api.read_mtx(path, fmt, r["read_mode"])
        text = "".join(oracle.print_memref(a) for a in (got.a1pos, got.a1crd, got.a2pos, got.a2crd, got.val))
        assert [l for l in text.splitlines() if l.strip() and not l.startswith("data")] == \
               [c for c in case["checks"] if not c.startswith("data")], name
        n += 1
    assert n == 10
    # a larger file: symmetric banner, repeated coordinates, a pattern-only line, empty rows
    rng = np.random.default_rng(21)
    path = tmp_path / "sym.mtx"
    m = 400
    with open(path, "w") as f:
        ent = [(int(a), int(b)) for a, b in zip(rng.integers(1, m + 1, 3000), rng.integers(1, m + 1, 3000)) if a >= b]
        ent += ent[:5]
        f.write("%%MatrixMarket matrix coordinate real symmetric\n% comment\n")
        f.write("%d %d %d\n" % (m, m, len(ent)))
        for i, (a, b) in enumerate(ent):
            f.write("%d %d\n" % (a, b) if i == 7 else "%d %d %.17g\n" % (a, b, rng.uniform(-1, 1)))
    for fmt in ("CSR", "COO", "DCSR"):
        for mode in (1, 2, 3, 4, 5):
            _same_arrays(api.read_mtx(str(path), fmt, mode), oracle.read_mtx(str(path), fmt, mode))
    g32 = api.read_mtx(str(path), "CSR", 1, index_dtype=np.int32)
    assert g32.a2pos.dtype == np.int32
    _same_arrays(g32, oracle.read_mtx(str(path), "CSR", 1))
    # the arrays feed the kernels directly
    A = api.read_mtx(str(path), "CSR")
    x = datasets.dense_uniform(A.ncols, 1)
    ref = oracle.spmv(oracle.read_mtx(str(path), "CSR"), x)
    _close(api.spmv(A, x), ref, np.abs(ref) + 1.0)


@pytest.mark.parametrize("k", [64, 128])
def test_sddmm_empty_rows_and_a_hub_row(k):
    """Empty rows at every position, single-entry rows and a row far longer than a chunk, at a size where
    both SDDMM kernels (entry stream for short rows, chunk list for long ones) carry work."""
    S = _gappy(n=70000, seed=8)
    X = datasets.dense_uniform((S.nrows, k), 1)
    Y = datasets.dense_uniform((S.ncols, k), 2)
    _close(api.sddmm(S, X, Y), oracle.sddmm(_orc(S), X, Y), oracle.sddmm(_abs(S), np.abs(X), np.abs(Y)))
