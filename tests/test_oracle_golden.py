"""Pins the CPU oracle against the reference's own golden outputs (the CHECK
lines of its integration tests).  CPU only."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from tests import golden_runner

_G = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "comet_golden.json")))


@pytest.mark.parametrize("name", sorted(_G["cases"]))
def test_oracle_matches_reference_check_lines(name, golden, mtx_dir):
    case = golden["cases"][name]
    got = golden_runner.run_case(case, mtx_dir, oracle)
    assert golden_runner.normalise(got) == golden_runner.expected_text(case)


def test_triangle_count_two_ways(golden, mtx_dir):
    """SUM((L*L) .* L) by materialising the masked product equals the direct count."""
    L = oracle.read_mtx(str(mtx_dir / "tc.mtx"), "CSR", 2)
    C = oracle.spgemm(L, L, L, oracle.PLUS_PAIR)
    assert oracle.reduce_sum(C.val) == 5.0
    assert oracle.masked_pair_count(L, L, L) == 5
    # unmasked product followed by the elementwise multiply (the first spelling)
    P = oracle.spgemm(L, L, None, oracle.PLUS_TIMES)
    E = oracle.elews_csr_csr(P, L)
    assert oracle.reduce_sum(E.val) == 5.0


def test_oracle_against_scipy_random():
    sp = pytest.importorskip("scipy.sparse")
    rng = np.random.default_rng(1)
    A = sp.random(200, 150, density=0.05, random_state=rng, format="csr", dtype=np.float64)
    B = sp.random(150, 180, density=0.05, random_state=rng, format="csr", dtype=np.float64)
    A.sort_indices(); B.sort_indices()
    oa, ob = oracle.from_scipy_csr(A), oracle.from_scipy_csr(B)
    C = oracle.spgemm(oa, ob)
    ref = (A @ B).tocsr(); ref.sort_indices()
    # scipy prunes nothing here either (no explicit zeros arise from random data)
    assert np.array_equal(C.a2pos, ref.indptr)
    assert np.array_equal(C.a2crd, ref.indices)
    np.testing.assert_allclose(C.val, ref.data, rtol=1e-13)
    x = rng.uniform(-1, 1, 150)
    np.testing.assert_allclose(oracle.spmv(oa, x), A @ x, rtol=1e-12, atol=1e-14)
    D = rng.uniform(-1, 1, (150, 7))
    np.testing.assert_allclose(oracle.spmm(oa, D), A @ D, rtol=1e-12, atol=1e-14)
    X = rng.uniform(-1, 1, (200, 9)); Y = rng.uniform(-1, 1, (150, 9))
    want = np.asarray(A.multiply(X @ Y.T).tocsr()[A.nonzero()]).ravel()
    np.testing.assert_allclose(oracle.sddmm(oa, X, Y), want, rtol=1e-12, atol=1e-14)


def test_transpose_restatement_against_scipy():
    """No reference test prints a transposed sparse matrix, so this piece of the oracle is held against
    scipy instead: CSR and COO, duplicates kept in input order."""
    import scipy.sparse as sp
    rng = np.random.default_rng(7)
    m = sp.random(60, 45, density=0.1, random_state=rng, format="csr")
    m.sort_indices()
    A = oracle.SparseArrays("CSR", 60, 45, np.array([60]), np.array([-1]), m.indptr.astype(np.int64),
                            m.indices.astype(np.int64), m.data.copy())
    T = oracle.transpose(A)
    want = m.T.tocsr()
    want.sort_indices()
    assert (T.nrows, T.ncols) == (45, 60)
    assert np.array_equal(T.a2pos, want.indptr) and np.array_equal(T.a2crd, want.indices)
    assert np.array_equal(T.val, want.data)
    # COO with a repeated coordinate: both copies survive, first one first
    C = oracle.SparseArrays("COO", 3, 4, np.array([0, 4]), np.array([0, 1, 1, 2]), np.array([-1]),
                            np.array([2, 3, 3, 0]), np.array([1.0, 2.0, 3.0, 4.0]))
    Tc = oracle.transpose(C)
    assert Tc.a1crd.tolist() == [0, 2, 3, 3] and Tc.a2crd.tolist() == [2, 0, 1, 1]
    assert Tc.val.tolist() == [4.0, 1.0, 2.0, 3.0]


def test_rowparallel_variants_equal_the_sequential_oracle():
    """The row-parallel CPU variants (a second, clearly labelled baseline: not COMET's schedule) give the
    same arrays and the same count as the sequential restatement."""
    import numpy as np
    from comet_b200 import datasets
    from oracle import oracle
    A = datasets.rmat_csr(10, 8, seed=2)
    oa = oracle.SparseArrays("CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd, A.val)
    ref, par = oracle.spgemm(oa, oa), oracle.spgemm_rowparallel(oa, oa)
    assert np.array_equal(ref.a2pos, par.a2pos) and np.array_equal(ref.a2crd, par.a2crd)
    assert np.array_equal(ref.val, par.val)
    L = datasets.config_triangles(scale=10, edge_factor=8)
    ol = oracle.SparseArrays("CSR", L.nrows, L.ncols, L.a1pos, L.a1crd, L.a2pos, L.a2crd, L.val)
    assert oracle.masked_pair_count(ol, ol, ol) == oracle.masked_pair_count_rowparallel(ol, ol, ol)
    assert oracle.masked_pair_count(ol, ol, ol, 100, 700) == oracle.masked_pair_count_rowparallel(ol, ol, ol, 100, 700)
