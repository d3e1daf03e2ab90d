"""MatrixMarket text parsed on the device (comet_b200/csrc/parse.cu) against the CPU restatement of the
reference's parser (oracle.read_mtx follows lib/ExecutionEngine/SparseUtils.cpp:145-533): every array
bit for bit, for files that exercise comments, odd spacing, pattern entries, symmetric
and skew-symmetric banners, dense `array` listings, repeated coordinates, a missing final newline,
values that the device parser hands back to the host (more than 19 digits, octal-looking integers)
and a file of a few hundred thousand %.17g values."""
import numpy as np
import pytest

import comet_b200.api as api
from comet_b200 import datasets
from oracle import oracle

pytestmark = pytest.mark.gpu


def _same(path, fmt, mode=1, fid=0):
    got = api.read_mtx(str(path), fmt, mode, file_id=fid)
    ref = oracle.read_mtx(str(path), fmt, mode)
    assert (got.nrows, got.ncols) == (ref.nrows, ref.ncols)
    for name in ("a1pos", "a1crd", "a2pos", "a2crd"):
        assert np.array_equal(getattr(got, name), getattr(ref, name)), name
    assert got.val.tobytes() == ref.val.tobytes()          # the same doubles, bit for bit
    return got


TRICKY = """%%MatrixMarket matrix coordinate real general
% a comment
%another
  6   7  14
1 1 1.5
2 3   -2.25e-3
\t3\t4\t+7.0E+2
4 5 0.1
4 5 0.30000000000000004
   6 7 1e-20
6 1 123456789012345678901234.5
5 5 .5
5 2 5.
1 7 9007199254740993
3 3 4.9406564584124654e-324
2 2 1e22
2 2 -0
6 6 12345678.9"""          # no newline at the end


def test_general_file_with_awkward_lines(tmp_path):
    p = tmp_path / "tricky.mtx"
    p.write_text(TRICKY)
    for i, fmt in enumerate(("CSR", "COO", "DCSR")):
        A = _same(p, fmt, fid=i)
        assert A.nnz == 14


def test_symmetric_skew_pattern_and_array_files(tmp_path):
    sym = tmp_path / "sym.mtx"
    sym.write_text("%%MatrixMarket matrix coordinate real symmetric\n4 4 5\n1 1 2.0\n3 1 -1.5\n4 2 0.25\n4 4 8\n2 1 3e1\n")
    skew = tmp_path / "skew.mtx"
    skew.write_text("%%MatrixMarket matrix coordinate real skew-symmetric\n3 3 2\n2 1 4.5\n3 2 -1\n")
    pat = tmp_path / "pat.mtx"
    pat.write_text("%%MatrixMarket matrix coordinate pattern general\n3 5 4\n1 5\n3 2\n2 2\n1 5\n")      # a coordinate twice
    arr = tmp_path / "arr.mtx"
    arr.write_text("%%MatrixMarket matrix array real general\n2 3\n1.0\n2.0\n3.5\n-4\n0\n6e-1\n")
    for path in (sym, skew, pat, arr):
        for fmt in ("CSR", "COO"):
            _same(path, fmt)
        for mode in (2, 3, 4, 5):
            _same(path, "CSR", mode)


def test_large_file_of_full_precision_values(tmp_path):
    A = datasets.rmat_csr(13, 24, seed=9)
    A.val[:] = np.random.default_rng(1).uniform(-1, 1, A.nnz) * 10.0 ** np.random.default_rng(2).integers(-12, 6, A.nnz)
    p = tmp_path / "big.mtx"
    datasets.write_mtx(str(p), A)
    got = _same(p, "CSR")
    assert got.nnz == A.nnz and np.array_equal(got.a2crd, A.a2crd) and got.val.tobytes() == A.val.tobytes()


def test_bad_entries_are_reported(tmp_path):
    from comet_b200._lib import CometB200Error
    outside = tmp_path / "outside.mtx"
    outside.write_text("%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1 1.0\n3 1 1.0\n")
    with pytest.raises(CometB200Error, match=r"entry \(3, 1\) outside 2 x 2"):
        api.read_mtx(str(outside))
    junk = tmp_path / "junk.mtx"
    junk.write_text("%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1 1.0\nx y z\n")
    with pytest.raises(CometB200Error, match="bad entry line"):
        api.read_mtx(str(junk))
    many = tmp_path / "many.mtx"
    many.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n1 1 1.0\n2 2 1.0\n")
    with pytest.raises(CometB200Error, match="more entries than the size line"):
        api.read_mtx(str(many))
