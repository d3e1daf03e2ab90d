"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (numpy ``default_rng(seed)``; no files, no network).

R-MAT: one quadrant draw per bit level with probabilities (a, b, c, d) =
(0.57, 0.19, 0.19, 0.05), no noise, no vertex permutation; duplicate edges are
removed by sorting the (row, col) keys, which also yields CSR order.
"""
import numpy as np

from .api import SparseTensor

RMAT_PROBS = (0.57, 0.19, 0.19, 0.05)


def _csr_from_sorted_keys(keys, n, vals):
    rows = keys // n
    cols = keys - rows * n
    pos = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=pos[1:])
    return SparseTensor("CSR", n, n, np.array([n], dtype=np.int64), np.array([-1], dtype=np.int64),
                        pos, cols.astype(np.int64), vals)


def rmat_edges(scale, edge_factor, seed=0, probs=RMAT_PROBS, chunk=1 << 24):
    """(rows, cols) int64 arrays of edge_factor * 2^scale R-MAT draws."""
    rng = np.random.default_rng(seed)
    a, b, c, _ = probs
    total = edge_factor << scale
    rows = np.empty(total, dtype=np.int64)
    cols = np.empty(total, dtype=np.int64)
    for lo in range(0, total, chunk):
        m = min(chunk, total - lo)
        r = np.zeros(m, dtype=np.int64)
        cc = np.zeros(m, dtype=np.int64)
        for _level in range(scale):
            u = rng.random(m)
            row_bit = u >= a + b                       # quadrants c and d
            col_bit = u >= a                           # quadrants b and d: [a, a+b) and [a+b+c, 1)
            col_bit ^= row_bit
            col_bit |= u >= a + b + c
            np.left_shift(r, 1, out=r)
            np.bitwise_or(r, row_bit, out=r)
            np.left_shift(cc, 1, out=cc)
            np.bitwise_or(cc, col_bit, out=cc)
        rows[lo:lo + m] = r
        cols[lo:lo + m] = cc
    return rows, cols


def rmat_csr(scale, edge_factor, seed=0, drop_self_loops=True, symmetrize=False, lower_strict=False,
             values="u0515"):
    """Deduplicated R-MAT matrix in CSR with sorted columns.

    values: 'u0515' -> U(0.5, 1.5), 'ones' -> 1.0."""
    n = 1 << scale
    rows, cols = rmat_edges(scale, edge_factor, seed)
    if symmetrize and lower_strict:
        # the strict lower triangle of the symmetrised graph: every draw off the diagonal, larger end first
        hi, lo = np.maximum(rows, cols), np.minimum(rows, cols)
        keep = hi != lo
        rows, cols = hi[keep], lo[keep]
        del hi, lo
    else:
        if symmetrize:
            rows, cols = np.concatenate([rows, cols]), np.concatenate([cols, rows])
        if drop_self_loops:
            keep = rows != cols
            rows, cols = rows[keep], cols[keep]
        if lower_strict:
            keep = rows > cols
            rows, cols = rows[keep], cols[keep]
    # sorted distinct keys (an in-place sort and one comparison pass; np.unique is many times slower here)
    keys = rows * n + cols
    del rows, cols
    keys.sort()
    if keys.shape[0] > 1:
        keys = keys[np.concatenate(([True], keys[1:] != keys[:-1]))]
    rng = np.random.default_rng(seed + 1)
    vals = np.ones(keys.shape[0]) if values == "ones" else rng.uniform(0.5, 1.5, keys.shape[0])
    return _csr_from_sorted_keys(keys, n, vals)


def uniform_rows_csr(n, per_row, seed=0):
    """Each row: ``per_row`` distinct columns drawn uniformly without replacement, sorted;
    values U(-1, 1)."""
    rng = np.random.default_rng(seed)
    # distinct columns per row: rank a random matrix, batched to bound memory
    cols = np.empty((n, per_row), dtype=np.int64)
    batch = max(1, (1 << 24) // n)
    for lo in range(0, n, batch):
        hi = min(n, lo + batch)
        u = rng.random((hi - lo, n))
        part = np.argpartition(u, per_row, axis=1)[:, :per_row]
        cols[lo:hi] = np.sort(part, axis=1)
    pos = np.arange(n + 1, dtype=np.int64) * per_row
    vals = rng.uniform(-1.0, 1.0, n * per_row)
    return SparseTensor("CSR", n, n, np.array([n], dtype=np.int64), np.array([-1], dtype=np.int64), pos,
                        cols.reshape(-1), vals)


def dense_uniform(shape, seed, lo=-1.0, hi=1.0):
    return np.random.default_rng(seed).uniform(lo, hi, shape)


def write_mtx(path, A):
    """MatrixMarket coordinate file, 1-based, values with 17 significant digits so
    that float64 round-trips through COMET's text reader."""
    with open(path, "w") as f:
        f.write("%%MatrixMarket matrix coordinate real general\n")
        f.write("%d %d %d\n" % (A.nrows, A.ncols, A.nnz))
        rows = np.repeat(np.arange(A.nrows), np.diff(A.a2pos))
        for r, c, v in zip(rows, A.a2crd, A.val):
            f.write("%d %d %.17g\n" % (r + 1, c + 1, v))


# The five benchmark configurations.  ``scale`` may be lowered for tests.
def config_spmv(n=16384, per_row=16, seed=0):
    A = uniform_rows_csr(n, per_row, seed)
    return A, dense_uniform(n, seed + 7)


def config_spmm(scale=20, edge_factor=16, k=128, seed=0):
    A = rmat_csr(scale, edge_factor, seed)
    return A, dense_uniform((A.ncols, k), seed + 7)


def config_sddmm(scale=18, edge_factor=32, k=64, seed=0):
    S = rmat_csr(scale, edge_factor, seed, drop_self_loops=False)
    return S, dense_uniform((S.nrows, k), seed + 7), dense_uniform((S.ncols, k), seed + 8)


def config_spgemm(scale=18, edge_factor=16, seed=0):
    return rmat_csr(scale, edge_factor, seed)


def config_triangles(scale=22, edge_factor=16, seed=0):
    return rmat_csr(scale, edge_factor, seed, symmetrize=True, lower_strict=True, values="ones")


def algorithmic_bytes(kind, nrows, ncols, nnz, k=0, nnz_b=0, nnz_c=0, nrows_b=0):
    """Compulsory traffic of one call at the ABI's widths (int64 indices, float64
    values): every input array read once, every output written once."""
    if kind == "spmv":
        return 8 * (nrows + 1) + 16 * nnz + 8 * ncols + 8 * nrows
    if kind == "spmm":
        return 8 * (nrows + 1) + 16 * nnz + 8 * ncols * k + 8 * nrows * k
    if kind == "sddmm":
        return 8 * (nrows + 1) + 24 * nnz + 8 * k * (nrows + ncols)
    if kind == "spgemm":
        size = lambda n, z: 8 * (n + 1) + 16 * z
        return size(nrows, nnz) + size(nrows_b, nnz_b) + size(nrows, nnz_c)
    if kind == "triangles":
        return 8 * (nrows + 1) + 8 * nnz
    raise ValueError(kind)
