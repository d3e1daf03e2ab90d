"""Runs one golden case (a restated COMET integration test) on a backend and
returns the text the program would print, so that it can be compared with the
reference test's CHECK lines.  The backend is either the CPU oracle or the
CUDA library behind its C-ABI; inputs are always read with the oracle's
restatement of the reference reader (reading files is not part of the path
the CUDA library replaces)."""
import numpy as np

from oracle import oracle


def _print_sparse(t):
    a1crd = t.a1crd if t.format in ("COO", "DCSR") else np.array([-1])
    a2pos = t.a2pos if t.format in ("CSR", "DCSR") else np.array([-1])
    return "".join(oracle.print_memref(a) for a in (t.a1pos, a1crd, a2pos, t.a2crd, t.val))


def _scalar(v):
    return "%g\n" % v


def run_case(case, mtx_dir, backend):
    """backend: object with spmv, spmm, sddmm, elews_sparse_dense, elews_csr_csr,
    spgemm, reduce_sum, masked_pair_count (same signatures as oracle.oracle)."""
    T = case["tensors"]
    read = {}
    for name, r in case["reads"].items():
        path = str(mtx_dir / case["files"][r["file_id"]])
        read[name] = oracle.read_mtx(path, T[name]["format"], r["read_mode"])
    fills = case["fills"]
    kind = case["kind"]
    semiring = {None: oracle.PLUS_TIMES, "*": oracle.PLUS_TIMES, "+,*": oracle.PLUS_TIMES,
                "+,pair": oracle.PLUS_PAIR, "+,first": oracle.PLUS_FIRST, "+,second": oracle.PLUS_SECOND,
                "min,+": oracle.MIN_PLUS, "min,first": oracle.MIN_FIRST, "min,second": oracle.MIN_SECOND,
                "any,pair": oracle.ANY_PAIR}[case["semiring"]]

    if kind == "reader":
        return _print_sparse(next(iter(read.values())))
    if kind == "sum":
        return _scalar(backend.reduce_sum(next(iter(read.values())).val))
    if kind == "spmv":
        A = read["A"]
        x = np.full(A.ncols, fills["B"])
        y = backend.spmv(A, x, np.full(A.nrows, fills["C"]), semiring)
        return oracle.print_memref(y)
    if kind == "spmm":
        A = read["A"]
        k = case["index_sizes"]["c"]
        B = np.full((A.ncols, k), fills["B"])
        C = backend.spmm(A, B, np.full((A.nrows, k), fills["C"]), semiring)
        return oracle.print_memref(C)
    if kind == "dense_sparse":
        B = read["B"]
        a_labels = T["A"]["labels"]
        if len(a_labels) == 1:
            A = np.full(B.nrows, fills["A"])
            C0 = np.full(B.ncols, fills["C"])
        else:
            A = np.full((case["index_sizes"][a_labels[0]], B.nrows), fills["A"])
            C0 = np.full((A.shape[0], B.ncols), fills["C"])
        return oracle.print_memref(backend.dense_times_sparse(A, B, C0, semiring))
    if kind == "sddmm":
        S = read["B"]
        k = case["index_sizes"]["k"]
        X = np.full((S.nrows, k), fills["C"])
        D = np.full((k, S.ncols), fills["D"])
        vals = backend.sddmm(S, X, D, y_is_kj=True)
        out = oracle.SparseArrays("CSR", S.nrows, S.ncols, S.a1pos, S.a1crd, S.a2pos, S.a2crd, vals)
        return _print_sparse(out)
    if kind == "elews_sparse_dense":
        A = read["A"]
        B = np.full((A.nrows, A.ncols), fills["B"])
        vals = backend.elews_sparse_dense(A, B)
        out = oracle.SparseArrays(A.format, A.nrows, A.ncols, A.a1pos, A.a1crd, A.a2pos, A.a2crd, vals)
        return _print_sparse(out)
    if kind == "elews_to_dense":
        name = next(iter(read))                      # the sparse operand is A or B; the other one is dense
        S = read[name]
        dense = "B" if name == "A" else "A"
        D = np.full((S.nrows, S.ncols), fills[dense])
        return oracle.print_memref(backend.elews_sparse_dense_to_dense(S, D, np.full((S.nrows, S.ncols), fills["C"])))
    if kind == "elews_sparse_sparse":
        return _print_sparse(backend.elews_csr_csr(read["A"], read["B"]))
    if kind == "spgemm":
        return _print_sparse(backend.spgemm(read["A"], read["B"], None, semiring))
    if kind == "spgemm_masked":
        M = read[case["mask"]["tensor"]]
        return _print_sparse(backend.spgemm(read["A"], read["B"], M, semiring))
    if kind == "triangle_count":
        L = read["L1"]
        # both spellings (elementwise form and push-masked form) define the same sum
        return _scalar(backend.masked_pair_count(L, L, L))
    raise ValueError(kind)


def expected_text(case):
    return "".join(line.strip() + "\n" for line in case["checks"])


def normalise(text):
    return "".join(line.strip() + "\n" for line in text.splitlines())
