#!/usr/bin/env python3
"""Extract golden vectors for the sparse hot path from the COMET source tree.

Run once, where the COMET checkout is available:

    python tests/golden/make_golden.py /path/to/COMET

It reads the integration tests under test/integration/{ops,semiring,kernels}
that exercise the readers, SpMV, SpMM, SDDMM, elementwise multiply, SpGEMM
(plain, masked, plus-pair), SUM and triangle counting, and writes
``tests/golden/comet_golden.json`` with, per test: what the program computes
(parsed from the .ta text: tensor formats, constant fills, comet_read ids and
read modes, index sizes), the expected printed output (the CHECK lines), and
the coordinate data of the .mtx files those tests read.  Only data and expected
outputs are stored; no program text or source code is copied.
"""
import json
import os
import re
import sys

CASES = {
    # reader goldens (print a tensor right after comet_read)
    "ops/utility_printCSR.ta": "reader",
    "ops/utility_printCSR_lowerTri.ta": "reader",
    "ops/utility_printCSR_lowerTriStrict.ta": "reader",
    "ops/utility_printCSR_upperTri.ta": "reader",
    "ops/utility_printCSR_upperTriStrict.ta": "reader",
    "ops/utility_printCOO.ta": "reader",
    "ops/utility_printCOO_lowerTri.ta": "reader",
    "ops/utility_printCOO_lowerTriStrict.ta": "reader",
    "ops/utility_printCOO_upperTri.ta": "reader",
    "ops/utility_printCOO_upperTriStrict.ta": "reader",
    # sparse x dense -> dense
    "ops/mult_spmv_CSRxDense.ta": "spmv",
    "ops/mult_spmv_DCSRxDense.ta": "spmv",
    "ops/mult_spmv_COOxDense.ta": "spmv",
    "semiring/mv_SemiringPlusTimes_CSRxDense_oDense.ta": "spmv",
    "semiring/mv_SemiringPlusTimes_DCSRxDense_oDense.ta": "spmv",
    "semiring/mv_SemiringPlusTimes_COOxDense_oDense.ta": "spmv",
    "ops/mult_spmm_CSRxDense.ta": "spmm",
    "ops/mult_spmm_DCSRxDense.ta": "spmm",
    "ops/mult_spmm_COOxDense.ta": "spmm",
    "semiring/mm_SemiringPlusTimes_CSRxDense_oDense.ta": "spmm",
    "semiring/mm_SemiringPlusTimes_DCSRxDense_oDense.ta": "spmm",
    "semiring/mm_SemiringPlusTimes_COOxDense_oDense.ta": "spmm",
    # dense x sparse -> dense
    "ops/mult_DenseMatxCSR.ta": "dense_sparse",
    "ops/mult_DenseMatxDCSR.ta": "dense_sparse",
    "ops/mult_DenseMatxCOO.ta": "dense_sparse",
    "ops/mult_DenseVecxCSR.ta": "dense_sparse",
    "ops/mult_DenseVecxDCSR.ta": "dense_sparse",
    "ops/mult_DenseVecxCOO.ta": "dense_sparse",
    "semiring/mm_SemiringPlusTimes_DensexCSR_oDense.ta": "dense_sparse",
    "semiring/mm_SemiringPlusTimes_DensexDCSR_oDense.ta": "dense_sparse",
    "semiring/mm_SemiringPlusTimes_DensexCOO_oDense.ta": "dense_sparse",
    "semiring/mv_SemiringPlusTimes_DensexCSR_oDense.ta": "dense_sparse",
    "semiring/mv_SemiringPlusTimes_DensexDCSR_oDense.ta": "dense_sparse",
    "semiring/mv_SemiringPlusTimes_DensexCOO_oDense.ta": "dense_sparse",
    # sampled dense-dense
    "kernels/sddmm.ta": "sddmm",
    # elementwise
    "ops/eltwise_mult_CSRxDense_oCSR.ta": "elews_sparse_dense",
    "ops/eltwise_mult_COOxDense_oCOO.ta": "elews_sparse_dense",
    "semiring/eltwise_monoidTimes_COOxDense_oCOO.ta": "elews_sparse_dense",
    "ops/eltwise_mult_CSRxCSR_oCSR.ta": "elews_sparse_sparse",
    "ops/eltwise_mult_CSRxDense_oDense.ta": "elews_to_dense",
    "ops/eltwise_mult_DCSRxDense_oDense.ta": "elews_to_dense",
    "ops/eltwise_mult_DensexCSR_oDense.ta": "elews_to_dense",
    # sparse x sparse -> sparse
    "ops/mult_spgemm_CSRxCSR_oCSR.ta": "spgemm",
    "ops/mult_spgemm_CSRxCSR_oCSR_wMasking.ta": "spgemm_masked",
    "semiring/mm_SemiringPlusTimes_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringPlusPair_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringPlusFirst_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringPlusSecond_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringMinPlus_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringMinFirst_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringMinSecond_CSRxCSR_oCSR.ta": "spgemm",
    "semiring/mm_SemiringAnyPair_CSRxCSR_oCSR.ta": "spgemm",
    # reductions / triangle counting
    "ops/sum_CSR.ta": "sum",
    "ops/sum_COO.ta": "sum",
    "kernels/triangleCount_SandiaLL.ta": "triangle_count",
    "kernels/triangleCount_SandiaLL_wMasking.ta": "triangle_count",
}


def parse_mtx(path):
    """Keep the banner flags and the raw 1-based entries, in file order."""
    banner, size, entries = "", None, []
    with open(path) as f:
        for line in f:
            if line.startswith("%%"):
                banner = line.strip()
                continue
            if line.startswith("%") or not line.strip():
                continue
            tok = line.split()
            if size is None:
                size = [int(t) for t in tok[:3]]
            else:
                entries.append([int(tok[0]), int(tok[1]), float(tok[2]) if len(tok) > 2 else None])
    return {"banner": banner, "size": size, "entries": entries}


def parse_ta(path):
    text = open(path).read()
    info = {"files": {}, "index_sizes": {}, "tensors": {}, "reads": {}, "fills": {},
            "semiring": None, "mask": None, "checks": []}
    for m in re.finditer(r"SPARSE_FILE_NAME(\d)=\S*/(\S+\.mtx)", text):
        info["files"][m.group(1)] = m.group(2)
    body = []
    for line in text.splitlines():
        s = line.strip()
        m = re.match(r"#\s*CHECK(?:-NEXT)?:\s?(.*)$", s)
        if m:
            info["checks"].append(m.group(1).strip())
            continue
        code = s.split("#", 1)[0].strip()
        if code:
            body.append(code)
    for code in body:
        m = re.match(r"IndexLabel \[(\w+)\] = \[(\?|\d+)\];", code)
        if m:
            info["index_sizes"][m.group(1)] = None if m.group(2) == "?" else int(m.group(2))
            continue
        m = re.match(r"Tensor<double> (\w+)\(\[([\w, ]+)\], ?\{(\w+)\}\);", code)
        if m:
            info["tensors"][m.group(1)] = {"labels": [t.strip() for t in m.group(2).split(",")],
                                           "format": m.group(3)}
            continue
        m = re.match(r"(\w+)\[[\w, ]+\] = comet_read\((\d)(?:, ?(\d))?\);", code)
        if m:
            info["reads"][m.group(1)] = {"file_id": m.group(2),
                                         "read_mode": int(m.group(3)) if m.group(3) else 1}
            continue
        m = re.match(r"(\w+)\[[\w, ]+\] = ([-+]?\d+\.?\d*);", code)
        if m:
            info["fills"][m.group(1)] = float(m.group(2))
            continue
        m = re.search(r"@\(([^)]*)\)", code)
        if m:
            info["semiring"] = m.group(1).replace(" ", "")
        m = re.search(r"\]<(\w+), ?(\w+)>", code)
        if m:
            info["mask"] = {"tensor": m.group(1), "type": m.group(2)}
    return info


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/COMET")
    root = sys.argv[1]
    tdir = os.path.join(root, "test", "integration")
    out = {"source": "pnnl/COMET test/integration (CHECK lines and data/*.mtx)", "matrices": {},
           "cases": {}}
    for rel, kind in sorted(CASES.items()):
        info = parse_ta(os.path.join(tdir, rel))
        info["kind"] = kind
        info["reference_test"] = "test/integration/" + rel
        out["cases"][rel[:-3]] = info
        for name in info["files"].values():
            if name not in out["matrices"]:
                out["matrices"][name] = parse_mtx(os.path.join(tdir, "data", name))
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "comet_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, indent=1, sort_keys=True)
    print("wrote", dst, "with", len(out["cases"]), "cases and", len(out["matrices"]), "matrices")


if __name__ == "__main__":
    main()
