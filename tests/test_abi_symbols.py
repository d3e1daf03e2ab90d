"""CPU checks of the boundary: the shared library loads and exports every symbol
that include/comet_b200.h declares, and fails loudly instead of falling back
when no CUDA device is present."""
import ctypes
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "comet_b200.h")).read()
    return sorted(set(re.findall(r"\b((?:_mlir_ciface_)?comet_b200_[A-Za-z0-9_]+)\s*\(", text)))


def test_header_declares_expected_entry_points():
    names = _declared()
    for want in ("comet_b200_spmv_f64_i64", "comet_b200_spmm_f64_i64", "comet_b200_sddmm_f64_i64",
                 "comet_b200_spgemm_symbolic_f64_i64", "comet_b200_spgemm_numeric_f64_i64",
                 "comet_b200_masked_spgemm_count_f64_i64", "comet_b200_dev_spmm_f64_i64"):
        assert want in names


def test_library_exports_every_declared_symbol():
    from comet_b200 import _lib, build
    build.build_library()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in _declared() if not hasattr(lib, n)]
    assert not missing, missing
    # and the ctypes table covers the same set
    assert sorted(_lib.SIGNATURES) == _declared()


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import scipy.sparse as sp
    import comet_b200
    from comet_b200._lib import CometB200Error
    A = sp.random(8, 8, density=0.3, format="csr", random_state=0)
    with pytest.raises(CometB200Error, match="no CUDA device|CUDA"):
        comet_b200.spmv(A, np.ones(8))


def test_reader_needs_a_device_and_reports_bad_files(tmp_path):
    import torch
    import comet_b200.api as api
    from comet_b200._lib import CometB200Error
    with pytest.raises(CometB200Error, match="cannot open"):
        api.read_mtx(str(tmp_path / "missing.mtx"))
    bad = tmp_path / "bad.mtx"
    bad.write_text("%%MatrixMarket matrix coordinate real general\n2 2\n3 1 1.0\n")
    with pytest.raises(CometB200Error, match="size line needs"):       # the header is parsed on the host
        api.read_mtx(str(bad))
    if torch.cuda.is_available():                                      # the entry lines are parsed on the device
        bad.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n3 1 1.0\n")
        os.environ.pop("SPARSE_FILE_NAME0", None)
        with pytest.raises(CometB200Error, match="outside"):
            api.read_mtx(str(bad), file_id=1)
    if not torch.cuda.is_available():
        ok = tmp_path / "ok.mtx"
        ok.write_text("%%MatrixMarket matrix coordinate real general\n2 2 1\n2 1 1.0\n")
        with pytest.raises(CometB200Error, match="no CUDA device"):
            api.read_mtx(str(ok))


def test_bad_descriptors_are_rejected_on_the_host():
    import comet_b200
    from comet_b200._lib import CometB200Error
    from comet_b200.api import SparseTensor
    bad = SparseTensor("CSR", 4, 4, np.array([4]), np.array([-1]), np.array([0, 1, 2]),  # pos too short
                       np.array([0, 1]), np.array([1.0, 2.0]))
    with pytest.raises(CometB200Error, match="pos array shorter"):
        comet_b200.spmv(bad, np.ones(4))
    ok = SparseTensor("CSR", 2, 2, np.array([2]), np.array([-1]), np.array([0, 1, 2]), np.array([0, 1]),
                      np.array([1.0, 2.0]))
    with pytest.raises(CometB200Error, match="x shorter"):
        comet_b200.spmv(ok, np.ones(1))
    with pytest.raises(ValueError, match="semiring"):
        comet_b200.spmv(ok, np.ones(2), semiring="min,plus")
    # 32-bit index arrays handed to the 64-bit entry point are refused on the host: read as
    # int64 the row pointer no longer starts at 0 / stops being monotone
    from comet_b200 import _lib
    from comet_b200.api import _Packer
    narrow = SparseTensor("CSR", 4, 4, np.array([4], dtype=np.int32), np.array([-1], dtype=np.int32),
                          np.array([0, 1, 2, 3, 4, 0, 0, 0, 0, 0], dtype=np.int32),
                          np.array([0, 1, 2, 3, 0, 0, 0, 0], dtype=np.int32), np.ones(8))
    pk = _Packer()
    x, y = np.ones(4), np.zeros(4)
    _lib.load().comet_b200_spmv_f64_i64(*pk.sparse(narrow), *pk.m1(x), *pk.m1(y), 0, 0)
    with pytest.raises(CometB200Error, match="pos"):
        _lib.check()


def test_default_error_mode_exits_like_the_reference_runtime():
    """Without COMET_B200_ON_ERROR=return a failure prints a message and exits with status 1, which is
    what COMET's own runtime does (lib/ExecutionEngine/SparseUtils.cpp:158-168)."""
    import subprocess
    import sys
    code = (
        "import ctypes, sys; sys.path.insert(0, %r)\n"
        "from comet_b200 import _lib\n"
        "lib = ctypes.CDLL(_lib.LIB_PATH)\n"
        "lib.comet_b200_spgemm_numeric_f64_i64.argtypes = [ctypes.c_int64] + [ctypes.c_int64, ctypes.c_void_p] * 2\n"
        "lib.comet_b200_spgemm_numeric_f64_i64(12345, 1, None, 1, None)\n"
        "print('survived')\n" % ROOT)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120)
    assert r.returncode == 1
    assert "libcomet_b200: ERROR" in r.stderr and "unknown handle" in r.stderr
    assert "survived" not in r.stdout


def test_the_concurrency_contract_of_the_device_layer_is_stated_where_callers_look():
    """The device-pointer entry points keep their work lists and counters in one scratch area per device, so
    calls on one device must not overlap.  That is a contract, not something the library can enforce across
    streams; it has to be written where a caller reads: beside the layer-2 declarations and in the
    integration notes."""
    header = open(os.path.join(ROOT, "include", "comet_b200.h")).read()
    layer2 = header[header.index("Layer 2: device pointers"):]
    assert "must therefore not overlap" in layer2 and "one stream at a time" in layer2
    notes = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    assert "One call at a time per device" in notes
