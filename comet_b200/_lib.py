"""Loads ``libcomet_b200.so`` (built in-tree by ``comet_b200.build``) and declares
the C ABI of ``include/comet_b200.h`` for ctypes.  There is no fallback: if the
library is missing or fails to load, importing an operation raises."""
import ctypes
import os
from ctypes import POINTER, Structure, c_double, c_int32, c_int64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcomet_b200.so")


class MemRef1D(Structure):
    """StridedMemRefType<T,1>; same field order as cometpy's memref_i64/f64
    (frontends/numpy-scipy/cometpy/MLIRGen/utils.py:5-21)."""
    _fields_ = [("allocated", c_void_p), ("aligned", c_void_p), ("offset", c_int64),
                ("sizes", c_int64 * 1), ("strides", c_int64 * 1)]


class MemRef2D(Structure):
    _fields_ = [("allocated", c_void_p), ("aligned", c_void_p), ("offset", c_int64),
                ("sizes", c_int64 * 2), ("strides", c_int64 * 2)]


_SPARSE = [c_int32] * 4 + [c_int64, c_void_p] * 10          # formats, 8 index arrays, vals, dims
_MEMREF = [c_int64, c_void_p]

SIGNATURES = {
    # layer 1: host memref descriptors
    "comet_b200_spmv_f64_i64": (None, _SPARSE + _MEMREF * 2 + [c_int32, c_int32]),
    "comet_b200_spmm_f64_i64": (None, _SPARSE + _MEMREF * 2 + [c_int32, c_int32]),
    "comet_b200_sddmm_f64_i64": (None, _SPARSE + _MEMREF * 2 + _SPARSE),
    "comet_b200_dense_times_sparse_f64_i64": (None, _MEMREF + _SPARSE + _MEMREF + [c_int32, c_int32]),
    "comet_b200_elews_mul_sparse_dense_f64_i64": (None, _SPARSE + _MEMREF + _SPARSE),
    "comet_b200_elews_mul_sparse_dense_to_dense_f64_i64": (None, _SPARSE + _MEMREF * 2),
    "comet_b200_spgemm_symbolic_f64_i64": (c_int64, _SPARSE * 3 + [c_int32, c_int32] + _MEMREF * 2),
    "comet_b200_spgemm_numeric_f64_i64": (None, [c_int64] + _MEMREF * 2),
    "comet_b200_elews_mul_sparse_sparse_symbolic_f64_i64": (c_int64, _SPARSE * 2 + _MEMREF * 2),
    "comet_b200_transpose_2D_f64_i64": (None, ([c_int32] * 4 + [c_int64, c_void_p] * 9) * 2 + _MEMREF),
    "comet_b200_read_input_sizes_2D_f64": (None, [c_int32] * 5 + _MEMREF + [c_int32]),
    "comet_b200_read_input_2D_f64_i64": (None, [c_int32] * 5 + [c_int64, c_void_p] * 9 + [c_int32]),
    "comet_b200_handle_destroy": (None, [c_int64]),
    "comet_b200_masked_spgemm_count_f64_i64": (None, _SPARSE * 3 + [c_int32, c_int32] + _MEMREF),
    # several GPUs: communicator, sharded host entry points, device-layer collectives
    "comet_b200_comm_unique_id": (c_int32, [c_void_p, c_int64]),
    "comet_b200_comm_init": (c_int32, [c_int32, c_int32, c_void_p]),
    "comet_b200_comm_nranks": (c_int32, []),
    "comet_b200_comm_rank": (c_int32, []),
    "comet_b200_comm_destroy": (c_int32, []),
    "comet_b200_comm_slice_bytes": (c_int64, [c_int64, c_int32]),
    "comet_b200_spmm_sharded_f64_i64": (None, _SPARSE + _MEMREF * 2 + [c_int32, c_int32]),
    "comet_b200_sddmm_sharded_f64_i64": (None, _SPARSE + _MEMREF * 2 + _SPARSE),
    "comet_b200_spgemm_symbolic_sharded_f64_i64": (c_int64, _SPARSE * 3 + [c_int32, c_int32] + _MEMREF * 2),
    "comet_b200_masked_spgemm_count_sharded_f64_i64": (None, _SPARSE * 3 + [c_int32, c_int32] + _MEMREF),
    "comet_b200_dev_allreduce_sum_i64": (c_int32, [c_void_p, c_int64, c_void_p]),
    "comet_b200_dev_allgather_i64": (c_int32, [c_void_p, c_void_p, c_void_p]),
    "comet_b200_dev_allgather_slices": (c_int32, [c_void_p, c_int64, c_void_p]),
    "comet_b200_last_error": (ctypes.c_char_p, []),
    "comet_b200_set_error_mode": (None, [c_int32]),
    "comet_b200_version": (c_int32, []),
    "comet_b200_release_scratch": (None, []),
    # layer 2: device pointers
    "comet_b200_dev_spmv_f64_i64": (c_int32, [c_int64, c_int64] + [c_void_p] * 6 + [c_int32, c_int32, c_void_p]),
    "comet_b200_dev_spmm_f64_i64": (c_int32, [c_int64] * 4 + [c_void_p] * 5 + [c_int64, c_void_p, c_int64,
                                              c_int32, c_int32, c_int32, c_void_p]),
    "comet_b200_dev_spmm_noalloc_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 5 + [c_int64, c_void_p, c_int64,
                                                      c_int32, c_int32, c_void_p]),
    "comet_b200_dev_dense_times_sparse_f64_i64": (c_int32, [c_int64] * 4 + [c_void_p] * 5 + [c_int64, c_void_p, c_int64,
                                                            c_int32, c_int32, c_void_p]),
    "comet_b200_dev_sddmm_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 4 + [c_int64, c_void_p, c_int64,
                                               c_void_p, c_void_p]),
    "comet_b200_dev_transpose_f64": (c_int32, [c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "comet_b200_dev_sort_coo_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 7),
    "comet_b200_dev_coo_to_csr_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 7),
    "comet_b200_dev_csr_transpose_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 7),
    "comet_b200_dev_elews_mul_sparse_dense_f64_i64": (c_int32, [c_int64, c_int64] + [c_void_p] * 5 +
                                                      [c_int64, c_void_p, c_void_p]),
    "comet_b200_dev_elews_mul_sparse_dense_to_dense_f64_i64": (c_int32, [c_int64, c_int64] + [c_void_p] * 6 +
                                                               [c_int64, c_void_p, c_int64, c_void_p]),
    "comet_b200_dev_spgemm_symbolic_f64_i64": (c_int32, [c_int64] * 3 + [c_void_p] * 8 + [c_int32, c_void_p,
                                                         POINTER(c_int64), POINTER(c_int64), c_void_p]),
    "comet_b200_dev_elews_mul_sparse_sparse_symbolic_f64_i64": (c_int32, [c_int64] + [c_void_p] * 7 +
                                                                [POINTER(c_int64), POINTER(c_int64), c_void_p]),
    "comet_b200_dev_spgemm_numeric_f64_i64": (c_int32, [c_int64, c_void_p, c_void_p, c_int32, c_void_p]),
    "comet_b200_dev_masked_spgemm_count_f64_i64": (c_int32, [c_int64] * 6 + [c_void_p] * 7 + [c_void_p]),
    "comet_b200_dev_noop": (c_int32, [c_void_p]),
    "comet_b200_dev_gather_probe_f64_i64": (c_int32, [c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int32,
                                                      c_void_p, c_int64, c_void_p]),
}

# cometpy's calling convention (_mlir_ciface_<kernel>): result pointers first, a CSR input as seven arguments
_CI_CSR = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p]
for _w in ("i64", "i32"):
    SIGNATURES.update({
        "_mlir_ciface_comet_b200_spmv_csr_f64_" + _w: (None, [c_void_p] + _CI_CSR + [c_void_p]),
        "_mlir_ciface_comet_b200_spmm_csr_f64_" + _w: (None, [c_void_p] + _CI_CSR + [c_void_p]),
        "_mlir_ciface_comet_b200_spgemm_csr_f64_" + _w: (None, [c_void_p] + _CI_CSR * 2 + [c_int64]),
        "_mlir_ciface_comet_b200_spgemm_masked_csr_f64_" + _w: (None, [c_void_p] + _CI_CSR * 3 + [c_int64]),
        "_mlir_ciface_comet_b200_masked_count_csr_f64_" + _w: (c_double, _CI_CSR * 3),
        "_mlir_ciface_comet_b200_sddmm_csr_f64_" + _w: (None, [c_void_p] + _CI_CSR + [c_void_p, c_void_p]),
    })
SIGNATURES["comet_b200_ciface_free"] = (None, [c_void_p])

# the host entry points exist once per index width
for _name in [n for n in SIGNATURES if n.endswith("_f64_i64") and "_dev_" not in n and not n.startswith("_mlir")]:
    SIGNATURES[_name[:-4] + "_i32"] = SIGNATURES[_name]

# float-valued forms of the main host entry points
for _op in ("spmv", "spmm", "sddmm", "spgemm_symbolic", "spgemm_numeric"):
    for _w in ("i64", "i32"):
        SIGNATURES["comet_b200_%s_f32_%s" % (_op, _w)] = SIGNATURES["comet_b200_%s_f64_i64" % _op]

_lib = None


class CometB200Error(RuntimeError):
    pass


def load():
    """Returns the loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CometB200Error(
                "libcomet_b200.so is missing (%s). Build it with `python -m comet_b200.build`; "
                "there is no CPU fallback." % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        # Python callers want exceptions, not exit(1)
        lib.comet_b200_set_error_mode(1)
        _lib = lib
    return _lib


def check(status=0):
    """Raises if the last call reported an error."""
    msg = load().comet_b200_last_error()
    if msg:
        raise CometB200Error(msg.decode())
    if status:
        raise CometB200Error("libcomet_b200 call failed with status %d" % status)
