"""Parity at the full sizes of the five benchmark configurations.

Where the CPU oracle finishes in seconds (SpMV, SpMM, SDDMM) the whole result is
compared.  For SpGEMM (2.9e9 products, 1.28e9 output entries) and triangle
counting (5.8e10 probes) the oracle would run for minutes, so the result is
checked through properties that do not depend on size -- row pointers
monotone, columns strictly ascending inside a row, row sums of C equal to
A*(B*1), additivity of the count over row blocks -- and bit-exactly against
the oracle on row samples."""
import numpy as np
import pytest
import torch

import comet_b200.device as dev
from comet_b200 import datasets, sharding
from oracle import oracle

pytestmark = pytest.mark.gpu

RTOL = 1e-12


def _orc(t):
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, t.val)


def _abs(t):
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, np.abs(t.val))


def _assert_close(got, ref, scale):
    err = np.abs(got - ref)
    bound = RTOL * np.maximum(np.abs(ref), scale)
    assert (err <= bound).all(), float((err / np.maximum(bound, 1e-300)).max() * RTOL)


def test_spmv_config1_full():
    A, x = datasets.config_spmv()
    assert A.nrows == 16384 and A.nnz == 262144
    y = dev.spmv(dev.to_device(A), torch.from_numpy(x).cuda()).cpu().numpy()
    _assert_close(y, oracle.spmv(_orc(A), x), oracle.spmv(_abs(A), np.abs(x)))


def test_spmm_config2_full():
    A, B = datasets.config_spmm()
    assert A.nrows == 1 << 20 and B.shape == (1 << 20, 128)
    dA, dB = dev.to_device(A), torch.from_numpy(B).cuda()
    C = dev.spmm(dA, dB)
    ref = oracle.spmm(_orc(A), B)
    scale = oracle.spmm(_abs(A), np.abs(B))
    _assert_close(C.cpu().numpy(), ref, scale)
    d_scale = torch.from_numpy(scale).cuda()
    del ref, scale
    # linearity: A*(2B) == 2*(A*B); scaling by two is exact, so only the order of the atomic
    # additions on long rows can differ
    C2 = dev.spmm(dA, dB * 2.0)
    assert bool(((C2 - 2.0 * C).abs() <= RTOL * 2.0 * torch.maximum(C.abs(), d_scale)).all())


def test_sddmm_config3_full():
    S, X, Y = datasets.config_sddmm()
    assert S.nrows == 1 << 18 and X.shape == (1 << 18, 64)
    out = dev.sddmm(dev.to_device(S), torch.from_numpy(X).cuda(), torch.from_numpy(Y).cuda()).cpu().numpy()
    _assert_close(out, oracle.sddmm(_orc(S), X, Y), oracle.sddmm(_abs(S), np.abs(X), np.abs(Y)))


def test_spgemm_config4_full_properties_and_row_samples():
    A = datasets.config_spgemm()
    assert A.nrows == 1 << 18
    dA = dev.to_device(A)
    C = dev.spgemm(dA, dA)
    pos = C.pos.cpu().numpy()
    assert pos[0] == 0 and pos[-1] == C.nnz and np.all(np.diff(pos) >= 0)
    assert C.nnz > 1_000_000_000
    # columns strictly ascending inside every row (checked on the device: 10 GB of coordinates)
    d = C.crd[1:] - C.crd[:-1]
    row_starts = torch.zeros(C.nnz, dtype=torch.bool, device="cuda")
    starts = C.pos[1:-1]
    row_starts[starts[starts < C.nnz]] = True
    assert bool(((d > 0) | row_starts[1:]).all())
    assert int(C.crd.min()) >= 0 and int(C.crd.max()) < A.ncols
    del d, row_starts
    # row sums: C*1 == A*(B*1)
    ones = torch.ones(A.ncols, dtype=torch.float64, device="cuda")
    dC = dev.DeviceCSR(A.nrows, A.ncols, C.pos, C.crd, C.val)
    lhs = dev.spmv(dC, ones)
    rhs = dev.spmv(dA, dev.spmv(dA, ones))
    assert float(((lhs - rhs).abs() / rhs.abs().clamp_min(1e-300)).max()) < 1e-11
    # bit-exact structure and 1e-12 values against the oracle on sampled row blocks (light and heavy)
    oa = _orc(A)
    for lo, hi in ((0, 40), (1000, 1400), (131072, 133000), (262000, 262144)):
        ref = oracle.spgemm(_orc(sharding.take_rows(A, lo, hi)), oa)
        s, e = int(pos[lo]), int(pos[hi])
        assert np.array_equal(pos[lo:hi + 1] - s, ref.a2pos)
        assert np.array_equal(C.crd[s:e].cpu().numpy(), ref.a2crd)
        got = C.val[s:e].cpu().numpy()
        assert np.all(np.abs(got - ref.val) <= RTOL * np.abs(ref.val))      # all terms are positive here


def test_triangles_config5_full_additivity_and_row_samples():
    L = datasets.config_triangles()
    assert L.nrows == 1 << 22
    dL = dev.to_device(L)
    total = int(dev.masked_pair_count(dL, dL, dL).item())
    assert total > 0
    # additivity over contiguous row blocks (the multi-GPU split) and repeatability
    bounds = sharding.row_blocks(L.a2pos, 4, weights=sharding.product_weights(L, L))
    parts = [int(dev.masked_pair_count(dL, dL, dL, int(bounds[i]), int(bounds[i + 1])).item()) for i in range(4)]
    assert sum(parts) == total
    assert int(dev.masked_pair_count(dL, dL, dL).item()) == total
    # exact agreement with the oracle on row ranges (short and long mask rows)
    ol = _orc(L)
    for lo, hi in ((0, 3000), (500000, 500400), (4190000, 4190040)):
        want = oracle.masked_pair_count(ol, ol, ol, lo, hi)
        assert int(dev.masked_pair_count(dL, dL, dL, lo, hi).item()) == want
