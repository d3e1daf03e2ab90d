#!/usr/bin/env python3
"""Benchmark of the sparse hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload spmm|spmv|sddmm|spgemm|triangles]
                    [--configs all|headline] [--impl reference] [--scale S] [--probe gather]

Headline workload: SpMM C = A*B, A = R-MAT scale 20 / edge factor 16 (CSR, int64
indices), B dense 1,048,576 x 128 float64 -- the second benchmark configuration.
One step = one pass of the operation over the whole matrix.  With N > 1 (one
process per GPU under torch.distributed.run) the rows of the sparse operand are
split into N contiguous blocks of equal measured work, the other operand is
replicated, and the step ends with the operation's collective where it has one.

Prints ONE JSON line.  `value` is GFLOP/s with operands resident in HBM; `e2e`
is the same metric through the host-memref entry point of the C ABI with
pinned host buffers (uploads and the download of the result inside the timed
region; with N > 1 the sharded entry points, where every rank uploads one N-th
of the replicated operand and the slices cross NVLink); `e2e_pageable` is the
same call on plain (malloc'ed) host arrays, which is what COMET's generated code
holds; `roofline` compares compulsory bytes / time with the measured HBM copy
rate; `cpu_baseline` times the CPU oracle (COMET's generated loop nest,
restated) on this host's cores.  `configs` carries the same measurements for
the other four benchmark configurations.  After the timed region every rank
compares its block of the result with the CPU oracle on sampled rows
(`parity_checked`); a mismatch ends the run with a non-zero exit code.
`--impl reference` times only the CPU path of the headline workload.
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
RTOL = 1e-12


# DRAM traffic of one step (dram__bytes_read.sum + dram__bytes_write.sum over the step's kernels, one-pass ncu
# capture at the full workload on one GPU) is kept in profiles/dram_traffic.json together with a hash of the
# kernel sources it was taken from; it is reported only while those sources are unchanged.
KERNEL_SOURCES = {
    "spmm": ["spmm_stream.cu", "stream.cuh", "spmm.cu"],
    "sddmm": ["sddmm.cu"],
    "spgemm": ["spgemm.cu", "util.cu"],
    "triangles": ["tc.cu"],
}


def kernel_source_hash(name):
    import hashlib
    h = hashlib.sha256()
    for f in KERNEL_SOURCES.get(name, []):
        with open(os.path.join(ROOT, "comet_b200", "csrc", f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def recorded_traffic(name, default_size):
    if not default_size or name not in KERNEL_SOURCES:
        return None
    try:
        with open(os.path.join(ROOT, "profiles", "dram_traffic.json")) as f:
            rec = json.load(f).get(name)
        if rec and rec.get("kernel_source_hash") == kernel_source_hash(name):
            return float(rec["dram_bytes_per_step"])
    except Exception:
        pass
    return None


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML while the GPU is under load."""

    def __init__(self, index, period=0.01):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def _orc(t):
    from oracle import oracle
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, t.val)


def _orc_abs(t):
    from oracle import oracle
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, np.abs(t.val))


def _within(got, ref, scale):
    got, ref, scale = np.asarray(got), np.asarray(ref), np.asarray(scale)
    return got.shape == ref.shape and bool((np.abs(got - ref) <= RTOL * np.maximum(np.abs(ref), scale)).all())


def _sample_rows(pos, count, seed=0):
    """Row numbers for the parity sample: the longest row, the first and last rows, and random ones."""
    n = pos.shape[0] - 1
    if n <= count:
        return np.arange(n, dtype=np.int64)
    rng = np.random.default_rng(seed)
    lens = np.diff(pos)
    pick = set(rng.integers(0, n, count).tolist()) | {0, n - 1, int(np.argmax(lens))}
    pick |= set(np.argsort(lens)[-4:].tolist())
    return np.array(sorted(pick), dtype=np.int64)


def _stack_rows(A, rows):
    """CSR made of the given rows of A (in that order)."""
    from comet_b200.api import SparseTensor
    lens = (A.a2pos[rows + 1] - A.a2pos[rows]).astype(np.int64)
    pos = np.zeros(rows.shape[0] + 1, dtype=np.int64)
    np.cumsum(lens, out=pos[1:])
    idx = np.concatenate([np.arange(A.a2pos[r], A.a2pos[r + 1]) for r in rows]) if rows.shape[0] else np.zeros(0, np.int64)
    idx = idx.astype(np.int64)
    return SparseTensor("CSR", rows.shape[0], A.ncols, np.array([rows.shape[0]], dtype=np.int64),
                        np.array([-1], dtype=np.int64), pos, A.a2crd[idx], A.val[idx]), idx


def _pin(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()


def _host_csr(torch, block, pinned):
    from comet_b200.api import SparseTensor
    f = (lambda a: _pin(torch, a)) if pinned else (lambda a: np.array(a, copy=True))
    return SparseTensor("CSR", block.nrows, block.ncols, block.a1pos, block.a1crd, f(block.a2pos), f(block.a2crd),
                        f(block.val))


def _host_empty(torch, shape, dtype, pinned):
    if pinned:
        tdt = {np.float64: torch.float64, np.int64: torch.int64}[dtype]
        return torch.empty(shape, dtype=tdt, pin_memory=True).numpy()
    a = np.empty(shape, dtype=dtype)
    a.fill(0)          # touch the pages: a first-touch page fault is not part of the operation
    return a


# ---------------------------------------------------------------------------
# Workloads.  Each one knows its data, its device step, its collective, its end-to-end call through the
# host-memref entry points (plain on one GPU, sharded on several), its parity sample and its CPU legs.
# ---------------------------------------------------------------------------
class Workload:
    name = ""
    launches_per_step = 0
    gather_bytes_per_entry = 0          # no-reuse gather model: extra bytes per stored entry / product / probe

    def __init__(self, args):
        self.args = args
        self.world, self.rank = 1, 0

    def place(self, bounds, torch, dev, sharding):
        """(Re)cut: this rank's rows are bounds[rank] .. bounds[rank + 1]."""
        self.bounds = bounds
        self.row_lo, self.row_hi = int(bounds[self.rank]), int(bounds[self.rank + 1])
        self.block = sharding.take_rows(self.A, self.row_lo, self.row_hi) if self.world > 1 else self.A
        self.to_device(self.block, torch, dev)

    def run_steps(self, n, dev, sharding, with_collective=True):
        for _ in range(n):
            self.step(dev)
            if with_collective:
                self.finish_step(sharding)

    def finish_step(self, sharding):
        pass

    def lib(self):
        from comet_b200 import _lib
        return _lib.load()

    def entry(self, name):
        return getattr(self.lib(), "comet_b200_%s%s_f64_i64" % (name, "_sharded" if self.world > 1 else ""))

    def cpu_alt(self):
        return None

    def e2e_weights(self):
        """Per-row bytes that cross PCIe in the end-to-end call (None: keep the kernel-balanced blocks).
        Through the host entry points the transfer, not the kernel, is what a rank spends its time on, so
        the host program cuts its row blocks for equal bytes there."""
        return None


class SpMM(Workload):
    name = "spmm"
    launches_per_step = 2     # plan kernel + entry-stream kernel
    gather_bytes_per_entry = None

    def build(self):
        from comet_b200 import datasets
        a = self.args
        scale = a.scale or 20
        self.k = a.k or 128
        self.A, self.B = datasets.config_spmm(scale=scale, edge_factor=16, k=self.k)
        self.desc = "SpMM C=A*B f64/i64, A = R-MAT scale %d ef 16 dedup (%d nnz) CSR, B %d x %d" % (
            scale, self.A.nnz, self.A.ncols, self.k)
        self.flops = 2.0 * self.A.nnz * self.k
        self.bytes = datasets.algorithmic_bytes("spmm", self.A.nrows, self.A.ncols, self.A.nnz, k=self.k)
        self.replicated_bytes = 8 * self.A.ncols * self.k
        self.gather_model_bytes = self.bytes + 8.0 * self.A.nnz * self.k
        # first cut: one gathered B row per stored entry plus one written C row (and its row pointer) per row
        self.weights = (np.diff(self.A.a2pos) + 2).astype(np.float64)

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        if getattr(self, "dB", None) is None:
            self.dB = torch.from_numpy(self.B).cuda()
        self.dC = torch.empty((block.nrows, self.k), dtype=torch.float64, device="cuda")

    def step(self, dev):
        dev.spmm(self.dA, self.dB, self.dC, variant=self.args.variant)

    def e2e_weights(self):
        return 16.0 * np.diff(self.A.a2pos) + 8.0 * self.k + 8.0      # the row's entries up, its row of C down

    def check(self, torch, dev):
        from oracle import oracle
        rows = _sample_rows(self.block.a2pos, 256, seed=self.rank)
        sub, _ = _stack_rows(self.block, rows)
        got = self.dC[torch.from_numpy(rows).cuda()].cpu().numpy()
        return _within(got, oracle.spmm(_orc(sub), self.B), oracle.spmm(_orc_abs(sub), np.abs(self.B)))

    def e2e_setup(self, torch, pinned):
        self.hA = _host_csr(torch, self.block, pinned)
        self.hB = _pin(torch, self.B) if pinned else self.B
        self.hC = _host_empty(torch, (self.block.nrows, self.k), np.float64, pinned)
        up = self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hB.nbytes // self.world
        return up, self.hC.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        pk = _Packer()
        self.entry("spmm")(*pk.sparse(self.hA), *pk.m2(self.hB), *pk.m2(self.hC), 0, 0)
        _lib.check()

    def e2e_check(self):
        from oracle import oracle
        rows = _sample_rows(self.block.a2pos, 64, seed=100 + self.rank)
        sub, _ = _stack_rows(self.block, rows)
        return _within(self.hC[rows], oracle.spmm(_orc(sub), self.B), oracle.spmm(_orc_abs(sub), np.abs(self.B)))

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload (all %d rows), %d columns" % (self.A.nrows, self.k)

    def cpu_step(self):
        from oracle import oracle
        oracle.spmm(self.oA, self.B)


class SpMV(Workload):
    name = "spmv"
    launches_per_step = 1     # one kernel below 2^20 stored entries, two (rows + long-row chunks) above

    def build(self):
        from comet_b200 import datasets
        n = 1 << (self.args.scale or 14)
        self.A, self.x = datasets.config_spmv(n=n, per_row=16)
        self.desc = "SpMV y=A*x f64/i64, A %dx%d CSR 16 per row (%d nnz)" % (n, n, self.A.nnz)
        self.flops = 2.0 * self.A.nnz
        self.bytes = datasets.algorithmic_bytes("spmv", self.A.nrows, self.A.ncols, self.A.nnz)
        self.replicated_bytes = 8 * self.A.ncols
        self.gather_model_bytes = self.bytes + 8.0 * self.A.nnz
        self.weights = (np.diff(self.A.a2pos) + 1).astype(np.float64)

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        self.dx = torch.from_numpy(self.x).cuda()
        self.torch = torch
        self.graphs = {}
        if self.world == 1:
            self.dy = torch.empty(block.nrows, dtype=torch.float64, device="cuda")
        else:
            # y blocks are exchanged in place: one buffer of `world` equal slices (the longest block, rounded up to
            # 256 bytes), every rank's kernel writes its slice, the library's all-gather fills in the others
            longest = max(int(self.bounds[r + 1] - self.bounds[r]) for r in range(self.world))
            self.slice_elems = (longest * 8 + 255) // 256 * 32
            self.ybuf = torch.zeros(self.world * self.slice_elems, dtype=torch.float64, device="cuda")
            self.dy = self.ybuf[self.rank * self.slice_elems:self.rank * self.slice_elems + block.nrows]

    def run_steps(self, n, dev, sharding, with_collective=True):
        # One SpMV at this size is shorter than a kernel launch from the host, so on one GPU
        # the n steps are captured once into a CUDA graph (n back-to-back SpMVs) and replayed.
        if self.world > 1:
            return Workload.run_steps(self, n, dev, sharding, with_collective)
        torch = self.torch
        if n not in self.graphs:
            dev.spmv(self.dA, self.dx, self.dy)          # library set-up outside the capture
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(n):
                    dev.spmv(self.dA, self.dx, self.dy)
            self.graphs[n] = g
        self.graphs[n].replay()

    def step(self, dev):
        dev.spmv(self.dA, self.dx, self.dy)

    def latency_table(self, dev):
        """Per-call time of back-to-back SpMVs replayed from a CUDA graph of 1, 10 and 1000 calls, and of the
        same graphs filled with EMPTY kernels: the floor set by launching, not by the kernel."""
        torch = self.torch
        lib = self.lib()
        out = {}

        def timed(fill, n):
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(n):
                    fill()
            for _ in range(3):
                g.replay()
            reps = max(3, 2000 // n)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / (reps * n)

        noop = lambda: lib.comet_b200_dev_noop(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        for n in (1, 10, 1000):
            out["calls_%d" % n] = {"spmv_us_per_call": timed(lambda: dev.spmv(self.dA, self.dx, self.dy), n),
                                   "empty_kernel_us_per_call": timed(noop, n)}
        return out

    def finish_step(self, sharding):
        if self.world > 1:
            from comet_b200 import _lib
            st = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
            _lib.check(self.lib().comet_b200_dev_allgather_slices(ctypes.c_void_p(self.ybuf.data_ptr()),
                                                                  self.slice_elems * 8, st))

    def check(self, torch, dev):
        from oracle import oracle
        ref = oracle.spmv(_orc(self.block), self.x)
        ok = _within(self.dy.cpu().numpy(), ref, oracle.spmv(_orc_abs(self.block), np.abs(self.x)))
        if self.world > 1:      # the gathered vector: every rank's slice, cut to its block length
            buf = self.ybuf.cpu().numpy()
            parts = [buf[r * self.slice_elems:r * self.slice_elems + int(self.bounds[r + 1] - self.bounds[r])]
                     for r in range(self.world)]
            full = oracle.spmv(_orc(self.A), self.x)
            ok = ok and _within(np.concatenate(parts), full, oracle.spmv(_orc_abs(self.A), np.abs(self.x)))
        return ok

    def e2e_setup(self, torch, pinned):
        self.hA = _host_csr(torch, self.block, pinned)
        self.hx = _pin(torch, self.x) if pinned else self.x
        self.hy = _host_empty(torch, (self.block.nrows,), np.float64, pinned)
        return self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hx.nbytes, self.hy.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        pk = _Packer()
        # no sharded form: the vector is 128 KB, every rank passes all of it with its block of A
        self.lib().comet_b200_spmv_f64_i64(*pk.sparse(self.hA), *pk.m1(self.hx), *pk.m1(self.hy), 0, 0)
        _lib.check()

    def e2e_check(self):
        from oracle import oracle
        return _within(self.hy, oracle.spmv(_orc(self.block), self.x), oracle.spmv(_orc_abs(self.block), np.abs(self.x)))

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload"

    def cpu_step(self):
        from oracle import oracle
        oracle.spmv(self.oA, self.x)


class SDDMM(Workload):
    name = "sddmm"
    launches_per_step = 2     # short-row stream kernel + long-row chunk kernel

    def build(self):
        from comet_b200 import datasets
        scale = self.args.scale or 18
        self.k = self.args.k or 64
        self.A, self.X, self.Y = datasets.config_sddmm(scale=scale, edge_factor=32, k=self.k)
        self.desc = "SDDMM C=S.*(X*Y^T) f64/i64, S = R-MAT scale %d ef 32 dedup (%d nnz) CSR, K=%d" % (
            scale, self.A.nnz, self.k)
        self.flops = float(self.A.nnz) * (2 * self.k + 1)
        self.bytes = datasets.algorithmic_bytes("sddmm", self.A.nrows, self.A.ncols, self.A.nnz, k=self.k)
        self.replicated_bytes = 8 * self.A.ncols * self.k
        self.gather_model_bytes = self.bytes + 8.0 * self.A.nnz * self.k
        self.weights = (np.diff(self.A.a2pos) + 1).astype(np.float64)   # one gathered Y row per entry, one X row per row

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        lo = self.row_lo
        self.dX = torch.from_numpy(np.ascontiguousarray(self.X[lo:lo + block.nrows])).cuda()
        if getattr(self, "dY", None) is None:
            self.dY = torch.from_numpy(self.Y).cuda()
        self.dout = torch.empty(block.nnz, dtype=torch.float64, device="cuda")

    def step(self, dev):
        dev.sddmm(self.dA, self.dX, self.dY, self.dout)

    def e2e_weights(self):
        return 24.0 * np.diff(self.A.a2pos) + 8.0 * self.k + 8.0      # entries up, values down, the row of X up

    def _check_vals(self, vals, seed):
        from oracle import oracle
        rows = _sample_rows(self.block.a2pos, 256, seed=seed)
        sub, idx = _stack_rows(self.block, rows)
        Xs = self.X[self.row_lo + rows]
        return _within(vals[idx], oracle.sddmm(_orc(sub), Xs, self.Y), oracle.sddmm(_orc_abs(sub), np.abs(Xs), np.abs(self.Y)))

    def check(self, torch, dev):
        return self._check_vals(self.dout.cpu().numpy(), self.rank)

    def e2e_setup(self, torch, pinned):
        from comet_b200.api import SparseTensor
        block = self.block
        self.hA = _host_csr(torch, block, pinned)
        self.hO = SparseTensor("CSR", block.nrows, block.ncols, np.zeros_like(block.a1pos), np.zeros_like(block.a1crd),
                               np.zeros_like(block.a2pos), np.zeros_like(block.a2crd),
                               _host_empty(torch, (block.nnz,), np.float64, pinned))
        lo = self.row_lo
        Xb = self.X[lo:lo + block.nrows]
        self.hX = _pin(torch, Xb) if pinned else np.array(Xb, copy=True)
        self.hY = _pin(torch, self.Y) if pinned else self.Y
        h2d = (self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hX.nbytes
               + self.hY.nbytes // self.world)
        return h2d, self.hO.val.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        pk = _Packer()
        self.entry("sddmm")(*pk.sparse(self.hA), *pk.m2(self.hX), *pk.m2(self.hY, transposed_view=True),
                            *pk.sparse(self.hO))
        _lib.check()

    def e2e_check(self):
        return self._check_vals(self.hO.val, 100 + self.rank)

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload, O(nnz*K) form (COMET's fused loop computes full dense rows and is not runnable at this size)"

    def cpu_step(self):
        from oracle import oracle
        oracle.sddmm(self.oA, self.X, self.Y)


def _tail_sample(weights, fraction):
    """First row of the tail of the matrix that holds about `fraction` of the total weight."""
    cum = np.concatenate([[0], np.cumsum(weights)])
    target = cum[-1] - cum[-1] * fraction
    lo = int(np.searchsorted(cum, target))
    return lo, float(cum[-1] - cum[lo])


class SpGEMM(Workload):
    name = "spgemm"
    launches_per_step = 9     # narrow, bin, hash+bitmap symbolic, 3 scan kernels, hash+bitmap numeric

    def build(self):
        from comet_b200 import datasets, sharding
        scale = self.args.scale or 18
        self.A = datasets.config_spgemm(scale=scale, edge_factor=16)
        self.weights = sharding.product_weights(self.A, self.A).astype(np.float64) + 1.0
        self.products = int(self.weights.sum() - self.A.nrows)
        self.desc = "SpGEMM C=A*A f64/i64 Gustavson, A = R-MAT scale %d ef 16 dedup (%d nnz, %d products) CSR" % (
            scale, self.A.nnz, self.products)
        self.flops = 2.0 * self.products
        self.bytes = None     # needs nnz(C); filled after the first step
        self.replicated_bytes = 8 * (self.A.nrows + 1) + 16 * self.A.nnz

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        if getattr(self, "dB", None) is None:
            self.dB = dev.to_device(self.A)
        self.torch = torch
        self.nnz_c = None
        self.crd = self.val = None
        self.one = torch.zeros(1, dtype=torch.int64, device="cuda")
        self.all = torch.zeros(self.world, dtype=torch.int64, device="cuda")

    def step(self, dev):
        h, self.cpos, nnz = dev.spgemm_symbolic(self.dA, self.dB)
        if self.crd is None or self.crd.shape[0] != nnz:
            self.crd = self.val = None
            self.crd = self.torch.empty(max(nnz, 1), dtype=self.torch.int64, device="cuda")[:nnz]
            self.val = self.torch.empty(max(nnz, 1), dtype=self.torch.float64, device="cuda")[:nnz]
        dev.spgemm_numeric(h, nnz, "cuda", crd=self.crd, val=self.val)
        self.nnz_c = nnz

    def finish_step(self, sharding):
        if self.world > 1:
            # per-rank entry counts -> this block's place in the whole C (the library's own communicator)
            from comet_b200 import _lib
            self.one.copy_(self.cpos[-1:])
            st = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
            _lib.check(self.lib().comet_b200_dev_allgather_i64(ctypes.c_void_p(self.one.data_ptr()),
                                                               ctypes.c_void_p(self.all.data_ptr()), st))

    def _check_block(self, pos, part, seed):
        """pos: the block's row pointer (host); part(lo, hi): host copies of crd[lo:hi], val[lo:hi]."""
        from oracle import oracle
        from comet_b200 import sharding
        n = self.block.nrows
        rng = np.random.default_rng(seed)
        ok = bool(np.all(np.diff(pos) >= 0)) and pos[0] == 0
        oa = _orc(self.A)
        absa = _orc_abs(self.A)
        starts = sorted(set([0, max(n - 48, 0)] + rng.integers(0, max(n - 48, 1), 3).tolist()))
        for s in starts:
            e = min(s + 48, n)
            sub = sharding.take_rows(self.block, s, e)
            ref = oracle.spgemm(_orc(sub), oa)
            lo, hi = int(pos[s]), int(pos[e])
            crd, val = part(lo, hi)
            ok = ok and np.array_equal(pos[s:e + 1] - lo, ref.a2pos) and np.array_equal(crd, ref.a2crd)
            ok = ok and _within(val, ref.val, oracle.spgemm(_orc_abs(sub), absa).val)
        return bool(ok)

    def check(self, torch, dev):
        ok = self._check_block(self.cpos.cpu().numpy(),
                               lambda lo, hi: (self.crd[lo:hi].cpu().numpy(), self.val[lo:hi].cpu().numpy()), self.rank)
        if self.world > 1:
            counts = self.all.cpu().numpy()
            ok = ok and int(counts[self.rank]) == int(self.nnz_c)
        return ok

    def e2e_setup(self, torch, pinned):
        from comet_b200.api import SparseTensor
        block, A = self.block, self.A
        self.hA = _host_csr(torch, block, pinned)
        self.hB = self.hA if self.world == 1 else SparseTensor(
            "CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, *[(_pin(torch, a) if pinned else a) for a in (A.a2pos, A.a2crd, A.val)])
        self.hpos = _host_empty(torch, (block.nrows + 1,), np.int64, pinned)
        nnz = int(self.nnz_c)
        self.hcrd = _host_empty(torch, (max(nnz, 1),), np.int64, pinned)[:nnz]
        self.hval = _host_empty(torch, (max(nnz, 1),), np.float64, pinned)[:nnz]
        self.sizes = np.zeros(13, dtype=np.int64)
        h2d = self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes
        if self.world > 1:
            h2d += (self.hB.a2pos.nbytes + self.hB.a2crd.nbytes + self.hB.val.nbytes) // self.world
        return h2d, self.hpos.nbytes + self.hcrd.nbytes + self.hval.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = self.lib()
        pk = _Packer()
        h = self.entry("spgemm_symbolic")(*pk.sparse(self.hA), *pk.sparse(self.hB), *pk.sparse(self.hA),
                                          0, 0, *pk.m1(self.hpos), *pk.m1(self.sizes))
        _lib.check()
        lib.comet_b200_spgemm_numeric_f64_i64(h, *pk.m1(self.hcrd), *pk.m1(self.hval))
        _lib.check()

    def e2e_check(self):
        ok = self._check_block(self.hpos, lambda lo, hi: (self.hcrd[lo:hi], self.hval[lo:hi]), 100 + self.rank)
        if self.world > 1:
            ok = ok and int(self.sizes[12]) == int(self.total_nnz_c)
        return ok

    def cpu_setup(self):
        from comet_b200 import sharding
        # bounded sample: the last rows holding ~1/64 of the products (single thread, like COMET's
        # sequential loops for sparse outputs)
        lo, w = _tail_sample(self.weights - 1.0, 1.0 / 64)
        self.sample = sharding.take_rows(self.A, lo, self.A.nrows)
        self.oS, self.oA = _orc(self.sample), _orc(self.A)
        self.cpu_flops = 2.0 * w
        return "rows %d..%d of A (%d of %d products), symbolic + numeric + sort, 1 thread" % (
            lo, self.A.nrows, int(w), self.products)

    def cpu_step(self):
        from oracle import oracle
        oracle.spgemm(self.oS, self.oA)

    def cpu_alt(self):
        from comet_b200 import sharding
        from oracle import oracle
        lo, w = _tail_sample(self.weights - 1.0, 1.0 / 8)
        sample = _orc(sharding.take_rows(self.A, lo, self.A.nrows))
        oa = _orc(self.A)
        return (lambda: oracle.spgemm_rowparallel(sample, oa)), 2.0 * w, "rows %d..%d of A (%d products)" % (
            lo, self.A.nrows, int(w))


class Triangles(Workload):
    name = "triangles"
    launches_per_step = 6     # index narrowing, binning, four counting kernels (units, slow rows, CTA rows, warp rows)

    def build(self):
        from comet_b200 import datasets, sharding
        scale = self.args.scale or 22
        self.A = datasets.config_triangles(scale=scale, edge_factor=16)
        self.weights = sharding.product_weights(self.A, self.A).astype(np.float64) + 1.0
        self.probes = int(self.weights.sum() - self.A.nrows)
        self.desc = ("triangle count sum((L*L).*L) plus-pair, L = strict lower of symmetrised R-MAT scale %d ef 16 "
                     "(%d nnz, %d push probes)") % (scale, self.A.nnz, self.probes)
        self.flops = 2.0 * self.probes
        self.bytes = datasets.algorithmic_bytes("triangles", self.A.nrows, self.A.ncols, self.A.nnz)
        self.replicated_bytes = self.bytes
        self.gather_model_bytes = self.bytes + 8.0 * self.probes

    def place(self, bounds, torch, dev, sharding):
        # the counting kernel takes a row range of the full L, which every rank holds: a re-cut moves no data
        self.bounds = bounds
        self.row_lo, self.row_hi = int(bounds[self.rank]), int(bounds[self.rank + 1])
        self.block = None
        if getattr(self, "dL", None) is None:
            self.dL = dev.to_device(self.A)
            self.count = torch.zeros(1, dtype=torch.int64, device="cuda")
            self.torch = torch

    def step(self, dev):
        dev.masked_pair_count(self.dL, self.dL, self.dL, self.row_lo, self.row_hi, out=self.count)

    def finish_step(self, sharding):
        if self.world > 1:
            from comet_b200 import _lib
            st = ctypes.c_void_p(self.torch.cuda.current_stream().cuda_stream)
            _lib.check(self.lib().comet_b200_dev_allreduce_sum_i64(ctypes.c_void_p(self.count.data_ptr()), 1, st))

    def _oracle_range(self, lo, hi):
        from oracle import oracle
        oa = _orc(self.A)
        return oracle.masked_pair_count_rowparallel(oa, oa, oa, lo, hi)

    def check(self, torch, dev):
        # (1) a row range small enough for the CPU (about 1/64 of the probes, inside this rank's block where it can be)
        cum = np.concatenate([[0], np.cumsum(self.weights)])
        budget = cum[-1] / 64
        lo = self.row_lo
        hi = int(np.searchsorted(cum, cum[lo] + budget))
        hi = max(min(hi, self.row_hi), lo + 1)
        got = int(dev.masked_pair_count(self.dL, self.dL, self.dL, lo, hi).item())
        ok = got == self._oracle_range(lo, hi)
        # (2) the count of the sharded step equals the count one GPU finds over all rows
        self.total = int(self.count.item())
        whole = int(dev.masked_pair_count(self.dL, self.dL, self.dL, 0, self.A.nrows).item())
        return ok and (whole == self.total)

    def e2e_setup(self, torch, pinned):
        from comet_b200 import sharding
        from comet_b200.api import SparseTensor
        A = self.A
        p = (lambda a: _pin(torch, a)) if pinned else (lambda a: a)
        self.hB = SparseTensor("CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, p(A.a2pos), p(A.a2crd), A.val)
        if self.world > 1:
            blk = sharding.take_rows(A, self.row_lo, self.row_hi)
            self.hA = SparseTensor("CSR", blk.nrows, blk.ncols, blk.a1pos, blk.a1crd, p(blk.a2pos), p(blk.a2crd), blk.val)
        else:
            self.hA = self.hB
        self.hout = _host_empty(torch, (1,), np.int64, pinned)
        up = self.hB.a2pos.nbytes + self.hB.a2crd.nbytes
        if self.world > 1:
            up = up // self.world + self.hA.a2pos.nbytes + self.hA.a2crd.nbytes
        return up, 8

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        pk = _Packer()
        self.entry("masked_spgemm_count")(*pk.sparse(self.hA), *pk.sparse(self.hB), *pk.sparse(self.hA),
                                          1, 1, *pk.m1(self.hout))
        _lib.check()

    def e2e_check(self):
        return int(self.hout[0]) == int(self.total)

    def cpu_setup(self):
        self.cpu_lo, w = _tail_sample(self.weights - 1.0, 1.0 / 64)
        self.oA = _orc(self.A)
        self.cpu_flops = 2.0 * w
        return "rows %d..%d of L (%d of %d probes), bitmap push mask, 1 thread" % (
            self.cpu_lo, self.A.nrows, int(w), self.probes)

    def cpu_step(self):
        from oracle import oracle
        oracle.masked_pair_count(self.oA, self.oA, self.oA, self.cpu_lo, self.A.nrows)

    def cpu_alt(self):
        from oracle import oracle
        lo, w = _tail_sample(self.weights - 1.0, 1.0 / 8)
        oa = _orc(self.A)
        return (lambda: oracle.masked_pair_count_rowparallel(oa, oa, oa, lo, self.A.nrows)), 2.0 * w, \
            "rows %d..%d of L (%d probes)" % (lo, self.A.nrows, int(w))


WORKLOADS = {w.name: w for w in (SpMM, SpMV, SDDMM, SpGEMM, Triangles)}
ORDER = ["spmm", "spmv", "sddmm", "spgemm", "triangles"]


# ---------------------------------------------------------------------------
def time_cpu(fn, budget_s=20.0, max_reps=3):
    fn()
    t0 = time.perf_counter()
    reps = 0
    while reps < max_reps and (reps == 0 or time.perf_counter() - t0 < budget_s):
        fn()
        reps += 1
    return (time.perf_counter() - t0) / reps


def cpu_baseline(w):
    """The CPU oracle on this host's cores: rows in parallel where COMET's loops are (dense outputs), one
    thread where they are sequential (sparse outputs); for those a second, row-parallel figure that is NOT
    COMET's schedule."""
    from oracle import oracle
    oracle.use_all_cores()
    sample = w.cpu_setup()
    flops = getattr(w, "cpu_flops", w.flops)
    dt = time_cpu(w.cpu_step)
    parallel = w.name in ("spmm", "spmv", "sddmm")
    out = {"value": flops / dt / 1e9, "unit": "GFLOP/s", "cores": oracle.num_threads() if parallel else 1,
           "kind": "port", "sample": sample, "ms": dt * 1e3}
    alt = w.cpu_alt()
    if alt is not None:
        fn, aflops, asample = alt
        adt = time_cpu(fn, budget_s=10.0, max_reps=2)
        out["row_parallel"] = {"value": aflops / adt / 1e9, "unit": "GFLOP/s", "cores": oracle.num_threads(),
                               "sample": asample, "ms": adt * 1e3,
                               "note": "not COMET's schedule: COMET runs sparse-output loops on one thread"}
    return out


def run_reference(args, w, rank):
    """Times the CPU restatement of COMET's loops on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import oracle
    oracle.use_all_cores()
    w.build()
    sample = w.cpu_setup()
    flops = getattr(w, "cpu_flops", w.flops)
    cores = oracle.num_threads() if w.name in ("spmm", "spmv", "sddmm") else 1
    for _ in range(args.warmup):
        w.cpu_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        w.cpu_step()
    dt = (time.perf_counter() - t0) / args.steps
    v = flops / dt / 1e9
    line = {
        "impl": "reference", "metric": "GFLOP/s", "value": v, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": {"workload": w.desc},
        "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


class Env:
    pass


def rebalance(w, env, args):
    """Cuts the rows into blocks of equal MEASURED work.  The first cut balances a model weight per row;
    each round then times one warm-up pass per rank, charges every row of a block with that block's
    measured time per unit of weight, and cuts again; the cut whose slowest rank was fastest is the one
    kept.  Part of set-up, like the first split.  Returns the per-rank times of every round and the
    index of the round whose cut was kept."""
    torch, dist, dev, sharding = env.torch, env.dist, env.dev, env.sharding
    weights = np.asarray(w.weights, dtype=np.float64)
    bounds = sharding.row_blocks(w.A.a2pos, env.world, weights=weights)
    w.place(bounds, torch, dev, sharding)
    history = []
    if env.world == 1:
        return history, 0
    best = None                                            # (slowest rank's time, round, bounds)
    for _ in range(args.rebalance_rounds + 1):
        w.run_steps(2, dev, sharding, with_collective=False)
        torch.cuda.synchronize()
        dist.barrier()
        reps = 3 if w.name in ("spgemm", "triangles") else 30      # short kernels need more repetitions for a steady figure
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        w.run_steps(reps, dev, sharding, with_collective=False)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device="cuda")
        ts = [torch.zeros_like(t) for _ in range(env.world)]
        dist.all_gather(ts, t)
        times = np.array([float(x.item()) for x in ts])
        history.append([round(float(x), 4) for x in times])
        if best is None or times.max() < best[0]:
            best = (float(times.max()), len(history) - 1, np.array(bounds).copy())
        if len(history) > args.rebalance_rounds or times.max() <= 1.04 * times.min():
            break
        cum = np.concatenate([[0.0], np.cumsum(weights)])
        for r in range(env.world):
            lo, hi = int(bounds[r]), int(bounds[r + 1])
            wsum = cum[hi] - cum[lo]
            if wsum > 0:
                # move three quarters of the way to the measured cost per unit of weight: the full step overshoots,
                # because a block's cost per unit changes with the rows it gains or loses
                weights[lo:hi] *= (times[r] / wsum) ** 0.75 * (times.mean() / (cum[-1] / env.world)) ** 0.25
        weights /= weights.sum() / 1e9
        bounds = sharding.row_blocks(w.A.a2pos, env.world, weights=weights)
        w.place(bounds, torch, dev, sharding)
    if best[1] != len(history) - 1:                        # (the times are all-gathered: every rank decides alike)
        w.place(best[2], torch, dev, sharding)
    return history, best[1]


def measure(w, args, env, headline):
    torch, dist, dev, sharding = env.torch, env.dist, env.dev, env.sharding
    world, rank = env.world, env.rank
    w.world, w.rank = world, rank

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    w.build()
    history, kept_round = rebalance(w, env, args)
    w.run_steps(args.warmup, dev, sharding)
    w.run_steps(args.steps, dev, sharding)      # also builds anything cached per step count
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    w.run_steps(args.steps, dev, sharding)
    ev1.record()
    barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps

    # kernel time of this rank's step (no collective), every rank's figure gathered
    if world == 1:
        kernel_ms = ev0.elapsed_time(ev1) / args.steps
        per_rank = [kernel_ms]
    else:
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        w.run_steps(args.steps, dev, sharding, with_collective=False)
        k1.record()
        torch.cuda.synchronize()
        kernel_ms = k0.elapsed_time(k1) / args.steps
        t = torch.tensor([kernel_ms], dtype=torch.float64, device="cuda")
        ts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(ts, t)
        per_rank = [float(x.item()) for x in ts]
        w.run_steps(1, dev, sharding)          # leave the collective's result in place for the check
        barrier()

    if w.bytes is None:   # SpGEMM: output size known after a step
        from comet_b200 import datasets
        nnz_c = torch.tensor([w.nnz_c], dtype=torch.int64, device="cuda")
        if world > 1:
            dist.all_reduce(nnz_c)
        w.total_nnz_c = int(nnz_c.item())
        w.bytes = datasets.algorithmic_bytes("spgemm", w.A.nrows, w.A.ncols, w.A.nnz, nnz_b=w.A.nnz,
                                             nnz_c=w.total_nnz_c, nrows_b=w.A.nrows)
        w.gather_model_bytes = w.bytes + 16.0 * w.products

    # parity of this rank's block against the CPU oracle (outside every timed region)
    ok = bool(w.check(torch, dev))
    kernel_bounds = list(w.bounds)

    # end to end through the host-memref entry points: pinned buffers, then plain ones
    e2e = {}
    e2e_bounds = None
    if not args.kernel_only and world > 1 and w.e2e_weights() is not None:
        e2e_bounds = sharding.row_blocks(w.A.a2pos, world, weights=w.e2e_weights())
        w.place(e2e_bounds, torch, dev, sharding)
    if not args.kernel_only:
        for key, pinned in (("e2e", True), ("e2e_pageable", False)):
            h2d, d2h = w.e2e_setup(torch, pinned)
            w.e2e_step()
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.e2e_steps):
                w.e2e_step()
            barrier()
            dt = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], dtype=torch.float64, device="cuda")
            tot = torch.tensor([h2d, d2h], dtype=torch.int64, device="cuda")
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
                dist.all_reduce(tot, op=dist.ReduceOp.MAX)
            ok = bool(w.e2e_check()) and ok
            e2e[key] = {"value": w.flops / float(dt.item()) / 1e9, "unit": "GFLOP/s",
                        "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()),
                        "ms_per_step": float(dt.item()) * 1e3, "steps": args.e2e_steps,
                        "host_buffers": "pinned" if pinned else "pageable (plain numpy arrays, as malloc gives them)",
                        "bytes_are": "per rank (largest rank)" if world > 1 else "whole job"}
            for name in ("hA", "hB", "hC", "hX", "hY", "hO", "hpos", "hcrd", "hval", "hout", "hx", "hy"):
                if hasattr(w, name):
                    delattr(w, name)

    flag = torch.tensor([1 if ok else 0], dtype=torch.int64, device="cuda")
    if world > 1:
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    parity_ok = bool(flag.item())

    peak, peak_kind = measured_peak()
    # bytes this rank's kernels have to move: its share of the sharded arrays plus ALL of the replicated operand
    rank_bytes = (w.bytes - w.replicated_bytes) / world + w.replicated_bytes
    slowest = max(per_rank)
    achieved = rank_bytes / (slowest * 1e-3) / 1e9
    res = {
        "workload": w.desc, "value": w.flops / (ms_per_step * 1e-3) / 1e9, "unit": "GFLOP/s",
        "ms_per_step": ms_per_step, "steps": args.steps,
        "per_rank_kernel_ms": [round(x, 5) for x in per_rank],
        "parity_checked": parity_ok,
        "gpu_launches": w.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS,
                     "traffic": recorded_traffic(w.name, world == 1 and not args.scale and not args.k and not args.variant),
                     "traffic_source": "profiles/dram_traffic.json (ncu, one GPU, same kernel sources) or null",
                     "peak_kind": peak_kind,
                     "algorithmic_bytes_per_step": int(rank_bytes), "kernel_ms_per_step": slowest,
                     "gather_model_gbs": (w.gather_model_bytes / world) / (slowest * 1e-3) / 1e9,
                     "gather_model_note": "no-reuse model: one dense row fetched per stored entry / product / probe"},
    }
    if world > 1:
        res["rebalance_per_rank_ms"] = history
        res["rebalance_kept_round"] = kept_round
        res["row_bounds"] = [int(b) for b in kernel_bounds]
        if e2e_bounds is not None:
            res["e2e_row_bounds"] = [int(b) for b in e2e_bounds]
            res["e2e_row_bounds_note"] = "the end-to-end leg cuts rows for equal bytes over PCIe, the kernel leg for equal kernel time"
    res.update(e2e)
    if "probes" in w.__dict__:
        res["probes_per_s"] = w.probes / (ms_per_step * 1e-3)
    if hasattr(w, "total_nnz_c"):
        res["nnz_c"] = w.total_nnz_c
    if hasattr(w, "latency_table") and world == 1 and not args.kernel_only:
        res["latency"] = w.latency_table(dev)
    if rank == 0 and world == 1 and not args.no_cpu and not args.kernel_only:
        res["cpu_baseline"] = cpu_baseline(w)
    return res, parity_ok


def probe_gather(args):
    """Ceilings of a gather-per-entry kernel on the SpMM / SDDMM column streams (see probe.cu)."""
    import torch
    from comet_b200 import _lib, datasets
    lib = _lib.load()
    torch.cuda.set_device(0)
    out = torch.zeros(148 * 64 * 8, dtype=torch.float64, device="cuda")
    res = {}
    for name, (A, B) in (("spmm_cfg2", datasets.config_spmm(scale=args.scale or 20, edge_factor=16, k=128)),
                         ("sddmm_cfg3", (lambda t: (t[0], t[2]))(datasets.config_sddmm(scale=min(args.scale or 18, 18),
                                                                                        edge_factor=32, k=64)))):
        crd = torch.from_numpy(A.a2crd).cuda()
        dB = torch.from_numpy(B).cuda()
        k = B.shape[1]
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        for label, fold in (("stream_as_is", 0), ("rows_folded_to_32MB", (32 << 20) // (8 * k))):
            best = None
            for ctas in (2, 4, 8):
                def go():
                    _lib.check(lib.comet_b200_dev_gather_probe_f64_i64(A.nnz, ctypes.c_void_p(crd.data_ptr()),
                                                                       ctypes.c_void_p(dB.data_ptr()), k, k, fold, ctas,
                                                                       ctypes.c_void_p(out.data_ptr()), out.shape[0], st))
                for _ in range(3):
                    go()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    go()
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / 10
                if best is None or ms < best[0]:
                    best = (ms, ctas)
            gathered = 8.0 * k * A.nnz
            res["%s/%s" % (name, label)] = {"ms": best[0], "ctas_per_sm": best[1], "gathered_GB": gathered / 1e9,
                                            "gather_TBps": gathered / (best[0] * 1e-3) / 1e12}
        del crd, dB
    print(json.dumps({"probe": "gather", "results": res}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="spmm", choices=sorted(WORKLOADS))
    ap.add_argument("--configs", default=None, choices=["all", "headline"],
                    help="all: also measure the other four configurations (default when --workload is not given)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=int, default=0, help="override the R-MAT scale (smaller runs)")
    ap.add_argument("--k", type=int, default=0, help="override the dense width")
    ap.add_argument("--variant", type=int, default=0, help="SpMM kernel family / panel shape (tuning)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--rebalance-rounds", type=int, default=5)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (no end-to-end leg, no CPU leg): for profiler runs")
    ap.add_argument("--probe", default=None, choices=["gather"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.configs is None:
        explicit = any(a.startswith("--workload") or a.startswith("--scale") or a.startswith("--k") for a in sys.argv[1:])
        args.configs = "headline" if (explicit or args.kernel_only) else "all"

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, WORKLOADS[args.workload](args), rank)
        return
    if args.probe:
        probe_gather(args)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libcomet_b200 has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    env = Env()
    env.torch, env.dist, env.world, env.rank = torch, dist, world, rank
    from comet_b200 import device as dev
    from comet_b200 import sharding
    env.dev, env.sharding = dev, sharding
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        sharding.init_library_comm()       # libcomet_b200's own communicator for the sharded entry points

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    head, ok = measure(WORKLOADS[args.workload](args), args, env, True)
    clocks = sampler.stop()
    others = {}
    if args.configs == "all":
        base = argparse.Namespace(**vars(args))
        base.scale = base.k = base.variant = 0
        for name in ORDER:
            if name == args.workload:
                continue
            torch.cuda.empty_cache()
            lib_release = getattr(__import__("comet_b200._lib", fromlist=["load"]).load(), "comet_b200_release_scratch")
            lib_release()
            sub_sampler = ClockSampler(physical_gpu_index(local_rank))
            sub_sampler.start()
            res, sub_ok = measure(WORKLOADS[name](base), base, env, False)
            res["clocks"] = sub_sampler.stop()
            ok = ok and sub_ok
            others[name] = res

    if rank == 0:
        line = {
            "metric": "GFLOP/s", "value": head["value"], "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": head["workload"]},
            "notes": {"l2": "inputs larger than L2 (no flush needed)" if args.workload != "spmv" else
                      "inputs fit in L2 (no flush: the operation is launch-bound at this size)",
                      "sharding": "contiguous row blocks of equal measured work, right operand replicated"},
            "clocks": clocks,
        }
        for key in ("e2e", "e2e_pageable", "gpu_launches", "roofline", "per_rank_kernel_ms", "parity_checked",
                    "cpu_baseline", "rebalance_per_rank_ms", "rebalance_kept_round", "row_bounds", "e2e_row_bounds", "e2e_row_bounds_note",
                    "probes_per_s", "nnz_c", "latency"):
            if key in head:
                line[key] = head[key]
        if others:
            line["configs"] = others
        print(json.dumps(line))
    if world > 1:
        env.torch.cuda.synchronize()
        dist.barrier()
        sharding.destroy_library_comm()
        dist.destroy_process_group()
    if not ok:
        sys.stderr.write("bench.py: PARITY MISMATCH against the CPU oracle on rank %d\n" % rank)
        sys.exit(3)


if __name__ == "__main__":
    main()
