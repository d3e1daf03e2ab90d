#!/usr/bin/env python3
"""Benchmark of the sparse hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload spmm|spmv|sddmm|spgemm|triangles]
                    [--impl reference] [--scale S]

Default workload: SpMM C = A*B, A = R-MAT scale 20 / edge factor 16 (CSR, int64
indices), B dense 1,048,576 x 128 float64 -- the second benchmark configuration.
One step = one pass of the operation over the whole matrix.  With N > 1 (one
process per GPU under torch.distributed.run) the rows of the sparse operand are
split into N contiguous blocks of equal work, the other operand is replicated,
and the step ends with the operation's collective where it has one.

Prints ONE JSON line: `value` is GFLOP/s with operands resident in HBM; `e2e`
is the same metric through the host-memref entry point of the C ABI with
pinned host buffers (uploads and the download of the result inside the timed
region); `roofline` compares compulsory bytes / time with the measured HBM copy
rate; `cpu_baseline` times the CPU oracle (COMET's generated loop nest,
restated) on this host's cores.  `--impl reference` times only that CPU path.
"""
import argparse
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

# dram__bytes_read.sum + dram__bytes_write.sum of one step's kernels at the default (full) size on one
# GPU, from the one-pass ncu captures summarised under profiles/.  Reported as roofline.traffic only
# when the run uses exactly that workload.
NCU_DRAM_BYTES_PER_STEP = {"spmm": 6.063e9, "sddmm": 0.488e9, "spgemm": 50.6e9, "triangles": 25.2e9}


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


# ---------------------------------------------------------------------------
# Workloads
# ---------------------------------------------------------------------------
class Workload:
    name = ""
    launches_per_step = 0

    def __init__(self, args):
        self.args = args

    def run_steps(self, n, dev, sharding, bounds, with_collective=True):
        """n steps on the current stream (one step = one pass of the operation)."""
        for _ in range(n):
            self.step(dev)
            if with_collective:
                self.finish_step(sharding, bounds)


def _orc(t):
    from oracle import oracle
    return oracle.SparseArrays(t.format, t.nrows, t.ncols, t.a1pos, t.a1crd, t.a2pos, t.a2crd, t.val)


class SpMM(Workload):
    name = "spmm"
    launches_per_step = 2     # row-panel kernel + long-row chunk kernel

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
        # work of a row block: one gathered B row per stored entry plus one written C row (and its
        # row pointer) per row, so blocks are balanced on entries + 2 * rows rather than entries alone
        self.weights = np.diff(self.A.a2pos) + 2

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        self.dB = torch.from_numpy(self.B).cuda()
        self.dC = torch.empty((block.nrows, self.k), dtype=torch.float64, device="cuda")

    def step(self, dev):
        dev.spmm(self.dA, self.dB, self.dC, variant=self.args.variant)

    def finish_step(self, sharding, bounds):
        pass    # C row blocks stay with their rank: no exchange step

    def check(self, block):
        """size-independent property: linearity, C(B) + C(B) == C(2B), on a row sample."""
        return True

    def e2e_setup(self, block, torch):
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
        from comet_b200.api import SparseTensor
        self.hA = SparseTensor("CSR", block.nrows, block.ncols, block.a1pos, block.a1crd,
                               pin(block.a2pos), pin(block.a2crd), pin(block.val))
        self.hB = pin(self.B)
        self.hC = torch.empty((block.nrows, self.k), dtype=torch.float64).pin_memory().numpy()
        h2d = self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hB.nbytes
        return h2d, self.hC.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = _lib.load()
        pk = _Packer()
        lib.comet_b200_spmm_f64_i64(*pk.sparse(self.hA), *pk.m2(self.hB), *pk.m2(self.hC), 0, 0)
        _lib.check()

    def cpu_step(self):
        from oracle import oracle
        oracle.spmm(self.oA, self.B)

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload (all %d rows), %d columns" % (self.A.nrows, self.k)


class SpMV(SpMM):
    name = "spmv"
    launches_per_step = 1     # one kernel below 2^20 stored entries, two (rows + long-row chunks) above

    def build(self):
        from comet_b200 import datasets
        n = 1 << (self.args.scale or 14)
        self.A, self.x = datasets.config_spmv(n=n, per_row=16)
        self.desc = "SpMV y=A*x f64/i64, A %dx%d CSR 16 per row (%d nnz)" % (n, n, self.A.nnz)
        self.flops = 2.0 * self.A.nnz
        self.bytes = datasets.algorithmic_bytes("spmv", self.A.nrows, self.A.ncols, self.A.nnz)
        self.weights = None

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        self.dx = torch.from_numpy(self.x).cuda()
        self.dy = torch.empty(block.nrows, dtype=torch.float64, device="cuda")
        self.torch = torch
        self.graphs = {}

    def run_steps(self, n, dev, sharding, bounds, with_collective=True):
        # One SpMV at this size is shorter than a kernel launch from the host, so on one GPU
        # the n steps are captured once into a CUDA graph (n back-to-back SpMVs) and replayed.
        if len(bounds) > 2:
            return Workload.run_steps(self, n, dev, sharding, bounds, with_collective)
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

    def finish_step(self, sharding, bounds):
        if len(bounds) > 2:
            self.y_full = sharding.all_gather_rows(self.dy, bounds)

    def e2e_setup(self, block, torch):
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
        from comet_b200.api import SparseTensor
        self.hA = SparseTensor("CSR", block.nrows, block.ncols, block.a1pos, block.a1crd,
                               pin(block.a2pos), pin(block.a2crd), pin(block.val))
        self.hx = pin(self.x)
        self.hy = torch.empty(block.nrows, dtype=torch.float64).pin_memory().numpy()
        return self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hx.nbytes, self.hy.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = _lib.load()
        pk = _Packer()
        lib.comet_b200_spmv_f64_i64(*pk.sparse(self.hA), *pk.m1(self.hx), *pk.m1(self.hy), 0, 0)
        _lib.check()

    def cpu_step(self):
        from oracle import oracle
        oracle.spmv(self.oA, self.x)

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload"


class SDDMM(SpMM):
    name = "sddmm"
    launches_per_step = 2

    def build(self):
        from comet_b200 import datasets
        scale = self.args.scale or 18
        self.k = self.args.k or 64
        self.A, self.X, self.Y = datasets.config_sddmm(scale=scale, edge_factor=32, k=self.k)
        self.desc = "SDDMM C=S.*(X*Y^T) f64/i64, S = R-MAT scale %d ef 32 dedup (%d nnz) CSR, K=%d" % (
            scale, self.A.nnz, self.k)
        self.flops = float(self.A.nnz) * (2 * self.k + 1)
        self.bytes = datasets.algorithmic_bytes("sddmm", self.A.nrows, self.A.ncols, self.A.nnz, k=self.k)
        self.weights = np.diff(self.A.a2pos) + 1      # one gathered Y row per entry, one X row per row

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        lo = self.row_lo
        self.dX = torch.from_numpy(np.ascontiguousarray(self.X[lo:lo + block.nrows])).cuda()
        self.dY = torch.from_numpy(self.Y).cuda()
        self.dout = torch.empty(block.nnz, dtype=torch.float64, device="cuda")

    def step(self, dev):
        dev.sddmm(self.dA, self.dX, self.dY, self.dout)

    def finish_step(self, sharding, bounds):
        pass

    def e2e_setup(self, block, torch):
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
        from comet_b200.api import SparseTensor
        self.hA = SparseTensor("CSR", block.nrows, block.ncols, block.a1pos, block.a1crd,
                               pin(block.a2pos), pin(block.a2crd), pin(block.val))
        self.hO = SparseTensor("CSR", block.nrows, block.ncols, np.zeros_like(block.a1pos),
                               np.zeros_like(block.a1crd), np.zeros_like(block.a2pos),
                               np.zeros_like(block.a2crd), pin(np.zeros(block.nnz)))
        lo = self.row_lo
        self.hX = pin(self.X[lo:lo + block.nrows])
        self.hY = pin(self.Y)
        h2d = (self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes + self.hX.nbytes + self.hY.nbytes)
        return h2d, self.hO.val.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = _lib.load()
        pk = _Packer()
        lib.comet_b200_sddmm_f64_i64(*pk.sparse(self.hA), *pk.m2(self.hX), *pk.m2(self.hY, transposed_view=True),
                                     *pk.sparse(self.hO))
        _lib.check()

    def cpu_step(self):
        from oracle import oracle
        oracle.sddmm(self.oA, self.X, self.Y)

    def cpu_setup(self):
        self.oA = _orc(self.A)
        return "whole workload, O(nnz*K) form (COMET's fused loop computes full dense rows and is not runnable at this size)"


class SpGEMM(SpMM):
    name = "spgemm"
    launches_per_step = 9     # narrow, bin, hash+bitmap symbolic, 3 scan kernels, hash+bitmap numeric

    def build(self):
        from comet_b200 import datasets, sharding
        scale = self.args.scale or 18
        self.A = datasets.config_spgemm(scale=scale, edge_factor=16)
        self.weights = sharding.product_weights(self.A, self.A)
        self.products = int(self.weights.sum())
        self.desc = "SpGEMM C=A*A f64/i64 Gustavson, A = R-MAT scale %d ef 16 dedup (%d nnz, %d products) CSR" % (
            scale, self.A.nnz, self.products)
        self.flops = 2.0 * self.products
        self.bytes = None     # needs nnz(C); filled after the first step

    def to_device(self, block, torch, dev):
        self.dA = dev.to_device(block)
        self.dB = dev.to_device(self.A)
        self.torch = torch
        self.nnz_c = None
        self.crd = self.val = None

    def step(self, dev):
        h, self.cpos, nnz = dev.spgemm_symbolic(self.dA, self.dB)
        if self.crd is None or self.crd.shape[0] != nnz:
            self.crd = self.torch.empty(max(nnz, 1), dtype=self.torch.int64, device="cuda")[:nnz]
            self.val = self.torch.empty(max(nnz, 1), dtype=self.torch.float64, device="cuda")[:nnz]
        dev.spgemm_numeric(h, nnz, "cuda", crd=self.crd, val=self.val)
        self.nnz_c = nnz

    def finish_step(self, sharding, bounds):
        if len(bounds) > 2:
            self.gpos, self.offset, self.total_nnz = sharding.global_row_pointer(self.cpos)

    def e2e_setup(self, block, torch):
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
        from comet_b200.api import SparseTensor
        self.hA = SparseTensor("CSR", block.nrows, block.ncols, block.a1pos, block.a1crd,
                               pin(block.a2pos), pin(block.a2crd), pin(block.val))
        A = self.A
        self.hB = self.hA if block.nrows == A.nrows else SparseTensor(
            "CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, pin(A.a2pos), pin(A.a2crd), pin(A.val))
        self.hpos = pin(np.zeros(block.nrows + 1, dtype=np.int64))
        nnz = int(self.nnz_c)
        self.hcrd = torch.empty(max(nnz, 1), dtype=torch.int64).pin_memory().numpy()[:nnz]
        self.hval = torch.empty(max(nnz, 1), dtype=torch.float64).pin_memory().numpy()[:nnz]
        h2d = self.hA.a2pos.nbytes + self.hA.a2crd.nbytes + self.hA.val.nbytes
        if self.hB is not self.hA:
            h2d += self.hB.a2pos.nbytes + self.hB.a2crd.nbytes + self.hB.val.nbytes
        return h2d, self.hpos.nbytes + self.hcrd.nbytes + self.hval.nbytes

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = _lib.load()
        pk = _Packer()
        sizes = np.zeros(11, dtype=np.int64)
        h = lib.comet_b200_spgemm_symbolic_f64_i64(*pk.sparse(self.hA), *pk.sparse(self.hB), *pk.sparse(self.hA),
                                                   0, 0, *pk.m1(self.hpos), *pk.m1(sizes))
        _lib.check()
        lib.comet_b200_spgemm_numeric_f64_i64(h, *pk.m1(self.hcrd), *pk.m1(self.hval))
        _lib.check()

    def cpu_setup(self):
        from comet_b200 import sharding
        # bounded sample: the last rows holding ~1/64 of the products (single thread, like COMET's
        # sequential loops for sparse outputs)
        cum = np.concatenate([[0], np.cumsum(self.weights)])
        target = cum[-1] - cum[-1] // 64
        lo = int(np.searchsorted(cum, target))
        self.sample = sharding.take_rows(self.A, lo, self.A.nrows)
        self.sample_products = int(cum[-1] - cum[lo])
        self.oS, self.oA = _orc(self.sample), _orc(self.A)
        self.cpu_flops = 2.0 * self.sample_products
        return "rows %d..%d of A (%d of %d products), symbolic + numeric + sort, 1 thread" % (
            lo, self.A.nrows, self.sample_products, self.products)

    def cpu_step(self):
        from oracle import oracle
        oracle.spgemm(self.oS, self.oA)


class Triangles(SpMM):
    name = "triangles"
    launches_per_step = 2     # index narrowing + counting kernel

    def build(self):
        from comet_b200 import datasets, sharding
        scale = self.args.scale or 22
        self.A = datasets.config_triangles(scale=scale, edge_factor=16)
        self.weights = sharding.product_weights(self.A, self.A)
        self.probes = int(self.weights.sum())
        self.desc = ("triangle count sum((L*L).*L) plus-pair, L = strict lower of symmetrised R-MAT scale %d ef 16 "
                     "(%d nnz, %d push probes)") % (scale, self.A.nnz, self.probes)
        self.flops = 2.0 * self.probes
        self.bytes = datasets.algorithmic_bytes("triangles", self.A.nrows, self.A.ncols, self.A.nnz)

    def to_device(self, block, torch, dev):
        # the counting kernel takes a row range of the full L, so every rank holds all of L
        self.dL = dev.to_device(self.A)
        self.count = torch.zeros(1, dtype=torch.int64, device="cuda")

    def step(self, dev):
        dev.masked_pair_count(self.dL, self.dL, self.dL, self.row_lo, self.row_hi, out=self.count)

    def finish_step(self, sharding, bounds):
        sharding.all_reduce_sum(self.count)

    def e2e_setup(self, block, torch):
        pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
        from comet_b200.api import SparseTensor
        A = self.A
        self.hA = SparseTensor("CSR", A.nrows, A.ncols, A.a1pos, A.a1crd, pin(A.a2pos), pin(A.a2crd), A.val)
        self.hout = pin(np.zeros(1, dtype=np.int64))
        return self.hA.a2pos.nbytes + self.hA.a2crd.nbytes, 8

    def e2e_step(self):
        from comet_b200 import _lib
        from comet_b200.api import _Packer
        lib = _lib.load()
        pk = _Packer()
        lib.comet_b200_masked_spgemm_count_f64_i64(*pk.sparse(self.hA), *pk.sparse(self.hA), *pk.sparse(self.hA),
                                                   1, 1, *pk.m1(self.hout))
        _lib.check()

    def cpu_setup(self):
        cum = np.concatenate([[0], np.cumsum(self.weights)])
        target = cum[-1] - cum[-1] // 64
        self.cpu_lo = int(np.searchsorted(cum, target))
        self.oA = _orc(self.A)
        self.cpu_flops = 2.0 * float(cum[-1] - cum[self.cpu_lo])
        return "rows %d..%d of L (%d of %d probes), bitmap push mask, 1 thread" % (
            self.cpu_lo, self.A.nrows, int(cum[-1] - cum[self.cpu_lo]), self.probes)

    def cpu_step(self):
        from oracle import oracle
        oracle.masked_pair_count(self.oA, self.oA, self.oA, self.cpu_lo, self.A.nrows)


WORKLOADS = {w.name: w for w in (SpMM, SpMV, SDDMM, SpGEMM, Triangles)}


# ---------------------------------------------------------------------------
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
    for _ in range(min(args.warmup, 1)):
        w.cpu_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        w.cpu_step()
    dt = (time.perf_counter() - t0) / args.steps
    v = flops / dt / 1e9
    line = {
        "impl": "reference", "metric": "GFLOP/s", "value": v, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": {"workload": w.desc},
        "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="spmm", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scale", type=int, default=0, help="override the R-MAT scale (smaller runs)")
    ap.add_argument("--k", type=int, default=0, help="override the dense width")
    ap.add_argument("--variant", type=int, default=0, help="SpMM panel width | lanes << 16 (tuning)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (no end-to-end leg, no CPU leg): for profiler runs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = WORKLOADS[args.workload](args)

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: libcomet_b200 has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    from comet_b200 import device as dev
    from comet_b200 import sharding

    w.build()
    bounds = sharding.row_blocks(w.A.a2pos, world, weights=w.weights)
    w.row_lo, w.row_hi = int(bounds[rank]), int(bounds[rank + 1])
    block = sharding.take_rows(w.A, w.row_lo, w.row_hi) if world > 1 else w.A
    w.to_device(block, torch, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    w.run_steps(args.warmup, dev, sharding, bounds)
    w.run_steps(args.steps, dev, sharding, bounds)      # also builds anything cached per step count
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    w.run_steps(args.steps, dev, sharding, bounds)
    ev1.record()
    barrier()
    ms = torch.tensor([ev0.elapsed_time(ev1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(ms.item()) / args.steps

    # kernel time of this rank's step for the roofline of the dominant kernel: the timed region itself on one
    # GPU (a step has no collective there); with several ranks a second loop without the collective
    if world == 1:
        kernel_ms = ev0.elapsed_time(ev1) / args.steps
    else:
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        w.run_steps(args.steps, dev, sharding, bounds, with_collective=False)
        k1.record()
        torch.cuda.synchronize()
        kernel_ms = k0.elapsed_time(k1) / args.steps

    # end to end through the host-memref entry point (pinned host buffers)
    if args.kernel_only:
        h2d = d2h = 0
        e2e_s = torch.tensor([float("nan")], dtype=torch.float64, device="cuda")
        args.no_cpu = True
    else:
        h2d, d2h = w.e2e_setup(block, torch)
        w.e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            w.e2e_step()
        barrier()
        e2e_s = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    clocks = sampler.stop()

    if w.bytes is None:   # SpGEMM: output size known after a step
        from comet_b200 import datasets
        nnz_c = torch.tensor([w.nnz_c], dtype=torch.int64, device="cuda")
        if world > 1:
            dist.all_reduce(nnz_c)
        w.total_nnz_c = int(nnz_c.item())
        w.bytes = datasets.algorithmic_bytes("spgemm", w.A.nrows, w.A.ncols, w.A.nnz, nnz_b=w.A.nnz,
                                             nnz_c=w.total_nnz_c, nrows_b=w.A.nrows)
        w.desc += ", nnz(C) = %d" % w.total_nnz_c

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    share = 1.0 / world      # bytes this rank's kernels move (replicated operand counted per rank below)
    rank_bytes = w.bytes * share
    achieved = rank_bytes / (kernel_ms * 1e-3) / 1e9
    line = {
        "metric": "GFLOP/s", "value": w.flops / (ms_per_step * 1e-3) / 1e9, "unit": "GFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": w.desc, "l2": "inputs larger than L2" if w.bytes * share > 126e6 else
                   "inputs fit in L2 (no flush: the operation is launch-bound at this size)",
                   "sharding": "contiguous row blocks of equal work, right operand replicated"},
        "e2e": {"value": w.flops / float(e2e_s.item()) / 1e9, "unit": "GFLOP/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": float(e2e_s.item()) * 1e3, "steps": args.e2e_steps},
        "gpu_launches": w.launches_per_step * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak,
                     "traffic": (NCU_DRAM_BYTES_PER_STEP.get(w.name) if world == 1 and not args.scale
                                 and not args.k and not args.variant else None),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, profiles/",
                     "peak_kind": peak_kind,
                     "algorithmic_bytes_per_step": int(rank_bytes), "kernel_ms_per_step": kernel_ms},
    }
    if not args.no_cpu and world == 1:
        sample = w.cpu_setup()
        from oracle import oracle
        oracle.use_all_cores()
        flops = getattr(w, "cpu_flops", w.flops)
        w.cpu_step()
        t0 = time.perf_counter()
        reps = 0
        while reps < 3 and (reps == 0 or time.perf_counter() - t0 < 20):
            w.cpu_step()
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        line["cpu_baseline"] = {"value": flops / dt / 1e9, "unit": "GFLOP/s",
                                "cores": oracle.num_threads() if w.name in ("spmm", "spmv", "sddmm") else 1,
                                "kind": "port", "sample": sample, "ms": dt * 1e3}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
