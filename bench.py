#!/usr/bin/env python
"""Benchmark of the Klas matrix-multiply hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one
batch of synthetic input: one kernel launch per rank on that rank's shard.

Workloads (seeded synthetic inputs of the shapes and value distributions of the
benchmark configurations; see kuiper_b200/synth.py):
  gemm_bf16   bf16 x bf16 -> f32 tensor-core GEMM, 8192 rows per GPU, N = K = 8192,
              A row-major, B column-major (default; at 8 GPUs this is the row-sharded
              65536 x 8192 x 8192 case).  Metric: TFLOP/s.
  gemm_bf16_65536  the same product with the TOTAL size fixed at 65536 x 8192 x 8192: 65536 / N rows
              per GPU (strong scaling).
  gemm_f16b   batched f16 x f16 -> f16, 2048^3 pages, 64 / N pages per GPU.
  gemm_u64    wrapping u64 GEMM 4096^3, rows sharded.
  gemm_f32    f32 GEMM 1024^3 (single GPU only).
  spmm        CSR(131072^2, Poisson 64) x dense 131072 x 256 f32, CSR rows sharded;
              metric GB/s of compulsory bytes.
Shards need no data-path collective: every rank owns its rows (or pages) of A and C
and a replica of B.

Beside the timed region the line carries, all measured outside it:
  check        sampled rows of this rank's result against an fp64 product of the same inputs; with
               more than one rank also one gathered pass (NCCL all-gather of C) compared with the
               rank-local blocks.
  sustained    (1 GPU, default workload) the same launch back to back for 3 s, with the clocks seen.
  configs      (1 GPU, default workload) a short run of each other benchmark configuration
               (spmm, gemm_f16b, gemm_u64, gemm_f32) with its own roofline and parity bit.
  comparisons  (1 GPU, default workload) the reference's own kernels compiled for sm_100a
               (oracle/_ref), cuBLAS and cuSPARSE through torch, on the same inputs.
`--no-extras` leaves the last three out (profiler captures, quick runs).

`--impl reference` times the reference's own host gold loop (test/matmul_common.c.inc
cpu_mul, compiled unmodified into oracle/_ref; the CSR loop of the oracle for spmm, which
the reference has for u32 only) on the host cores, one instance per hardware thread on
disjoint row blocks of a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

L2_BYTES = 126 * 1024 * 1024


# --------------------------------------------------------------------------- helpers
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    return rank, world, local


def load_peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
        0x2: "applications_clocks_setting", 0x10: "sync_boost", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.mask, self.watts = 0, []   # every reason bit seen (0x1 = idle included), board power
        self.recording = True           # False: the thread polls (and stays warm) but keeps nothing
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            # LOCAL_RANK indexes CUDA_VISIBLE_DEVICES; map through the device UUID
            import torch
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
            except Exception:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _poll(self):
        nv = self.nv
        reasons_of = nv.nvmlDeviceGetCurrentClocksEventReasons if hasattr(
            nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons
        turn = 0
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                mask = reasons_of(self.h)
                if self.recording:
                    self.samples.append(mhz)
                    self.mask |= mask
                    for bit, name in self.REASONS.items():
                        if mask & bit:
                            self.reasons.add(name)
                    if turn % 16 == 2:   # the power query is the slow one: a short timed region must still get its clock samples
                        self.watts.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            turn = turn + 1 if self.recording else 0
            time.sleep(0.001)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples), "reasons_mask": hex(self.mask)}
        if self.watts:
            out["power_w"] = round(statistics.median(self.watts), 1)
            try:
                out["power_limit_w"] = self.nv.nvmlDeviceGetEnforcedPowerLimit(self.h) / 1000.0
            except Exception:
                pass
        return out


# --------------------------------------------------------------------------- workloads
class Workload:
    """Per-rank shard of one workload: device-resident inputs, the launch, its work figures."""
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "tensor"
    launches_per_step = 1

    def per_step_units(self) -> float:        # flop (or bytes) this rank performs per step
        raise NotImplementedError

    def launch(self):                          # one kernel launch on the current stream
        raise NotImplementedError

    def e2e_step(self):                        # C-ABI host-buffer call: H2D + kernel + D2H
        raise NotImplementedError

    def check(self):                           # parity of the last launch's result, outside any timed region
        return None


class GemmBf16(Workload):
    name, metric, unit, dtype, bound = "gemm_bf16", "bf16_gemm_tflops", "TFLOP/s", "bf16", "tensor"
    ROWS_PER_GPU, N, K = 8192, 8192, 8192

    def __init__(self, rank, world, device):
        import torch
        from kuiper_b200 import synth
        self.torch = torch
        self.m_total = self.ROWS_PER_GPU * world
        self.rows = self.ROWS_PER_GPU
        self.A, self.Bt = synth.gemm_bf16(1, self.m_total, self.N, self.K, row0=rank * self.rows,
                                          rows=self.rows, b_col_major=True, device=device)
        self.D = torch.empty((self.rows, self.N), dtype=torch.float32, device=device)
        self.config = self.describe(world)
        self.algorithmic_bytes = 2 * (self.rows * self.K + self.K * self.N) + 4 * self.rows * self.N
        self.h2d = self.A.numel() * 2 + self.Bt.numel() * 2
        self.d2h = self.D.numel() * 4
        self._host = None

    @classmethod
    def describe(cls, world):
        return {"workload": "bf16 x bf16 -> f32 GEMM (tensor-core path), M=%d (8192 rows per GPU) N=K=8192, "
                            "A row-major, B column-major, N(0,1) values, seed 1" % (cls.ROWS_PER_GPU * world),
                "rows_per_gpu": cls.ROWS_PER_GPU, "sharding": "M row blocks, B replicated, no collective",
                "cache": "inputs+output 512 MiB per GPU > 126 MB L2"}

    def per_step_units(self):
        return 2.0 * self.rows * self.N * self.K

    def launch(self):
        from kuiper_b200 import klas
        klas.gemm_tc(self.A, self.Bt, out_dtype=self.torch.float32, b_col_major=True, D=self.D)

    TOL = 2e-3          # bf16 x bf16 -> f32 against fp64, relative to (|A|.|B|)_ij

    def check(self):
        """64 rows of this rank's block of D against an fp64 product of the same seeded rows."""
        t = self.torch
        idx = t.arange(0, self.rows, max(1, self.rows // 64), device=self.A.device)[:64]
        b64 = self.Bt.double()
        want = self.A[idx].double() @ b64.t()
        scale = self.A[idx].double().abs() @ b64.abs().t()
        err = float(((self.D[idx].double() - want).abs() / scale.clamp_min(1e-300)).max())
        return {"what": "64 rows of this rank's block against an fp64 product of the same inputs",
                "rows": int(idx.numel()), "max_rel_err": err, "tol": self.TOL, "ok": err <= self.TOL}

    def e2e_step(self):
        from kuiper_b200 import _lib
        if self._host is None:
            t = self.torch
            self._host = (self.A.cpu().pin_memory(), self.Bt.cpu().pin_memory(),
                          t.empty((self.rows, self.N), dtype=t.float32).pin_memory())
        hA, hB, hD = self._host
        _lib.check(_lib.load().klas_b200_gemm_tc_host(_lib.BF16, _lib.F32, _lib.B_COL_MAJOR, 1, self.rows, self.K,
                                                      self.N, hA.data_ptr(), hB.data_ptr(), None, hD.data_ptr(),
                                                      1.0, 0.0))
        return float(hD[0, 0])

    # ---- CPU legs ------------------------------------------------------------
    def cpu_inputs(self, rows):
        from kuiper_b200 import synth
        a, b = synth.gemm_bf16(1, self.ROWS_PER_GPU, self.N, self.K, row0=0, rows=rows, b_col_major=False)
        return a, b

    def cpu_units(self, rows):
        return 2.0 * rows * self.N * self.K


class GemmBf16Sharded(GemmBf16):
    """The row-sharded 65536 x 8192 x 8192 case with its TOTAL size fixed: 65536 / N rows per GPU
    (strong scaling; at N = 8 it is the default workload's 8192 rows per GPU)."""
    name = "gemm_bf16_65536"
    TOTAL_ROWS = 65536

    def __init__(self, rank, world, device):
        if self.TOTAL_ROWS % (world * 512) != 0:
            raise SystemExit("gemm_bf16_65536 wants the 65536 rows to split into whole 512-row tiles per GPU")
        type(self).ROWS_PER_GPU = self.TOTAL_ROWS // world     # read by the base class
        super().__init__(rank, world, device)
        self.config = {"workload": "bf16 x bf16 -> f32 GEMM (tensor-core path), M=65536 in total (%d rows per GPU) N=K=8192, "
                                   "A row-major, B column-major, N(0,1) values, seed 1" % self.rows,
                       "rows_per_gpu": self.rows, "sharding": "M row blocks, B replicated, no collective",
                       "cache": "inputs+output %d MiB per GPU > 126 MB L2" % ((self.h2d + self.d2h) >> 20)}


class CublasBf16(GemmBf16):
    """COMPARISON ONLY: the headline product through cuBLAS (torch.mm with f32 output) on the same
    inputs, so that a profiler can capture the vendor kernel with the same command line.  Nothing of
    this library runs in its launch; its line reports gpu_launches = 0."""
    name, metric = "cublas_bf16", "cublas_bf16_gemm_tflops_comparison_only"
    launches_per_step = 0

    def launch(self):
        t = self.torch
        try:
            self.D = t.mm(self.A, self.Bt.t(), out_dtype=t.float32)
        except TypeError:
            self.D = t.mm(self.A, self.Bt.t()).float()

    def e2e_step(self):
        hA, hB = self.A.cpu().pin_memory(), self.Bt.cpu().pin_memory()
        self.A.copy_(hA, non_blocking=True)
        self.Bt.copy_(hB, non_blocking=True)
        self.launch()
        return float(self.D.cpu()[0, 0])


class GemmF16Batched(Workload):
    name, metric, unit, dtype, bound = "gemm_f16b", "f16_batched_gemm_tflops", "TFLOP/s", "f16", "tensor"

    def __init__(self, rank, world, device):
        import torch
        from kuiper_b200 import synth
        self.torch = torch
        self.pages = 64 // world
        self.m = self.n = self.k = 2048
        self.A, self.B = synth.gemm_f16_batched(2, self.pages, self.m, self.n, self.k, batch0=rank * self.pages, device=device)
        self.D = torch.empty((self.pages, self.m, self.n), dtype=torch.float16, device=device)
        self.config = {"workload": "batched f16 x f16 -> f16 GEMM, 64 pages of 2048^3, %d pages per GPU, U[-0.5,0.5), seed 2" % self.pages,
                       "sharding": "batch pages, no collective", "cache": "1.5 GiB of pages in total > L2"}
        self.algorithmic_bytes = self.pages * 3 * self.m * self.n * 2
        self.h2d, self.d2h = 2 * self.A.numel() * 2, self.D.numel() * 2
        self._host = None

    def per_step_units(self):
        return 2.0 * self.pages * self.m * self.n * self.k

    def launch(self):
        from kuiper_b200 import klas
        klas.gemm_tc(self.A, self.B, out_dtype=self.torch.float16, D=self.D)

    TOL = 1e-2

    def check(self):
        """16 rows of EVERY page against fp64 products of the same rows."""
        t = self.torch
        idx = t.arange(0, self.m, self.m // 16, device=self.A.device)[:16]
        worst = 0.0
        for pg in range(self.pages):
            b64 = self.B[pg].double()
            want = self.A[pg][idx].double() @ b64
            scale = self.A[pg][idx].double().abs() @ b64.abs()
            worst = max(worst, float(((self.D[pg][idx].double() - want).abs() / scale.clamp_min(1e-300)).max()))
        return {"what": "16 rows of each of the %d pages against fp64 products" % self.pages, "rows": 16 * self.pages,
                "max_rel_err": worst, "tol": self.TOL, "ok": worst <= self.TOL}

    def e2e_step(self):
        from kuiper_b200 import _lib
        if self._host is None:
            self._host = (self.A.cpu().pin_memory(), self.B.cpu().pin_memory(), self.D.cpu().pin_memory())
        hA, hB, hD = self._host
        _lib.check(_lib.load().klas_b200_gemm_tc_host(_lib.F16, _lib.F16, _lib.B_ROW_MAJOR, self.pages, self.m, self.k,
                                                      self.n, hA.data_ptr(), hB.data_ptr(), None, hD.data_ptr(), 1.0, 0.0))
        return float(hD[0, 0, 0])


class GemmSimt(Workload):
    bound = "issue"

    def __init__(self, rank, world, device, kind):
        import torch
        from kuiper_b200 import synth
        self.torch = torch
        self.kind = kind
        if kind == "u64":
            self.name, self.metric, self.unit, self.dtype = "gemm_u64", "u64_gemm_tops", "Tops/s", "u64"
            n = 4096
            self.rows = n // world
            self.A, self.B = synth.gemm_u64(3, n, n, n, row0=rank * self.rows, rows=self.rows, device=device)
            es = 8
            self.config = {"workload": "wrapping u64 GEMM 4096^3, entries < 2^32, seed 3, %d rows per GPU" % self.rows,
                           "sharding": "M row blocks, B replicated", "cache": "384 MiB of matrices > L2"}
        else:
            self.name, self.metric, self.unit, self.dtype = "gemm_f32", "f32_gemm_tflops", "TFLOP/s", "f32"
            n = 1024
            self.rows = n // world
            self.A, self.B = synth.gemm_f32(0, n, n, n, row0=rank * self.rows, rows=self.rows, device=device)
            es = 4
            self.config = {"workload": "f32 GEMM 1024^3, U[-1,1), seed 0", "cache": "L2 flushed between steps: no (12 MiB fits L2)"}
        self.n = n
        self.C = torch.empty((self.rows, n), dtype=self.A.dtype, device=device)
        self.algorithmic_bytes = es * (self.rows * n + n * n + self.rows * n)
        self.h2d, self.d2h = es * (self.A.numel() + self.B.numel()), es * self.C.numel()
        self._host = None

    def per_step_units(self):
        return 2.0 * self.rows * self.n * self.n

    def launch(self):
        from kuiper_b200 import klas
        klas.gemm(self.A, self.B, self.C)

    def check(self):
        t = self.torch
        if self.kind == "u64":
            # 8 rows, exact: int64 products and sums wrap mod 2^64 exactly as the kernel's do
            idx = list(range(0, self.rows, max(1, self.rows // 8)))[:8]
            bad = 0
            for r in idx:
                want = (self.A[r][:, None] * self.B).sum(0)
                bad += int((want != self.C[r]).sum())
            return {"what": "8 rows, bit for bit, against wrapping int64 arithmetic", "rows": len(idx),
                    "mismatches": bad, "ok": bad == 0}
        want = self.A.double() @ self.B.double()
        scale = self.A.double().abs() @ self.B.double().abs()
        err = float(((self.C.double() - want).abs() / scale.clamp_min(1e-300)).max())
        return {"what": "the whole result against an fp64 product", "rows": self.rows, "max_rel_err": err,
                "tol": 1e-5, "ok": err <= 1e-5}

    def e2e_step(self):
        from kuiper_b200 import _lib
        if self._host is None:
            self._host = (self.A.cpu().pin_memory(), self.B.cpu().pin_memory(), self.C.cpu().pin_memory())
        hA, hB, hC = self._host
        code = _lib.U64 if self.kind == "u64" else _lib.F32
        _lib.check(_lib.load().klas_b200_gemm_host(code, _lib.RRR, 1, self.rows, self.n, self.n, None, None,
                                                   hA.data_ptr(), hB.data_ptr(), hC.data_ptr()))
        return float(hC[0, 0])


class Spmm(Workload):
    name, metric, unit, dtype, bound = "spmm", "spmm_compulsory_gbs", "GB/s", "f32", "hbm"
    ROWS = SHARED = 131072
    COLS = 256

    def __init__(self, rank, world, device):
        import torch
        from kuiper_b200 import synth
        self.torch = torch
        self.rows = self.ROWS // world
        self.csr = synth.csr_poisson(4, self.ROWS, self.SHARED, 64.0, row0=rank * self.rows, nrows=self.rows, device=device)
        self.B = synth.spmm_dense_b(4, self.SHARED, self.COLS, device=device)
        self.C = torch.empty((self.rows, self.COLS), dtype=torch.float32, device=device)
        nnz = self.csr.nnz
        self.nnz = nnz
        # compulsory bytes: values+columns, row offsets, row order, B once, C once
        self.algorithmic_bytes = nnz * 8 + (self.rows + 1) * 4 + self.rows * 4 + 4 * self.SHARED * self.COLS + 4 * self.rows * self.COLS
        self.config = {"workload": "CSR x dense SpMM, A 131072^2 Poisson(64) nnz per row, B 131072 x 256 f32, seed 4, %d CSR rows per GPU" % self.rows,
                       "nnz_per_gpu": nnz, "sharding": "CSR row ranges, B replicated, no collective",
                       "cache": "B 128 MiB + A 64 MiB + C 128 MiB > 126 MB L2",
                       "bytes_model": "compulsory: nnz*8 + row_off + row_indices + B + C"}
        self.h2d = nnz * 8 + (2 * self.rows + 1) * 4 + 4 * self.SHARED * self.COLS
        self.d2h = 4 * self.rows * self.COLS
        self._host = None

    def per_step_units(self):
        return float(self.algorithmic_bytes)

    def launch(self):
        from kuiper_b200 import klas
        klas.spmm(self.csr, self.B, self.C)

    def launch_gather_probe(self):
        from kuiper_b200 import klas
        klas.spmm_gather_probe(self.csr, self.B)

    def check(self):
        """64 rows against an fp64 gather-and-sum of the same rows."""
        t = self.torch
        ro = self.csr.row_off.long()
        worst = 0.0
        rows = list(range(0, self.rows, max(1, self.rows // 64)))[:64]
        for r in rows:
            lo, hi = int(ro[r]), int(ro[r + 1])
            prod = self.csr.elems[lo:hi].double()[:, None] * self.B[self.csr.col_ind[lo:hi].long()].double()
            want, scale = prod.sum(0), prod.abs().sum(0)
            worst = max(worst, float(((self.C[r].double() - want).abs() / scale.clamp_min(1e-300)).max()))
        return {"what": "64 rows against an fp64 sum of the same products", "rows": len(rows), "max_rel_err": worst,
                "tol": 1e-5, "ok": worst <= 1e-5}

    def e2e_step(self):
        from kuiper_b200 import _lib
        if self._host is None:
            c = self.csr
            self._host = tuple(t.cpu().pin_memory() for t in (c.elems, c.col_ind, c.row_off, c.row_indices, self.B, self.C))
        e, ci, ro, ri, b, cc = self._host
        _lib.check(_lib.load().klas_b200_spmm_host(_lib.F32, self.rows, self.SHARED, self.COLS, self.nnz, e.data_ptr(),
                                                   ci.data_ptr(), ro.data_ptr(), ri.data_ptr(), b.data_ptr(), cc.data_ptr()))
        return float(cc[0, 0])


class Softmax(Workload):
    name, metric, unit, dtype, bound = "softmax_f32", "softmax_gbs", "GB/s", "f32", "hbm"
    launches_per_step = 2          # per-chunk statistics, then the rewrite
    N = 1 << 28                    # elements per GPU (1 GiB of f32)

    def __init__(self, rank, world, device, log2n=28):
        import torch
        from kuiper_b200 import _lib, synth
        self.torch = torch
        self.N = 1 << log2n
        self.x = synth.normal(5 + rank, 21, 0, self.N, dtype=torch.float32, device=device) * 4.0
        torch.cuda.empty_cache()       # the generator's float64 temporaries
        need = _lib.load().klas_b200_softmax_scratch_bytes(1, self.N)
        self.scratch = torch.empty(need, dtype=torch.uint8, device=device)
        self.algorithmic_bytes = 3 * 4 * self.N          # two reads and one write of the vector
        self.traffic_scaled = log2n == 28   # the DRAM-traffic capture is of the bench size only
        self.config = {"workload": "in-place softmax of one f32 vector of 2^%d elements per GPU, N(0,16) values, seed 5+rank; "
                                   "steps after the first run on the previous step's output (same traffic and instruction count)" % log2n,
                       "sharding": "one independent vector per GPU, no collective",
                       "cache": "%d MiB vector > 126 MB L2" % (self.N * 4 >> 20),
                       "bytes_model": "3 x 4 bytes per element: read for the statistics, read and write for the result"}
        self.h2d = self.d2h = 4 * self.N
        self._host = None

    def per_step_units(self):
        return float(self.algorithmic_bytes)

    def launch(self):
        from kuiper_b200 import _lib
        _lib.check(_lib.load().klas_b200_softmax(_lib.F32, 0, 1, self.N, self.x.data_ptr(), self.scratch.data_ptr(),
                                                 self.scratch.numel(), self.torch.cuda.current_stream().cuda_stream))

    def e2e_step(self):
        from kuiper_b200 import _lib
        if self._host is None:
            self._host = self.x.cpu().pin_memory()
        _lib.check(_lib.load().klas_b200_softmax_host(_lib.F32, 0, 1, self.N, self._host.data_ptr()))
        return float(self._host[0])


class Attention(Workload):
    name, metric, unit, dtype, bound = "attention_f16", "attention_tflops", "TFLOP/s", "f16", "tensor"
    e2e_api = "pinned host copies around klas_b200_sdpa_fused (C ABI, device pointers)"
    L = S = 2048
    E = 128

    def __init__(self, rank, world, device, heads=256):
        import torch
        from kuiper_b200 import synth
        self.torch = torch
        self.heads = heads
        n = heads * self.L * self.E
        mk = lambda stream: synth.normal(6 + rank, stream, 0, n, dtype=torch.float16, device=device).reshape(heads, self.L, self.E)
        self.Q, self.K, self.V = mk(31), mk(32), mk(33)
        self.out = torch.empty_like(self.Q)
        torch.cuda.empty_cache()
        self.algorithmic_bytes = 4 * n * 2
        self.config = {"workload": "fused attention softmax(Q.K^T / sqrt(e)).V, f16, %d heads per GPU, l = s = %d, e = %d, N(0,1) values, seed 6+rank"
                                   % (heads, self.L, self.E),
                       "sharding": "heads, no collective", "cache": "%d MiB of Q, K, V, O" % (4 * n * 2 >> 20)}
        self.h2d, self.d2h = 3 * n * 2, n * 2
        self._host = None

    def per_step_units(self):
        return 4.0 * self.heads * self.L * self.S * self.E

    def launch(self):
        from kuiper_b200 import _lib
        _lib.check(_lib.load().klas_b200_sdpa_fused(_lib.F16, self.heads, self.L, self.S, self.E, self.Q.data_ptr(), self.K.data_ptr(),
                                                    self.V.data_ptr(), self.out.data_ptr(), self.E ** -0.5,
                                                    self.torch.cuda.current_stream().cuda_stream))

    def e2e_step(self):
        # no host-buffer entry point for attention: pinned copies around the device call
        if self._host is None:
            self._host = tuple(t.cpu().pin_memory() for t in (self.Q, self.K, self.V, self.out))
        hq, hk, hv, ho = self._host
        self.Q.copy_(hq, non_blocking=True)
        self.K.copy_(hk, non_blocking=True)
        self.V.copy_(hv, non_blocking=True)
        self.launch()
        ho.copy_(self.out, non_blocking=True)
        self.torch.cuda.current_stream().synchronize()
        return float(ho[0, 0, 0])


def make_workload(name, rank, world, device, args=None):
    if name == "attention_f16":
        return Attention(rank, world, device, args.attention_heads if args else 256)
    if name == "softmax_f32":
        return Softmax(rank, world, device, args.softmax_log2n if args else 28)
    if name == "gemm_bf16":
        return GemmBf16(rank, world, device)
    if name == "gemm_bf16_65536":
        return GemmBf16Sharded(rank, world, device)
    if name == "cublas_bf16":
        return CublasBf16(rank, world, device)
    if name == "gemm_f16b":
        return GemmF16Batched(rank, world, device)
    if name == "gemm_u64":
        return GemmSimt(rank, world, device, "u64")
    if name == "gemm_f32":
        return GemmSimt(rank, world, device, "f32")
    if name == "spmm":
        return Spmm(rank, world, device)
    raise SystemExit("unknown workload " + name)


# --------------------------------------------------------------------------- CPU legs
CPU_METRICS = {"gemm_bf16": ("bf16_gemm_tflops", "TFLOP/s", "bf16"), "gemm_f16b": ("f16_batched_gemm_tflops", "TFLOP/s", "f16"),
               "gemm_u64": ("u64_gemm_tops", "Tops/s", "u64"), "gemm_f32": ("f32_gemm_tflops", "TFLOP/s", "f32"),
               "spmm": ("spmm_compulsory_gbs", "GB/s", "f32")}


def reference_cpu_leg(workload: str, threads: int):
    """The reference's own host gold loop for `workload` (test/matmul_common.c.inc cpu_mul per element
    type, compiled unmodified into oracle/_ref; the oracle port where oracle/_ref is absent, and for
    spmm, whose f32 CSR loop the reference does not have) on a bounded sample of the workload: every
    thread multiplies its own block of rows of A by all of B.
    Returns (one_pass -> seconds, kind, sample description, units per pass)."""
    import numpy as np
    sys.path.insert(0, str(REPO / "oracle"))
    import build as oracle_build
    from oracle_api import Oracle, RefCpu, bf16_bits
    from kuiper_b200 import synth
    have_ref = RefCpu.available()
    ref = RefCpu() if have_ref else None
    if not have_ref or workload == "spmm":
        oracle_build.build_oracle()
    orc = Oracle() if (not have_ref or workload == "spmm") else None
    kind = "reference" if have_ref and workload != "spmm" else "port"

    def gemm_leg(ref_kind, port_kind, a_np, b_np, rows_per_thread, units, sample):
        def run_block(t):
            blk = np.ascontiguousarray(a_np[t * rows_per_thread:(t + 1) * rows_per_thread])
            if have_ref:
                ref.cpu_mul(ref_kind, blk, b_np)
            elif port_kind in ("u64",):
                orc.gemm_int(blk, b_np)
            else:
                orc.gemm(blk, b_np, kind=port_kind, threads=1)
        return run_block, units, sample

    if workload == "gemm_bf16":
        rpt = 2
        a, b = synth.gemm_bf16(1, GemmBf16.ROWS_PER_GPU, GemmBf16.N, GemmBf16.K, row0=0, rows=rpt * threads, b_col_major=False)
        run_block, units, sample = gemm_leg("bf16_f32", "bf16", bf16_bits(a), bf16_bits(b), rpt, 2.0 * rpt * threads * GemmBf16.N * GemmBf16.K,
                                            "%d rows of A (%d per thread) x full 8192 x 8192 B per step" % (rpt * threads, rpt))
    elif workload == "gemm_f16b":
        rpt = 16
        a, b = synth.gemm_f16_batched(2, 1, 2048, 2048, 2048)
        a_np, b_np = a[0][:rpt * threads].contiguous().view(torch_int16()).numpy().view(np.uint16), b[0].view(torch_int16()).numpy().view(np.uint16)
        run_block, units, sample = gemm_leg("f16_f16", "f16", a_np, b_np, rpt, 2.0 * min(rpt * threads, 2048) * 2048 * 2048,
                                            "%d rows of page 0 (%d per thread) x its 2048 x 2048 B per step" % (min(rpt * threads, 2048), rpt))
    elif workload == "gemm_u64":
        rpt = 4
        a, b = synth.gemm_u64(3, 4096, 4096, 4096, row0=0, rows=rpt * threads)
        run_block, units, sample = gemm_leg("u64", "u64", a.numpy().view(np.uint64), b.numpy().view(np.uint64), rpt, 2.0 * rpt * threads * 4096 * 4096,
                                            "%d rows of A (%d per thread) x full 4096 x 4096 B per step" % (rpt * threads, rpt))
    elif workload == "gemm_f32":
        rpt = max(1, min(64, 1024 // threads))
        a, b = synth.gemm_f32(0, 1024, 1024, 1024, row0=0, rows=rpt * threads)
        run_block, units, sample = gemm_leg("f32", "f32", a.numpy(), b.numpy(), rpt, 2.0 * rpt * threads * 1024 * 1024,
                                            "%d rows of A (%d per thread) x full 1024 x 1024 B per step" % (rpt * threads, rpt))
    elif workload == "spmm":
        rpt = 256
        nrows = rpt * threads
        csr = synth.csr_poisson(4, Spmm.ROWS, Spmm.SHARED, 64.0, row0=0, nrows=nrows)
        bmat = synth.spmm_dense_b(4, Spmm.SHARED, Spmm.COLS).numpy()
        el, ci, ro = csr.elems.numpy(), csr.col_ind.numpy().view(np.uint32), csr.row_off.numpy().view(np.uint32)

        def run_block(t):
            lo, hi = int(ro[t * rpt]), int(ro[(t + 1) * rpt])
            orc.spmm_f32(rpt, Spmm.COLS, el[lo:hi], ci[lo:hi], np.ascontiguousarray(ro[t * rpt:(t + 1) * rpt + 1] - ro[t * rpt]), bmat, threads=1)
        nnz = int(ro[nrows])
        # the GPU line's byte model, scaled to the sample: its nonzeros, row offsets and order, its rows of C,
        # and its share (rows / all rows) of the one read of B
        units = nnz * 8 + (2 * nrows + 1) * 4 + 4 * nrows * Spmm.COLS + 4 * Spmm.SHARED * Spmm.COLS * nrows / Spmm.ROWS
        sample = "%d CSR rows (%d per thread, %d nonzeros) x full 131072 x 256 B per step; the oracle's f32 CSR loop (the reference has one for u32 only)" % (nrows, rpt, nnz)
    else:
        return None

    def one_pass():
        ts = [threading.Thread(target=run_block, args=(t,)) for t in range(threads)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0

    return one_pass, kind, sample, float(units)


def torch_int16():
    import torch
    return torch.int16


def run_reference_arm(args, rank, world):
    if rank != 0:
        return 0
    if args.workload not in CPU_METRICS:
        print(json.dumps({"impl": "reference", "unavailable": "the reference has no host loop for workload %s" % args.workload}))
        return 0
    threads = os.cpu_count() or 1
    one_pass, kind, sample, units = reference_cpu_leg(args.workload, threads)
    metric, unit, dtype = CPU_METRICS[args.workload]
    scale = 1e12 if unit in ("TFLOP/s", "Tops/s") else 1e9
    for _ in range(max(args.warmup, 1)):
        one_pass()
    t = 0.0
    for _ in range(args.steps):
        t += one_pass()
    value = units * args.steps / t / scale
    describe = {"gemm_bf16": GemmBf16.describe(max(args.gpus, 1))}.get(args.workload, {"workload": args.workload})
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak" if args.workload == "gemm_bf16" else "strong", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": dict(describe, sample=sample, impl="host gold loop on a row sample, one instance per hardware thread"),
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def cpu_baseline_softmax():
    """The reference drivers' gold softmax (test/softmax_test_common.c.inc, compiled unmodified into
    oracle/_ref; float64, one thread) -- or the oracle port -- on a 2^24-element sample."""
    import numpy as np
    sys.path.insert(0, str(REPO / "oracle"))
    import build as oracle_build
    from oracle_api import Oracle, RefCpu
    n = 1 << 24
    x = np.random.default_rng(5).normal(size=n) * 4.0
    if RefCpu.available():
        fn, kind = RefCpu().cpu_softmax, "reference"
    else:
        oracle_build.build_oracle()
        fn, kind = Oracle().softmax, "port"
    fn(x[:1024])
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0:
        fn(x)
        reps += 1
    t = time.perf_counter() - t0
    # same byte model as the GPU line, on the sample's f32-equivalent size
    return {"value": 3 * 4 * n * reps / t / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
            "sample": "%d x softmax of 2^24 elements in float64, single thread as written; bytes counted as 12 per element" % reps}


def cpu_baseline_leg(workload_name, seconds=12.0):
    """Single-threaded, as the reference's loop is written; about `seconds` of CPU work."""
    if workload_name == "softmax_f32":
        return cpu_baseline_softmax()
    if workload_name not in CPU_METRICS:
        return None
    one_pass, kind, sample, units = reference_cpu_leg(workload_name, 1)
    unit = CPU_METRICS[workload_name][1]
    scale = 1e12 if unit in ("TFLOP/s", "Tops/s") else 1e9
    t1 = one_pass()
    reps = max(1, min(64, int(seconds / max(t1, 1e-3))))
    t = sum(one_pass() for _ in range(reps))
    return {"value": units * reps / t / scale, "unit": unit, "cores": 1, "kind": kind,
            "sample": "%d x (%s), single thread as written" % (reps, sample)}


# --------------------------------------------------------------------------- measurement helpers
# DRAM traffic of one launch (dram__bytes_read.sum + dram__bytes_write.sum) from an ncu capture of
# the same kernel on the same workload (the summaries are under profiles/).  Each figure is tied
# to the SHA-256 of the kernel source it was captured from: when the source has changed since,
# the figure is withheld (traffic null, with a note) instead of going stale silently.
NCU_TRAFFIC = {
    "gemm_bf16": (1.148e+09, "kuiper_b200/csrc/gemm_umma.cu", "d152cda6d0ff23f4"),
    "gemm_f16b": (1.645e+09, "kuiper_b200/csrc/gemm_umma.cu", "d152cda6d0ff23f4"),
    "spmm": (1.131e+09, "kuiper_b200/csrc/spmm.cu", "00fe2789a6167b7d"),
    "gemm_u64": (2.167e+09, "kuiper_b200/csrc/gemm_simt.cu", "1347f823e1dfa70e"),
    "gemm_f32": (1.261e+07, "kuiper_b200/csrc/gemm_simt.cu", "1347f823e1dfa70e"),
    "softmax_f32": (3.163e+09, "kuiper_b200/csrc/rowops.cu", "06bc7eefe6fa1b1b"),
}
NOMINAL_BF16_TFLOPS = 2250.0     # dense bf16, vendor figure
NOMINAL_HBM_GBS = 8000.0


def ncu_traffic(name):
    """(bytes or None, note) for workload `name`."""
    if name not in NCU_TRAFFIC:
        return None, "no capture"
    nbytes, rel, digest = NCU_TRAFFIC[name]
    src = REPO / rel
    if not src.exists():
        return None, "kernel source not found"
    now = hashlib.sha256(src.read_bytes()).hexdigest()[:16]
    if now != digest:
        return None, "withheld: %s has changed since the capture (%s then, %s now)" % (rel, digest, now)
    return nbytes, "ncu capture of this source (%s)" % digest


def time_launches(torch, fn, steps, warm=3):
    """Average device time of `fn` (ms) over `steps` back-to-back calls after `warm` untimed ones."""
    for _ in range(warm):
        fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    s.record()
    for _ in range(steps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps


def roofline_of(wl, per_launch_ms, peaks, sm_mhz=None):
    """The roofline block of one workload: algorithmic work of a launch over its device time,
    against the measured peak (and, for the tensor-core and HBM bounds, the other denominators)."""
    sec = per_launch_ms * 1e-3
    out = {}
    if wl.bound == "tensor":
        achieved = wl.per_step_units() / sec / 1e12
        peak, runit = peaks["bf16_tflops"], "TFLOP/s"
        peak_note = "cuBLAS bf16 burst, of %s" % peaks["source"]
        out["frac_burst"] = achieved / peaks["bf16_tflops"]
        if peaks.get("bf16_tflops_sustained"):
            out["frac_sustained"] = achieved / peaks["bf16_tflops_sustained"]
        out["frac_nominal"] = achieved / NOMINAL_BF16_TFLOPS
        out["denominators"] = {"burst_of_%s" % peaks["source"]: peaks["bf16_tflops"],
                               "sustained_of_%s" % peaks["source"]: peaks.get("bf16_tflops_sustained"),
                               "nominal_dense_bf16": NOMINAL_BF16_TFLOPS}
    elif wl.bound == "hbm":
        achieved = wl.algorithmic_bytes / sec / 1e9
        peak, runit = peaks["hbm_gbs"], "GB/s"
        peak_note = "stream copy, of %s" % peaks["source"]
        out["frac_nominal"] = achieved / NOMINAL_HBM_GBS
    else:
        # CUDA-core GEMMs are issue-bound: reported against the nominal issue peak at max clock
        achieved = wl.per_step_units() / sec / 1e12
        if wl.name == "gemm_u64":
            # a wrapping u64 multiply-add = one widening 32x32 multiply-add (2 issue slots of the
            # 64-lane integer-multiply pipe) + two 32-bit ones: 4 slots per MAC, 2 ops per MAC
            peak, runit = 2 * (64 / 4) * 148 * 1.965e9 / 1e12, "Tops/s"
            peak_note = "64 integer-multiply lanes/clk/SM, 4 slots per u64 MAC, 148 SMs, 1965 MHz (nominal)"
        else:
            peak, runit = 2 * 128 * 148 * 1.965e9 / 1e12, "TFLOP/s"
            peak_note = "2*128 lanes*148 SMs*1965 MHz FP32 issue peak (nominal)"
    traffic, traffic_note = ncu_traffic(wl.name)
    if getattr(wl, "traffic_scaled", True) is False:
        traffic, traffic_note = None, "the capture is of the bench size only"
    roof = {"bound": "tensor" if wl.bound == "tensor" else "hbm" if wl.bound == "hbm" else "issue",
            "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
            "traffic": traffic, "traffic_note": traffic_note, "peak_note": peak_note,
            "algorithmic_bytes_per_launch": wl.algorithmic_bytes, "kernel_ms": per_launch_ms}
    if sm_mhz:
        roof["sm_mhz"] = sm_mhz
    roof.update(out)
    return roof


def spmm_gather_block(torch, wl, per_launch_ms):
    """What really bounds the SpMM kernel: with random columns every nonzero moves 4 * cols bytes of a
    row of B from L2 to an SM whatever the schedule.  The ceiling is measured here, on the same
    matrix: a kernel that issues exactly those reads and nothing else (klas_b200_spmm_gather_probe)."""
    gather = wl.nnz * 4 * wl.COLS
    probe_ms = time_launches(torch, wl.launch_gather_probe, 20)
    return {"gather_bytes_per_launch": gather, "gather_achieved_gbs": gather / (per_launch_ms * 1e-3) / 1e9,
            "gather_probe_ms": probe_ms, "gather_ceiling_gbs": gather / (probe_ms * 1e-3) / 1e9,
            "frac_of_gather_ceiling": probe_ms / per_launch_ms,
            "note": "compulsory DRAM bytes are 1/25 of the L2->SM gather volume at this size: the kernel is bound by "
                    "the gather rate, measured by the probe (same index stream, same 512-byte reads, no values, "
                    "products or stores)"}


def sustained_leg(torch, wl, local, peaks, seconds=3.0):
    """The headline launch back to back for `seconds` (the power cap settles within about a second):
    what the kernel sustains, with the SM clock and throttle reasons seen while it ran."""
    per = time_launches(torch, wl.launch, 10)
    n = max(50, int(seconds * 1e3 / per))
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    torch.cuda.synchronize()
    with sampler:
        s.record()
        for _ in range(n):
            wl.launch()
        e.record()
        torch.cuda.synchronize()
    ms = s.elapsed_time(e)
    value = wl.per_step_units() * n / (ms * 1e-3) / 1e12
    out = {"seconds": ms * 1e-3, "launches": n, "value": value, "unit": "TFLOP/s", "ms_per_launch": ms / n,
           "clocks": sampler.summary(), "frac_nominal": value / NOMINAL_BF16_TFLOPS, "frac_burst": value / peaks["bf16_tflops"]}
    if peaks.get("bf16_tflops_sustained"):
        out["frac_sustained"] = value / peaks["bf16_tflops_sustained"]
    return out


def config_leg(torch, name, device, peaks, args):
    """A short run (>= 20 launches) of one of the other benchmark configurations on this GPU: value,
    roofline, parity of the result, and the host loop on a small sample."""
    t0 = time.perf_counter()
    wl = make_workload(name, 0, 1, device, args)
    steps = 20 if name != "gemm_f32" else 200
    per = time_launches(torch, wl.launch, steps)
    scale = 1e12 if wl.unit in ("TFLOP/s", "Tops/s") else 1e9
    out = {"metric": wl.metric, "value": wl.per_step_units() / (per * 1e-3) / scale, "unit": wl.unit, "steps": steps,
           "ms_per_step": per, "config": wl.config, "roofline": roofline_of(wl, per, peaks), "parity": wl.check()}
    if name == "spmm":
        out["roofline"]["gather"] = spmm_gather_block(torch, wl, per)
    wl.e2e_step()
    t1 = time.perf_counter()
    for _ in range(2):
        wl.e2e_step()
    torch.cuda.synchronize()
    out["e2e"] = {"value": wl.per_step_units() * 2 / (time.perf_counter() - t1) / scale, "unit": wl.unit,
                  "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h, "steps": 2}
    if not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline_leg(name, seconds=2.0)
    del wl
    torch.cuda.empty_cache()
    out["leg_seconds"] = time.perf_counter() - t0
    return out


class RefGpuLib:
    """The reference's own extracted kernels compiled for sm_100a (oracle/_ref, built from the
    FStarLang/kuiper tree by oracle/build.py).  Comparison rows only: nothing here is timed as ours."""

    class SMatrixF32(ctypes.Structure):
        _fields_ = [("nnz", ctypes.c_uint32), ("elems", ctypes.c_void_p), ("col_ind", ctypes.c_void_p), ("row_off", ctypes.c_void_p)]

    def __init__(self):
        d = REPO / "oracle" / "_ref"
        self.lib = ctypes.CDLL(str(d / "libklas_ref_gpu.so"))
        self.symbols = json.loads((d / "symbols.json").read_text())
        ng = d / "libklas_ref_spmm_noguard.so"
        self.noguard = ctypes.CDLL(str(ng)) if ng.exists() else None

    @staticmethod
    def available():
        d = REPO / "oracle" / "_ref"
        return (d / "libklas_ref_gpu.so").exists() and (d / "symbols.json").exists()

    def gemm(self, name, m, k, n, A, B, Cc):
        f = getattr(self.lib, self.symbols[name])
        f.restype = None
        f.argtypes = [ctypes.c_uint32] * 3 + [ctypes.c_void_p] * 3
        f(m, k, n, A.data_ptr(), B.data_ptr(), Cc.data_ptr())

    def spmm(self, name, rows, shared, cols, csr, B, Cc):
        f = getattr(self.noguard, self.symbols[name])
        f.restype = None
        f.argtypes = [ctypes.c_uint32] * 3 + [self.SMatrixF32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        sm = self.SMatrixF32(csr.nnz, csr.elems.data_ptr(), csr.col_ind.data_ptr(), csr.row_off.data_ptr())
        f(rows, shared, cols, sm, csr.row_indices.data_ptr(), B.data_ptr(), Cc.data_ptr())


def wall_ms(torch, fn, reps):
    """Per-call wall time of a blocking call (the reference's entry points create a stream, launch,
    synchronise and destroy the stream: test/tensor_core_gemm_alpha_beta_1_driver.c.inc:139-149 times them so)."""
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / reps * 1e3


def comparisons_leg(torch, device, ours_gemm_ms):
    """Other implementations on the same GPU and the same seeded inputs.  GEMM: the reference's
    TensorCore2D kernels (row-major B, as its API has it) -- all 72 bf16 -> f32 instances swept at
    4096^3 as tuning/tune_tc2d.sh does, the fastest then timed at 8192^3 -- and cuBLAS with f32
    output through torch.  SpMM: the reference's kernels with the size guard compiled out, cuSPARSE
    through torch.sparse."""
    from kuiper_b200 import klas, synth
    out = {}
    flop = 2.0 * 8192 ** 3
    A, B = synth.gemm_bf16(1, 8192, 8192, 8192, b_col_major=False, device=device)
    D = torch.empty((8192, 8192), dtype=torch.float32, device=device)
    ours_rm = time_launches(torch, lambda: klas.gemm_tc(A, B, D=D), 20)
    out["gemm_bf16_8192_row_major_b"] = {"ours_ms": ours_rm, "ours_tflops": flop / ours_rm / 1e9,
                                         "ours_col_major_b_ms": ours_gemm_ms}
    try:
        f = lambda: torch.mm(A, B, out_dtype=torch.float32)
        f()
        what = "torch.mm(bf16, bf16, out_dtype=float32)"
    except Exception:
        f = lambda: torch.mm(A, B)
        what = "torch.mm(bf16, bf16) with bf16 output (this torch has no f32-output form)"
    ms = time_launches(torch, f, 20)
    out["gemm_bf16_8192_row_major_b"]["cublas"] = {"ms": ms, "tflops": flop / ms / 1e9, "call": what}
    if RefGpuLib.available():
        ref = RefGpuLib()
        n = 4096
        a4, b4, d4 = A[:n, :n].contiguous(), B[:n, :n].contiguous(), torch.empty((n, n), dtype=torch.float32, device=device)
        names = sorted(k for k in ref.symbols if k.startswith("Klas_GEMM_TensorCore2D_g_gemm_bf16_f32_"))
        best = None
        for nm in names:
            t = wall_ms(torch, lambda: ref.gemm(nm, n, n, n, a4, b4, d4), 2)
            if best is None or t < best[1]:
                best = (nm, t)
        t8 = wall_ms(torch, lambda: ref.gemm(best[0], 8192, 8192, 8192, A, B, D), 3)
        out["gemm_bf16_8192_row_major_b"]["reference_kernel"] = {
            "instance": best[0], "swept": len(names), "sweep": "per-call wall time at 4096^3, 2 calls each",
            "ms_per_call_4096": best[1], "ms_per_call_8192": t8, "tflops_8192": flop / t8 / 1e9,
            "note": "the reference's entry points are blocking (fresh stream, launch, sync, destroy); ours above is device time"}
    del A, B, D
    torch.cuda.empty_cache()

    rows = shared = Spmm.ROWS
    cols = Spmm.COLS
    csr = synth.csr_poisson(4, rows, shared, 64.0, device=device)
    Bd = synth.spmm_dense_b(4, shared, cols, device=device)
    Cd = torch.empty((rows, cols), device=device)
    sp = torch.sparse_csr_tensor(csr.row_off.long(), csr.col_ind.long(), csr.elems, size=(rows, shared))
    ours = time_launches(torch, lambda: klas.spmm(csr, Bd, Cd), 20)
    ms = time_launches(torch, lambda: torch.sparse.mm(sp, Bd), 10)
    out["spmm_131072"] = {"ours_ms": ours, "cusparse": {"ms": ms, "call": "torch.sparse.mm(csr, dense)"}}
    if RefGpuLib.available() and ref.noguard is not None:
        theirs = torch.empty_like(Cd)
        res = {}
        for nm in ("Klas_SPMM_spmm_f32", "Klas_SPMM_g_spmm_f32_512x512x64"):
            if nm in ref.symbols:
                res[nm] = wall_ms(torch, lambda: ref.spmm(nm, rows, shared, cols, csr, Bd, theirs), 2)
        klas.spmm(csr, Bd, Cd)
        torch.cuda.synchronize()
        out["spmm_131072"]["reference_kernel"] = {
            "ms_per_call": res, "bit_equal_to_ours": bool(torch.equal(Cd, theirs)),
            "note": "the reference's wrappers abort at rows, shared or cols >= 10000 (dist/Klas_SPMM.cu:196-198); this is a "
                    "comparison copy with the guards compiled out (oracle/ref_wrap/ref_spmm_noguard.cu)"}
    else:
        out["spmm_131072"]["reference_kernel"] = "aborts by guard (rows >= 10000); comparison copy not built"
    return out


def pcie_probe(torch, device, seconds=0.5, mib=256):
    """Host<->device copy rates of this rank, pinned memory: host->device alone, device->host alone,
    both at once (GB/s; the third is the sum of the two directions).  Every rank of a job runs it
    at the same time, so the figures include the contention for the host's memory and PCIe roots."""
    n = mib << 20
    h_in = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(n, dtype=torch.uint8, device=device)
    d_out = torch.empty(n, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def run(h2d, d2h):
        reps, out = 1, 0.0
        while True:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(reps):
                if h2d:
                    with torch.cuda.stream(s1):
                        d_in.copy_(h_in, non_blocking=True)
                if d2h:
                    with torch.cuda.stream(s2):
                        h_out.copy_(d_out, non_blocking=True)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            out = (int(h2d) + int(d2h)) * n * reps / dt / 1e9
            if dt >= seconds or reps >= 4096:
                return out
            reps = max(reps * 2, int(reps * seconds / max(dt, 1e-4)) + 1)

    return {"h2d_gbs": run(True, False), "d2h_gbs": run(False, True), "both_gbs": run(True, True)}


def run_mg_api(args):
    """`--mg-api`: the headline workload through the multi-GPU entry points of the C ABI
    (klas_b200_mg_*), ONE process and one host thread driving args.gpus devices -- what a C or C++
    caller gets; no torch.distributed.  Timed as host wall-clock between two all-device
    synchronisations, max over devices by construction."""
    import torch
    from kuiper_b200 import _lib, synth
    lib = _lib.load()
    n = args.gpus
    if torch.cuda.device_count() < n:
        raise SystemExit("--mg-api --gpus %d needs %d visible devices" % (n, n))
    rows, N, K = GemmBf16.ROWS_PER_GPU, GemmBf16.N, GemmBf16.K
    devs = (ctypes.c_int * n)(*range(n))
    ctx = ctypes.c_void_p()
    _lib.check(lib.klas_b200_mg_create(devs, n, ctypes.byref(ctx)))
    A, B, D = [], [], []
    for i in range(n):
        dev = torch.device("cuda", i)
        a, bt = synth.gemm_bf16(1, rows * n, N, K, row0=i * rows, rows=rows, b_col_major=True, device=dev)
        A.append(a)
        B.append(bt)
        D.append(torch.empty((rows, N), dtype=torch.float32, device=dev))
    bounds = (ctypes.c_uint64 * (n + 1))(*[i * rows for i in range(n + 1)])
    pa = (ctypes.c_void_p * n)(*[t.data_ptr() for t in A])
    pb = (ctypes.c_void_p * n)(*[t.data_ptr() for t in B])
    pd = (ctypes.c_void_p * n)(*[t.data_ptr() for t in D])

    def step(gather=_lib.MG_NO_GATHER, full=None):
        _lib.check(lib.klas_b200_mg_gemm_tc(ctx, _lib.BF16, _lib.F32, _lib.B_COL_MAJOR, bounds, K, N, pa, pb, pd, gather, full))

    for _ in range(max(args.warmup, 3)):
        step()
    _lib.check(lib.klas_b200_mg_synchronize(ctx))
    sampler = ClockSampler(0)
    with sampler:
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        _lib.check(lib.klas_b200_mg_synchronize(ctx))
        dt = time.perf_counter() - t0
    flop = 2.0 * rows * n * N * K
    # one gathered pass, checked against the per-device blocks
    fulls = [torch.empty((rows * n, N), dtype=torch.float32, device=torch.device("cuda", i)) for i in range(n)]
    pf = (ctypes.c_void_p * n)(*[t.data_ptr() for t in fulls])
    step(_lib.MG_GATHER_ALL, pf)
    _lib.check(lib.klas_b200_mg_synchronize(ctx))
    gather_ok = all(torch.equal(fulls[i][j * rows:(j + 1) * rows].cpu(), D[j].cpu()) for i in (0, n - 1) for j in range(n))
    _lib.check(lib.klas_b200_mg_destroy(ctx))
    line = {"metric": "bf16_gemm_tflops", "value": flop * args.steps / dt / 1e12, "unit": "TFLOP/s", "n_gpus": n,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(GemmBf16.describe(n), api="klas_b200_mg_gemm_tc: one process, one host thread, %d devices" % n,
                           timing="host wall-clock between two all-device synchronisations"),
            "clocks": sampler.summary(), "gpu_launches": args.steps * n, "check": {"gather_ok": bool(gather_ok)}}
    print(json.dumps(line), flush=True)
    return 0


# --------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_bf16")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="leave out the sustained leg, the other configurations and the comparison rows")
    ap.add_argument("--mg-api", action="store_true",
                    help="gemm_bf16 through the multi-GPU C entry points: one process drives --gpus devices (no torchrun)")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="do not bind this rank's host thread and pinned buffers to the NUMA node of its GPU")
    ap.add_argument("--tc-mode", default="auto", choices=["auto", "single", "narrow", "slim", "pair", "wide"],
                    help="force one tile shape of the tensor-core kernel (profiler captures of the variants)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--attention-heads", type=int, default=256,
                    help="attention_f16 only: heads per GPU (256 is the bench size; fewer for profiler captures)")
    ap.add_argument("--softmax-log2n", type=int, default=28,
                    help="softmax_f32 only: log2 of the vector length (28 is the bench size; smaller for profiler captures)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        return run_reference_arm(args, rank, world)
    if args.mg_api:
        return run_mg_api(args)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # Libraries (NCCL's version banner, for one) may write to stdout; the contract is ONE JSON
    # line there, so stdout is parked on stderr until the line is printed.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from kuiper_b200 import _lib, klas, sharding  # noqa: F401  (fails loudly if libklas_b200.so is missing)
    # host placement: this rank's thread and the pinned buffers it allocates go to the socket its GPU hangs off
    numa = {"node": _lib.load().klas_b200_host_numa_node(), "bound": False}
    if not args.no_numa_bind:
        numa["bound"] = _lib.load().klas_b200_host_bind_near_device() == _lib.OK

    if args.tc_mode != "auto":
        klas.debug_set("tc_mode", args.tc_mode)
    wl = make_workload(args.workload, rank, world, device, args)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        wl.launch()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    sampler.recording = False
    with sampler:                     # the polling thread is up and warm before the region starts ...
        barrier()
        sampler.recording = True      # ... and keeps what it reads only while the timed launches run
        start.record()
        for _ in range(args.steps):
            wl.launch()
        stop.record()
        torch.cuda.synchronize()
        sampler.recording = False
    barrier()
    ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    total_ms = float(ms)
    units = torch.tensor([wl.per_step_units()], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    scale = 1e12 if wl.unit in ("TFLOP/s", "Tops/s") else 1e9
    value = float(units) * args.steps / (total_ms * 1e-3) / scale
    klas.gemm_tc_status()

    # parity of what was just timed, outside the timed region: sampled rows of every rank's block ...
    check = wl.check()
    if check is not None and world > 1:
        flags = torch.tensor([1.0 if check["ok"] else 0.0, check.get("max_rel_err", 0.0)], dtype=torch.float64, device=device)
        worst = flags.clone()
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        check = dict(check, ok=bool(flags[0] > 0), max_rel_err=float(worst[1]), ranks=world,
                     rows=check["rows"] * world)
    # ... and, with several ranks, one pass with C assembled on every rank (NCCL all-gather over
    # NVLink): each rank compares its own block of the gathered matrix bit for bit, and the other
    # ranks' blocks through a checksum every rank computed of its local block.
    if world > 1 and wl.name in ("gemm_bf16", "gemm_bf16_65536") and check is not None:
        ranks = sharding.Ranks(rank, world, local, device)
        ranges = [(r * wl.rows, (r + 1) * wl.rows) for r in range(world)]
        t0 = time.perf_counter()
        full = sharding.gemm_tc_sharded(wl.A, wl.Bt, ranges, ranks, gather=True, out_dtype=torch.float32, b_col_major=True)
        torch.cuda.synchronize()
        gather_s = time.perf_counter() - t0
        lo, hi = ranges[rank]
        mine_ok = bool(torch.equal(full[lo:hi], wl.D))
        sums = torch.zeros(world, dtype=torch.int64, device=device)
        sums[rank] = wl.D.view(torch.int32).to(torch.int64).sum()
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
        got = torch.stack([full[a:b].view(torch.int32).to(torch.int64).sum() for a, b in ranges])
        ok = torch.tensor([1.0 if (mine_ok and bool(torch.equal(got, sums))) else 0.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        check.update(gather_ok=bool(ok[0] > 0), gathered_shape=list(full.shape), gather_pass_seconds=gather_s,
                     gather="all_gather_into_tensor of the %d row blocks; own block compared bit for bit, the others by a "
                            "64-bit sum of their bit patterns" % world)
        del full
        torch.cuda.empty_cache()

    # end to end through the host-buffer C ABI (pinned host memory, H2D + kernel + D2H per step)
    wl.e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        wl.e2e_step()
    torch.cuda.synchronize()
    e2e_s = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_value = float(units) * args.e2e_steps / float(e2e_s) / scale
    # what the host links give every rank while all ranks copy at once
    barrier()
    probe = pcie_probe(torch, device)
    mine = torch.tensor([probe["h2d_gbs"], probe["d2h_gbs"], probe["both_gbs"], float(numa["node"]), float(numa["bound"]),
                         float(e2e_s)], dtype=torch.float64, device=device)
    per_rank = [torch.zeros_like(mine) for _ in range(world)]
    if world > 1:
        dist.all_gather(per_rank, mine)
    else:
        per_rank = [mine]

    if rank == 0:
        peaks = load_peaks()
        per_launch_ms = total_ms / args.steps
        clocks = sampler.summary()
        roofline = roofline_of(wl, per_launch_ms, peaks, clocks.get("sm_mhz"))
        if wl.name == "spmm":
            roofline["gather"] = spmm_gather_block(torch, wl, per_launch_ms)
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": per_launch_ms, "higher_is_better": True, "scaling": "weak" if wl.name in ("gemm_bf16", "softmax_f32", "attention_f16") else "strong",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    "steps": args.e2e_steps, "api": getattr(wl, "e2e_api", "klas_b200_*_host (C ABI, pinned host buffers)"),
                    "ms_per_call_per_rank": [float(t[5]) / args.e2e_steps * 1e3 for t in per_rank],
                    "h2d_gbs": [float(t[0]) for t in per_rank], "d2h_gbs": [float(t[1]) for t in per_rank],
                    "both_gbs": [float(t[2]) for t in per_rank],
                    "node_aggregate_gbs": {"h2d": sum(float(t[0]) for t in per_rank), "d2h": sum(float(t[1]) for t in per_rank),
                                           "both": sum(float(t[2]) for t in per_rank)},
                    "numa_node_per_rank": [int(t[3]) for t in per_rank], "numa_bound": [bool(t[4]) for t in per_rank],
                    "copy_rates_note": "pinned 256 MiB copies, all ranks at once: host->device alone, device->host alone, both"},
            "gpu_launches": args.steps * wl.launches_per_step,
            "roofline": roofline,
        }
        if check is not None:
            line["check"] = check
        extras = world == 1 and wl.name == "gemm_bf16" and not args.no_extras
        if extras:
            line["sustained"] = sustained_leg(torch, wl, local, peaks)
            # A short timed region can run below the maximum clock before the driver flags why (its
            # throttle reasons lag the clock by more than the region lasts); the seconds-long leg of
            # the same process shows the reason.
            ck, sk = line["clocks"], line["sustained"]["clocks"]
            if ck.get("sm_mhz") and ck.get("sm_max_mhz") and ck["sm_mhz"] < 0.9 * ck["sm_max_mhz"] and not ck["reasons"] and sk.get("reasons"):
                ck["note"] = ("no reason flagged within the %.0f ms timed region; the sustained leg of this process ran at %s MHz with %s"
                              % (line["ms_per_step"] * line["steps"], sk.get("sm_mhz"), "+".join(sk["reasons"])))
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline_leg(wl.name)
            if cb:
                line["cpu_baseline"] = cb
        if extras:
            ours_ms = per_launch_ms
            del wl
            torch.cuda.empty_cache()
            klas.release_workspace()
            line["configs"] = {}
            for name in ("spmm", "gemm_f16b", "gemm_u64", "gemm_f32"):
                try:
                    line["configs"][name] = config_leg(torch, name, device, peaks, args)
                except Exception as exc:     # one configuration failing must not lose the headline line
                    line["configs"][name] = {"error": "%s: %s" % (type(exc).__name__, exc)}
                klas.release_workspace()
            try:
                line["comparisons"] = comparisons_leg(torch, device, ours_ms)
            except Exception as exc:
                line["comparisons"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
