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
  gemm_f16b   batched f16 x f16 -> f16, 2048^3 pages, 64 / N pages per GPU.
  gemm_u64    wrapping u64 GEMM 4096^3, rows sharded.
  gemm_f32    f32 GEMM 1024^3 (single GPU only).
  spmm        CSR(131072^2, Poisson 64) x dense 131072 x 256 f32, CSR rows sharded;
              metric GB/s of compulsory bytes.
Shards need no data-path collective: every rank owns its rows (or pages) of A and C
and a replica of B.

`--impl reference` times the reference's own host gold loop (test/matmul_common.c.inc
cpu_mul, compiled unmodified into oracle/_ref) on the host cores, one instance per
hardware thread on disjoint row blocks of a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
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
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


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

    def result_scalar(self):
        return float(self.D[0, 0])

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
        self.traffic = NCU_TRAFFIC["softmax_f32"] if log2n == 28 else None   # the capture is scaled to the bench size only
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
def reference_cpu_gemm_bf16(seconds_target: float, threads: int):
    """Times the reference's cpu_mul (bf16 in, f32 out, double accumulation; compiled unmodified
    into oracle/_ref) -- or the oracle port when oracle/_ref is absent -- on a row sample of the
    gemm_bf16 workload, one instance per thread on disjoint row blocks.
    Returns (tflops, kind, cores, sample description, seconds)."""
    import numpy as np
    sys.path.insert(0, str(REPO / "oracle"))
    import build as oracle_build
    from oracle_api import Oracle, RefCpu, bf16_bits
    wl = GemmBf16.__new__(GemmBf16)
    rows_per_thread = 2
    a, b = GemmBf16.cpu_inputs(wl, rows_per_thread * threads)
    a_bits, b_bits = bf16_bits(a), bf16_bits(b)
    if RefCpu.available():
        ref = RefCpu()
        kind = "reference"

        def run_block(t):
            blk = np.ascontiguousarray(a_bits[t * rows_per_thread:(t + 1) * rows_per_thread])
            ref.cpu_mul("bf16_f32", blk, b_bits)
    else:
        oracle_build.build_oracle()
        orc = Oracle()
        kind = "port"

        def run_block(t):
            blk = np.ascontiguousarray(a_bits[t * rows_per_thread:(t + 1) * rows_per_thread])
            orc.gemm(blk, b_bits, kind="bf16", threads=1)

    def one_pass():
        ts = [threading.Thread(target=run_block, args=(t,)) for t in range(threads)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return time.perf_counter() - t0

    return one_pass, kind, rows_per_thread * threads, GemmBf16.cpu_units(wl, rows_per_thread * threads)


def run_reference_arm(args, rank, world):
    if rank != 0:
        return 0
    if args.workload != "gemm_bf16":
        print(json.dumps({"impl": "reference", "unavailable": "reference arm implemented for the gemm_bf16 headline workload only"}))
        return 0
    threads = os.cpu_count() or 1
    one_pass, kind, rows, units = reference_cpu_gemm_bf16(0, threads)
    for _ in range(max(args.warmup, 1)):
        one_pass()
    t = 0.0
    for _ in range(args.steps):
        t += one_pass()
    value = units * args.steps / t / 1e12
    sample = "%d rows of A (2 per thread) x full 8192 x 8192 B per step" % rows
    line = {
        "impl": "reference", "metric": "bf16_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(GemmBf16.describe(max(args.gpus, 1)), sample=sample, impl="host gold loop cpu_mul on a row sample"),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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


def cpu_baseline_leg(workload_name):
    """Single-threaded, as the reference's loop is written; ~10-20 s of CPU work."""
    if workload_name == "softmax_f32":
        return cpu_baseline_softmax()
    if workload_name != "gemm_bf16":
        return None
    one_pass, kind, rows, units = reference_cpu_gemm_bf16(0, 1)
    t1 = one_pass()
    reps = max(1, min(64, int(12.0 / max(t1, 1e-3))))
    t = sum(one_pass() for _ in range(reps))
    return {"value": units * reps / t / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
            "sample": "%d x (%d rows of A x full 8192 x 8192 B), single thread as written" % (reps, rows)}


# --------------------------------------------------------------------------- main
# DRAM traffic of one launch from an ncu capture of the same kernel (profiles/): bytes read + written.
NCU_TRAFFIC = {"gemm_bf16": 1.150e9, "spmm": 1.141e9, "gemm_u64": 2.163e9, "gemm_f32": 8.4e6, "softmax_f32": 3.18e9}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm_bf16")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--attention-heads", type=int, default=256,
                    help="attention_f16 only: heads per GPU (256 is the bench size; fewer for profiler captures)")
    ap.add_argument("--softmax-log2n", type=int, default=28,
                    help="softmax_f32 only: log2 of the vector length (28 is the bench size; smaller for profiler captures)")
    args = ap.parse_args()
    rank, world, local = dist_env()
    if args.impl == "reference":
        return run_reference_arm(args, rank, world)

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
    from kuiper_b200 import klas  # noqa: F401  (fails loudly if libklas_b200.so is missing)

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
    barrier()
    with sampler:
        start.record()
        for _ in range(args.steps):
            wl.launch()
        stop.record()
        torch.cuda.synchronize()
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

    if rank == 0:
        peaks = load_peaks()
        per_launch_ms = total_ms / args.steps
        if wl.bound == "tensor":
            achieved = wl.per_step_units() / (per_launch_ms * 1e-3) / 1e12
            peak, runit = peaks["bf16_tflops"], "TFLOP/s"
            peak_note = "cuBLAS bf16 burst, of %s" % peaks["source"]
        elif wl.bound == "hbm":
            achieved = wl.algorithmic_bytes / (per_launch_ms * 1e-3) / 1e9
            peak, runit = peaks["hbm_gbs"], "GB/s"
            peak_note = "stream copy, of %s" % peaks["source"]
        else:
            # CUDA-core GEMMs are issue-bound: reported against the nominal issue peak at max clock
            achieved = wl.per_step_units() / (per_launch_ms * 1e-3) / 1e12
            if wl.name == "gemm_u64":
                # a wrapping u64 multiply-add = one widening 32x32 multiply-add (2 issue slots of the
                # 64-lane integer-multiply pipe) + two 32-bit ones: 4 slots per MAC, 2 ops per MAC
                peak, runit = 2 * (64 / 4) * 148 * 1.965e9 / 1e12, "Tops/s"
                peak_note = "64 integer-multiply lanes/clk/SM, 4 slots per u64 MAC, 148 SMs, 1965 MHz (nominal)"
            else:
                peak, runit = 2 * 128 * 148 * 1.965e9 / 1e12, "TFLOP/s"
                peak_note = "2*128 lanes*148 SMs*1965 MHz FP32 issue peak (nominal)"
        extra = {}
        if wl.name == "spmm":
            # every nonzero moves 4*cols bytes of a random row of B through L2 whatever the schedule
            gather = wl.nnz * (8 + 4 * wl.COLS) + 4 * wl.rows * wl.COLS + 8 * wl.rows
            extra = {"l2_gather_bytes_per_launch": gather,
                     "l2_gather_achieved_gbs": gather / (per_launch_ms * 1e-3) / 1e9,
                     "l2_gather_note": "random 512-byte row segments of B; highest L2->SM rate measured on this GPU "
                                       "(tensor-core GEMM, 128x256 tiles) is 15600 GB/s"}
        roofline = {"bound": "tensor" if wl.bound == "tensor" else "hbm" if wl.bound == "hbm" else "issue",
                    "achieved": achieved, "peak": peak, "unit": runit, "frac": achieved / peak,
                    "traffic": getattr(wl, "traffic", NCU_TRAFFIC.get(wl.name)), "peak_note": peak_note,
                    "algorithmic_bytes_per_launch": wl.algorithmic_bytes,
                    "kernel_ms": per_launch_ms, **extra}
        line = {
            "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": per_launch_ms, "higher_is_better": True, "scaling": "weak" if wl.name in ("gemm_bf16", "softmax_f32", "attention_f16") else "strong",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config,
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h,
                    "steps": args.e2e_steps, "api": getattr(wl, "e2e_api", "klas_b200_*_host (C ABI, pinned host buffers)")},
            "gpu_launches": args.steps * wl.launches_per_step,
            "roofline": roofline,
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline_leg(wl.name)
            if cb:
                line["cpu_baseline"] = cb
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
