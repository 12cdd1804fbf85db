"""numpy-facing binding of the CPU checkers.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline legs of bench.py.  The product package never imports this module.

`Oracle` wraps oracle/libklas_oracle.so (the restatement, always buildable with
gcc); `RefCpu` wraps oracle/_ref/libklas_ref_cpu.so (the reference's own host
loops, present only where the reference tree was available at build time).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

ORACLE_DIR = Path(__file__).resolve().parent
ORACLE_LIB = ORACLE_DIR / "libklas_oracle.so"
REF_CPU_LIB = ORACLE_DIR / "_ref" / "libklas_ref_cpu.so"

_sz, _vp, _int = C.c_size_t, C.c_void_p, C.c_int


def _p(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"], "array must be C-contiguous"
    return a.ctypes.data


def bf16_bits(t) -> np.ndarray:
    """uint16 bit patterns of a torch bf16/f16 tensor (on the CPU)."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


class Oracle:
    def __init__(self):
        if not ORACLE_LIB.exists():
            raise FileNotFoundError("%s missing: run `python oracle/build.py`" % ORACLE_LIB)
        self.lib = C.CDLL(str(ORACLE_LIB))
        self.lib.klas_oracle_max_threads.restype = _int
        for name in ("klas_oracle_sgemm_f32",):
            getattr(self.lib, name).argtypes = [_sz, _sz, _sz, C.c_float, C.c_float, _vp, _vp, _vp, _vp, _int]
        self.lib.klas_oracle_gemm_u32.argtypes = [_sz, _sz, _sz, C.c_uint32, C.c_uint32, _int, _vp, _vp, _vp, _int]
        self.lib.klas_oracle_gemm_u64.argtypes = [_sz, _sz, _sz, C.c_uint64, C.c_uint64, _int, _vp, _vp, _vp, _int]
        for name in ("klas_oracle_acc_f32", "klas_oracle_acc_f64", "klas_oracle_acc_bf16",
                     "klas_oracle_acc_f16", "klas_oracle_acc_bf16_bt", "klas_oracle_absacc_f64",
                     "klas_oracle_gemm_f32", "klas_oracle_gemm_f64", "klas_oracle_gemm_bf16_f32",
                     "klas_oracle_gemm_f16_f16"):
            getattr(self.lib, name).argtypes = [_sz, _sz, _sz, _vp, _vp, _vp, _int]
        self.lib.klas_oracle_batched_f32.argtypes = [_sz, _sz, _sz, _sz, _vp, _vp, _vp]
        self.lib.klas_oracle_spmm_u32.argtypes = [C.c_uint32, C.c_uint32, _vp, _vp, _vp, _vp, _vp, _int]
        self.lib.klas_oracle_spmm_f32.argtypes = [C.c_uint32, C.c_uint32, _vp, _vp, _vp, _vp, _vp, _vp, _int]
        self.lib.klas_oracle_dense_matmul_f32.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp]
        for name in ("klas_oracle_f64_to_f16_bits", "klas_oracle_f64_to_bf16_bits", "klas_oracle_f16_bits_to_f64"):
            getattr(self.lib, name).argtypes = [_vp, _vp, _sz]

    def softmax(self, x: np.ndarray, log: bool = False) -> np.ndarray:
        """Row-wise softmax (or log-softmax) in float64 of a 1-D or 2-D array."""
        x = np.ascontiguousarray(x, np.float64)
        out = np.empty_like(x)
        rows = x.reshape(-1, x.shape[-1])
        o2 = out.reshape(-1, x.shape[-1])
        self.lib.klas_oracle_softmax_f64.argtypes = [_vp, _vp, _sz, _int]
        for r in range(rows.shape[0]):
            self.lib.klas_oracle_softmax_f64(rows[r].ctypes.data, o2[r].ctypes.data, rows.shape[1], int(log))
        return out

    def minplus_u16(self, A: np.ndarray, B: np.ndarray, C: np.ndarray) -> np.ndarray:
        """C' = add(C, A (min,+) B) on uint16 path lengths with 0 = no path; returns a new array."""
        A, B = np.ascontiguousarray(A, dtype=np.uint16), np.ascontiguousarray(B, dtype=np.uint16)
        out = np.array(C, dtype=np.uint16, order="C", copy=True)
        m, k = A.shape
        k2, n = B.shape
        assert k == k2 and out.shape == (m, n)
        self.lib.klas_oracle_minplus_u16.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp]
        self.lib.klas_oracle_minplus_u16(m, n, k, _p(A), _p(B), _p(out))
        return out

    def sparsify(self, M: np.ndarray):
        """(row_off, elems, col_ind) of a dense float32 / uint32 matrix, entries != 0 in scan order."""
        M = np.ascontiguousarray(M)
        assert M.dtype in (np.float32, np.uint32) and M.ndim == 2
        rows, cols = M.shape
        words = M.view(np.uint32)
        row_off = np.empty(rows + 1, dtype=np.uint32)
        fn = self.lib.klas_oracle_sparsify32
        fn.argtypes = [_vp, _sz, _sz, _int, _vp, _vp, _vp]
        fn.restype = C.c_uint32
        nnz = fn(_p(words), rows, cols, int(M.dtype == np.float32), _p(row_off), None, None)
        elems = np.empty(nnz, dtype=np.uint32)
        col_ind = np.empty(nnz, dtype=np.uint32)
        if nnz:
            fn(_p(words), rows, cols, int(M.dtype == np.float32), _p(row_off), _p(elems), _p(col_ind))
        return row_off, elems.view(M.dtype), col_ind

    @staticmethod
    def row_order(row_off: np.ndarray) -> np.ndarray:
        """Rows by decreasing length, equal lengths by increasing row (a stable sort; the drivers'
        std::sort, test/spmm_common.c.inc:139-157, leaves ties open)."""
        lens = np.diff(row_off.astype(np.int64))
        return np.argsort(-lens, kind="stable").astype(np.uint32)

    def map16(self, bits: np.ndarray, kind: str, op: int) -> np.ndarray:
        """Element-wise operand map (0 id, 1 sqrt, 2 abs, 3 square, 4 relu, 5 neg) on bf16 / f16 bit
        patterns: evaluated in float, rounded once back to the 16-bit type."""
        bits = np.ascontiguousarray(bits, dtype=np.uint16)
        out = np.empty_like(bits)
        self.lib.klas_oracle_map16.argtypes = [_vp, _vp, _sz, _int, _int]
        self.lib.klas_oracle_map16(_p(bits), _p(out), bits.size, int(kind == "bf16"), int(op))
        return out

    @property
    def max_threads(self) -> int:
        return self.lib.klas_oracle_max_threads()

    # ---- double accumulators -------------------------------------------------
    def acc(self, A: np.ndarray, B: np.ndarray, kind: str | None = None, threads: int = 0) -> np.ndarray:
        """float64 A.B with the drivers' i-k-j double accumulation.  `kind` is 'bf16' or
        'f16' when A and B hold uint16 bit patterns."""
        m, k = A.shape
        k2, n = B.shape
        assert k == k2
        out = np.empty((m, n), dtype=np.float64)
        fn = {("float32", None): "klas_oracle_acc_f32", ("float64", None): "klas_oracle_acc_f64",
              ("uint16", "bf16"): "klas_oracle_acc_bf16", ("uint16", "f16"): "klas_oracle_acc_f16"}[(A.dtype.name, kind)]
        assert B.dtype == A.dtype
        getattr(self.lib, fn)(m, n, k, _p(A), _p(B), _p(out), threads)
        return out

    def acc_bf16_bt(self, A: np.ndarray, Bt: np.ndarray, threads: int = 0) -> np.ndarray:
        m, k = A.shape
        n, k2 = Bt.shape
        assert k == k2 and A.dtype == np.uint16 and Bt.dtype == np.uint16
        out = np.empty((m, n), dtype=np.float64)
        self.lib.klas_oracle_acc_bf16_bt(m, n, k, _p(A), _p(Bt), _p(out), threads)
        return out

    def absacc(self, A: np.ndarray, B: np.ndarray, threads: int = 0) -> np.ndarray:
        """|A|.|B| in float64: the component-wise scale of a relative-error bound."""
        A = np.ascontiguousarray(A, dtype=np.float64)
        B = np.ascontiguousarray(B, dtype=np.float64)
        out = np.empty((A.shape[0], B.shape[1]), dtype=np.float64)
        self.lib.klas_oracle_absacc_f64(A.shape[0], B.shape[1], A.shape[1], _p(A), _p(B), _p(out), threads)
        return out

    # ---- typed gold ------------------------------------------------------------
    def gemm(self, A: np.ndarray, B: np.ndarray, kind: str | None = None, threads: int = 0) -> np.ndarray:
        m, k = A.shape
        n = B.shape[1]
        if A.dtype == np.float32:
            out = np.empty((m, n), np.float32)
            self.lib.klas_oracle_gemm_f32(m, n, k, _p(A), _p(B), _p(out), threads)
        elif A.dtype == np.float64:
            out = np.empty((m, n), np.float64)
            self.lib.klas_oracle_gemm_f64(m, n, k, _p(A), _p(B), _p(out), threads)
        elif A.dtype == np.uint16 and kind == "bf16":
            out = np.empty((m, n), np.float32)
            self.lib.klas_oracle_gemm_bf16_f32(m, n, k, _p(A), _p(B), _p(out), threads)
        elif A.dtype == np.uint16 and kind == "f16":
            out = np.empty((m, n), np.uint16)
            self.lib.klas_oracle_gemm_f16_f16(m, n, k, _p(A), _p(B), _p(out), threads)
        else:
            raise TypeError(A.dtype)
        return out

    def sgemm_f32(self, alpha, beta, A, B, Cin, threads: int = 0) -> np.ndarray:
        m, k = A.shape
        n = B.shape[1]
        out = np.empty((m, n), np.float32)
        self.lib.klas_oracle_sgemm_f32(m, n, k, alpha, beta, _p(A), _p(B), _p(Cin), _p(out), threads)
        return out

    def gemm_int(self, A: np.ndarray, B: np.ndarray, Cin: np.ndarray | None = None, alpha: int = 1,
                 beta: int = 0, threads: int = 0) -> np.ndarray:
        """Wrapping u32/u64 product; with Cin computes beta*Cin + alpha*A.B."""
        m, k = A.shape
        n = B.shape[1]
        assert A.dtype in (np.uint32, np.uint64) and B.dtype == A.dtype
        out = np.zeros((m, n), A.dtype) if Cin is None else np.array(Cin, dtype=A.dtype, order="C")
        fn = self.lib.klas_oracle_gemm_u32 if A.dtype == np.uint32 else self.lib.klas_oracle_gemm_u64
        bits = 32 if A.dtype == np.uint32 else 64
        fn(m, n, k, alpha & ((1 << bits) - 1), beta & ((1 << bits) - 1), 0 if Cin is None else 1,
           _p(A), _p(B), _p(out), threads)
        return out

    def batched_f32(self, A: np.ndarray, B: np.ndarray) -> np.ndarray:
        b, m, k = A.shape
        n = B.shape[2]
        out = np.empty((b, m, n), np.float32)
        self.lib.klas_oracle_batched_f32(b, m, n, k, _p(A), _p(B), _p(out))
        return out

    # ---- SpMM ------------------------------------------------------------------
    def spmm_u32(self, rows, cols, elems, col_ind, row_off, B, threads: int = 0) -> np.ndarray:
        out = np.empty((rows, cols), np.uint32)
        self.lib.klas_oracle_spmm_u32(rows, cols, _p(elems), _p(col_ind), _p(row_off), _p(B), _p(out), threads)
        return out

    def spmm_f32(self, rows, cols, elems, col_ind, row_off, B, with_abs: bool = False, threads: int = 0):
        out = np.empty((rows, cols), np.float64)
        ab = np.empty((rows, cols), np.float64) if with_abs else None
        self.lib.klas_oracle_spmm_f32(rows, cols, _p(elems), _p(col_ind), _p(row_off), _p(B), _p(out),
                                      _p(ab) if with_abs else None, threads)
        return (out, ab) if with_abs else out

    def dense_matmul_f32(self, A, B) -> np.ndarray:
        out = np.empty((A.shape[0], B.shape[1]), np.float32)
        self.lib.klas_oracle_dense_matmul_f32(A.shape[0], A.shape[1], B.shape[1], _p(A), _p(B), _p(out))
        return out

    # ---- 16-bit conversions ------------------------------------------------------
    def to_f16_bits(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float64)
        out = np.empty(x.shape, np.uint16)
        self.lib.klas_oracle_f64_to_f16_bits(_p(x), _p(out), x.size)
        return out

    def to_bf16_bits(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float64)
        out = np.empty(x.shape, np.uint16)
        self.lib.klas_oracle_f64_to_bf16_bits(_p(x), _p(out), x.size)
        return out

    def f16_bits_to_f64(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, np.uint16)
        out = np.empty(x.shape, np.float64)
        self.lib.klas_oracle_f16_bits_to_f64(_p(x), _p(out), x.size)
        return out


class RefCpu:
    """The reference's own gold loops (cpu_mul / cpu_sgemm per element type, the u32 CSR loop)."""

    KINDS = {"f32": (np.float32, np.float32), "f64": (np.float64, np.float64),
             "u32": (np.uint32, np.uint32), "u64": (np.uint64, np.uint64),
             "bf16_f32": (np.uint16, np.float32), "f16_f16": (np.uint16, np.uint16)}

    def __init__(self):
        if not REF_CPU_LIB.exists():
            raise FileNotFoundError(str(REF_CPU_LIB))
        self.lib = C.CDLL(str(REF_CPU_LIB))

    @staticmethod
    def available() -> bool:
        return REF_CPU_LIB.exists()

    def cpu_mul(self, kind: str, A: np.ndarray, B: np.ndarray) -> np.ndarray:
        et, cet = self.KINDS[kind]
        assert A.dtype == et and B.dtype == et
        out = np.empty((A.shape[0], B.shape[1]), cet)
        fn = getattr(self.lib, "ref_cpu_mul_" + kind)
        fn.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp]
        fn(A.shape[0], A.shape[1], B.shape[1], _p(A), _p(B), _p(out))
        return out

    def cpu_sgemm(self, kind: str, A, B, Cin, alpha, beta) -> np.ndarray:
        et, cet = self.KINDS[kind]
        out = np.empty((A.shape[0], B.shape[1]), cet)
        al = np.array([alpha], dtype=cet)
        be = np.array([beta], dtype=cet)
        fn = getattr(self.lib, "ref_cpu_sgemm_" + kind)
        fn.argtypes = [_sz, _sz, _sz, _vp, _vp, _vp, _vp, _vp, _vp]
        fn(A.shape[0], A.shape[1], B.shape[1], _p(A), _p(B), _p(Cin), _p(al), _p(be), _p(out))
        return out

    def cpu_softmax(self, x: np.ndarray, log: bool = False) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float64)
        out = np.empty_like(x)
        fn = self.lib.ref_cpu_logsoftmax if log else self.lib.ref_cpu_softmax
        fn.argtypes = [_vp, _vp, _int]
        fn(_p(x), _p(out), x.size)
        return out

    def sparsify(self, M: np.ndarray):
        """The drivers' sparsify_f32 / sparsify_u32: (row_off, elems, col_ind)."""
        M = np.ascontiguousarray(M)
        rows, cols = M.shape
        fn = self.lib.ref_sparsify_f32 if M.dtype == np.float32 else self.lib.ref_sparsify_u32
        fn.argtypes = [_vp, _int, _int, _vp, _vp, _vp]
        fn.restype = C.c_uint32
        row_off = np.empty(rows + 1, dtype=np.uint32)
        nnz = fn(_p(M), rows, cols, _p(row_off), None, None)
        elems, col_ind = np.empty(nnz, dtype=M.dtype), np.empty(nnz, dtype=np.uint32)
        fn(_p(M), rows, cols, _p(row_off), _p(elems) if nnz else None, _p(col_ind) if nnz else None)
        return row_off, elems, col_ind

    def mk_row_indices(self, row_off: np.ndarray) -> np.ndarray:
        row_off = np.ascontiguousarray(row_off, dtype=np.uint32)
        out = np.empty(row_off.size - 1, dtype=np.uint32)
        self.lib.ref_mk_row_indices.argtypes = [_int, _vp, _vp]
        self.lib.ref_mk_row_indices(out.size, _p(row_off), _p(out))
        return out

    def mmsd_u32_rr(self, rows, shared, cols, elems, col_ind, row_off, B) -> np.ndarray:
        out = np.empty((rows, cols), np.uint32)
        fn = self.lib.ref_mmsd_u32_rr
        fn.argtypes = [C.c_uint32] * 4 + [_vp] * 5
        fn(rows, shared, cols, elems.size, _p(elems), _p(col_ind), _p(row_off), _p(B), _p(out))
        return out
