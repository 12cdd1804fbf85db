"""ctypes access to the reference's own extracted kernels compiled for sm_100a
(oracle/_ref/libklas_ref_gpu.so + symbols.json, built by oracle/build.py).  Test-side only."""
import ctypes as C
import json
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent.parent / "oracle" / "_ref"


class _SMatrixF32(C.Structure):
    _fields_ = [("nnz", C.c_uint32), ("elems", C.c_void_p), ("col_ind", C.c_void_p), ("row_off", C.c_void_p)]


class RefGpu:
    def __init__(self):
        self.lib = C.CDLL(str(REF_DIR / "libklas_ref_gpu.so"))
        self.symbols = json.loads((REF_DIR / "symbols.json").read_text())

    @staticmethod
    def available():
        return (REF_DIR / "libklas_ref_gpu.so").exists() and (REF_DIR / "symbols.json").exists()

    def fn(self, name, argtypes):
        f = getattr(self.lib, self.symbols[name])
        f.restype = None
        f.argtypes = argtypes
        return f

    def mnk(self, name, m, n, k, A, B, Cc, pre=()):
        """(pre..., m, n, k, gA, gB, gC) entry points; `pre` = leading (ctype, value) pairs."""
        f = self.fn(name, [t for t, _ in pre] + [C.c_uint32] * 3 + [C.c_void_p] * 3)
        f(*[v for _, v in pre], m, n, k, A.data_ptr(), B.data_ptr(), Cc.data_ptr())

    def spmm_f32(self, name, rows, shared, cols, csr, B, Cc):
        f = self.fn(name, [C.c_uint32] * 3 + [_SMatrixF32, C.c_void_p, C.c_void_p, C.c_void_p])
        sm = _SMatrixF32(csr.nnz, csr.elems.data_ptr(), csr.col_ind.data_ptr(), csr.row_off.data_ptr())
        f(rows, shared, cols, sm, csr.row_indices.data_ptr(), B.data_ptr(), Cc.data_ptr())
