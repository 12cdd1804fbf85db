"""ctypes binding of libklas_b200.so.  There is no fallback: if the library is
missing or does not export a symbol of include/klas_b200.h, importing fails."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libklas_b200.so"

# klas_status / klas_dtype / klas_layout / klas_b_major of include/klas_b200.h
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_TOO_LARGE = range(6)
F32, F64, U32, U64, BF16, F16 = range(6)
RRR, CCC = 0, 1
B_ROW_MAJOR, B_COL_MAJOR = 0, 1
MAP_ID, MAP_SQRT, MAP_ABS, MAP_SQUARE, MAP_RELU, MAP_NEG = range(6)
COMB_NEW, COMB_AXPBY, COMB_MAX, COMB_MIN, COMB_MUL, COMB_RELU, COMB_SCALED = range(7)

MG_NO_GATHER, MG_GATHER_ALL, MG_GATHER_FIRST = range(3)
KNOB_TC_MODE, KNOB_TC_RASTER, KNOB_SIMT_SPLIT_K, KNOB_F64_MODE, KNOB_SIMT_TILE, KNOB_HOST_GRID, KNOB_SPMM_SLAB, KNOB_TC_KSPLIT, KNOB_TC_TAIL = range(9)

_u32, _u64, _vp, _int, _f32 = C.c_uint32, C.c_uint64, C.c_void_p, C.c_int, C.c_float

# name -> (restype, argtypes): every function declared in include/klas_b200.h
SIGNATURES = {
    "klas_b200_last_error": (C.c_char_p, []),
    "klas_b200_version": (_int, []),
    "klas_b200_sm_count": (_int, []),
    "klas_b200_gemm": (_int, [_int, _int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp, _vp, _vp]),
    "klas_b200_gemm_compensated": (_int, [_int, _int, _u64, _u64, _u64, _vp, _vp, _vp, _vp]),
    "klas_b200_gemm_tc": (_int, [_int, _int, _int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp,
                                  _f32, _f32, _vp, _vp]),
    "klas_b200_gemm_strided": (_int, [_int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _u64, _u64, _vp, _u64, _u64,
                                       _vp, _u64, _u64, _int, _int, _int, _vp]),
    "klas_b200_csr_count": (_int, [_int, _u32, _u32, _vp, _vp, _vp]),
    "klas_b200_csr_fill": (_int, [_int, _u32, _u32, _vp, _vp, _vp, _vp, _vp]),
    "klas_b200_csr_row_order_scratch_bytes": (C.c_size_t, [_u32]),
    "klas_b200_csr_row_order": (_int, [_u32, _vp, _vp, _vp, C.c_size_t, _vp]),
    "klas_b200_minplus_u16": (_int, [_u32, _u32, _u32, _vp, _vp, _vp, _vp]),
    "klas_b200_sdpa": (_int, [_int, _u32, _u64, _u64, _u64, _u64, _vp, _vp, _vp, _vp, _int, _vp, _f32, _vp]),
    "klas_b200_sdpa_fused": (_int, [_int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp, _f32, _vp]),
    "klas_b200_gemm_tc_fused": (_int, [_int, _int, _int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp,
                                        _f32, _f32, _int, _int, _int, _vp, _vp]),
    "klas_b200_gemm_tc_strided": (_int, [_int, _int, _int, _u32, _u64, _u64, _u64, _vp, _u64, _u64, _vp, _u64, _u64,
                                          _vp, _vp, _u64, _u64, _f32, _f32, _int, _int, _int, _vp, _vp]),
    "klas_b200_gemm_tc_status": (_int, [C.POINTER(_int)]),
    "klas_b200_gemm_tc_status_peek": (_int, []),
    "klas_b200_debug_wait_probe": (_int, [_u32, _vp, _vp]),
    "klas_b200_spmm": (_int, [_int, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "klas_b200_spmm_gather_probe": (_int, [_u32, _u32, _u32, _vp, _vp, _vp]),
    "klas_b200_gemm_host": (_int, [_int, _int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp, _vp]),
    "klas_b200_gemm_tc_host": (_int, [_int, _int, _int, _u32, _u64, _u64, _u64, _vp, _vp, _vp, _vp,
                                       _f32, _f32]),
    "klas_b200_spmm_host": (_int, [_int, _u32, _u32, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp]),
    "klas_b200_host_numa_node": (_int, []),
    "klas_b200_host_bind_near_device": (_int, []),
    "klas_b200_softmax_scratch_bytes": (C.c_size_t, [_u64, _u64]),
    "klas_b200_softmax": (_int, [_int, _int, _u64, _u64, _vp, _vp, C.c_size_t, _vp]),
    "klas_b200_softmax_host": (_int, [_int, _int, _u64, _u64, _vp]),
    "klas_b200_softmax_static": (_int, [_int, _int, _u64, _vp, _vp]),
    "klas_b200_rowscale": (_int, [_int, _int, _u64, _u64, _vp, _vp, _vp]),
    "klas_b200_reduce_scratch_bytes": (C.c_size_t, [_u64]),
    "klas_b200_reduce_sum": (_int, [_int, _u64, _vp, _vp, _vp, C.c_size_t, _vp]),
    "klas_b200_reduce_sum_host": (_int, [_int, _u64, _vp, _vp]),
    "klas_b200_mg_create": (_int, [_vp, _int, _vp]),
    "klas_b200_mg_destroy": (_int, [_vp]),
    "klas_b200_mg_count": (_int, [_vp]),
    "klas_b200_mg_stream": (_vp, [_vp, _int]),
    "klas_b200_mg_synchronize": (_int, [_vp]),
    "klas_b200_mg_row_blocks": (_int, [_u64, _int, _u64, _vp]),
    "klas_b200_mg_csr_row_ranges": (_int, [_vp, _u32, _int, _int, _vp]),
    "klas_b200_mg_broadcast": (_int, [_vp, _vp, C.c_size_t, _int]),
    "klas_b200_mg_gemm_tc": (_int, [_vp, _int, _int, _int, _vp, _u64, _u64, _vp, _vp, _vp, _int, _vp]),
    "klas_b200_mg_gemm_tc_batched": (_int, [_vp, _int, _int, _int, _vp, _u64, _u64, _u64, _vp, _vp, _vp, _int, _vp]),
    "klas_b200_mg_gemm": (_int, [_vp, _int, _vp, _u64, _u64, _vp, _vp, _vp, _int, _vp]),
    "klas_b200_mg_spmm": (_int, [_vp, _int, _vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
    "klas_b200_debug_set": (_int, [_int, _int]),
    "klas_b200_debug_get": (_int, [_int]),
    "klas_b200_gemm_tc_plan": (_int, [_u64, _u64, _u64, _u32, _int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "klas_b200_release_workspace": (_int, []),
}

_lib = None


class KlasError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__("klas status %d: %s" % (status, message))
        self.status = status


def load() -> C.CDLL:
    """Loads the shared library once and types every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            "%s not found: build it with `python -m kuiper_b200.build` (needs nvcc); "
            "there is no CPU or PyTorch fallback" % LIB_PATH)
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is missing
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        raise KlasError(status, load().klas_b200_last_error().decode())
