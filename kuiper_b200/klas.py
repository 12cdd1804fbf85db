"""Host-side mirror of the Klas entry points over the C ABI (include/klas_b200.h).

Two levels:

* `gemm`, `gemm_tc`, `spmm` -- typed wrappers that take CUDA tensors, launch on
  torch's current stream and return the output tensor;
* `call(name, *args)` -- the reference's own entry-point names
  (dist/Klas_GEMM_*.h, dist/Klas_SPMM.h) with the reference's argument order
  and guards, e.g.
  `call("Klas_GEMM_SHMem_g_matmul_f32_tile32_rrr", m, n, k, A, B, C)`.
  A violated guard raises `KlasGuardError` where the reference aborts.

torch is used for device memory and streams only; every flop runs in
libklas_b200.so.
"""
from __future__ import annotations

import ctypes as C
import re
from typing import Optional

import torch

from . import _lib
from ._lib import KlasError, check
from .synth import Csr

_DTYPES = {
    torch.float32: _lib.F32, torch.float64: _lib.F64,
    torch.int32: _lib.U32, torch.int64: _lib.U64,
    torch.bfloat16: _lib.BF16, torch.float16: _lib.F16,
}
for _name, _code in (("uint32", _lib.U32), ("uint64", _lib.U64)):
    if hasattr(torch, _name):
        _DTYPES[getattr(torch, _name)] = _code

_CTYPE = {_lib.F32: C.c_float, _lib.F64: C.c_double, _lib.U32: C.c_uint32, _lib.U64: C.c_uint64}


class KlasGuardError(ValueError):
    """A precondition the reference checks with KPR_GUARD (include/kuiper.h:57-66) does not hold."""


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError("unsupported dtype %s" % t.dtype) from None


def _dev(t: torch.Tensor, what: str) -> int:
    if not t.is_cuda:
        raise ValueError("%s must be a CUDA tensor" % what)
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous" % what)
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _scalar(code: int, value):
    """Host scalar of the matrix dtype, as the C ABI wants alpha/beta."""
    if code == _lib.BF16:
        bits = torch.tensor(float(value), dtype=torch.bfloat16).view(torch.int16).item() & 0xFFFF
        return C.c_uint16(bits)
    if code in (_lib.U32, _lib.U64):
        return _CTYPE[code](int(value) & ((1 << (32 if code == _lib.U32 else 64)) - 1))
    return _CTYPE[code](float(value))


def gemm(A: torch.Tensor, B: torch.Tensor, C_: Optional[torch.Tensor] = None, *, alpha=None,
         beta=None, layout: str = "rrr") -> torch.Tensor:
    """CUDA-core GEMM.  `A` is [batch,] m x k and `B` [batch,] k x n as seen through `layout`
    ("rrr": tensors are row-major m x k etc.; "ccc": tensors hold the column-major data, i.e.
    A.shape == (k, m), B.shape == (n, k), C.shape == (n, m)).  With alpha/beta given computes
    beta*C + alpha*A.B in place in `C_`, otherwise overwrites / allocates C."""
    code = _code(A)
    if B.dtype != A.dtype:
        raise TypeError("A and B dtypes differ")
    batch = 1
    if A.dim() not in (2, 3) or B.dim() != A.dim():
        raise ValueError("A and B must both be 2-D, or both 3-D with one page count (A %s, B %s); a matrix shared "
                         "by all pages goes through gemm_strided with a page stride of 0" % (tuple(A.shape), tuple(B.shape)))
    if A.dim() == 3:
        batch = A.shape[0]
        if B.shape[0] != batch:
            raise ValueError("A has %d pages, B %d" % (batch, B.shape[0]))
        a2, b2 = A.shape[1:], B.shape[1:]
    else:
        a2, b2 = A.shape, B.shape
    if layout == "rrr":
        m, k = a2
        k2, n = b2
        cshape = (m, n)
    elif layout == "ccc":
        k, m = a2
        n, k2 = b2
        cshape = (n, m)
    else:
        raise ValueError("layout must be 'rrr' or 'ccc'")
    if k != k2:
        raise ValueError("inner dimensions differ: %d vs %d" % (k, k2))
    if A.dim() == 3:
        cshape = (batch,) + tuple(cshape)
    if C_ is None:
        if alpha is not None:
            raise ValueError("alpha/beta need an existing C")
        C_ = torch.empty(cshape, dtype=A.dtype, device=A.device)
    elif tuple(C_.shape) != tuple(cshape) or C_.dtype != A.dtype:
        raise ValueError("C has shape %s / dtype %s, expected %s / %s"
                         % (tuple(C_.shape), C_.dtype, tuple(cshape), A.dtype))
    pa = pb = None
    if (alpha is None) != (beta is None):
        raise ValueError("give both alpha and beta or neither")
    if alpha is not None:
        sa, sb = _scalar(code, alpha), _scalar(code, beta)
        pa, pb = C.addressof(sa), C.addressof(sb)
    lib = _lib.load()
    with torch.cuda.device(A.device):
        check(lib.klas_b200_gemm(code, _lib.RRR if layout == "rrr" else _lib.CCC, batch, m, n, k,
                                 pa, pb, _dev(A, "A"), _dev(B, "B"), _dev(C_, "C"), _stream()))
    return C_


def gemm_compensated(A: torch.Tensor, B: torch.Tensor, C_: Optional[torch.Tensor] = None, *, layout: str = "rrr") -> torch.Tensor:
    """C = A.B with the accuracy of the reference's compensated sums (Klas_GEMM_Naive3_*): f32 is
    accumulated in f64 and rounded once; the other dtypes run as gemm.  2-D operands, layouts as gemm."""
    if A.dim() != 2 or B.dim() != 2 or B.dtype != A.dtype:
        raise ValueError("gemm_compensated takes two 2-D matrices of one dtype")
    if layout == "rrr":
        (m, k), (k2, n) = A.shape, B.shape
        cshape = (m, n)
    elif layout == "ccc":
        (k, m), (n, k2) = A.shape, B.shape
        cshape = (n, m)
    else:
        raise ValueError("layout must be 'rrr' or 'ccc'")
    if k != k2:
        raise ValueError("inner dimensions differ: %d vs %d" % (k, k2))
    if C_ is None:
        C_ = torch.empty(cshape, dtype=A.dtype, device=A.device)
    elif tuple(C_.shape) != cshape or C_.dtype != A.dtype:
        raise ValueError("C has the wrong shape or dtype")
    with torch.cuda.device(A.device):
        check(_lib.load().klas_b200_gemm_compensated(_code(A), _lib.RRR if layout == "rrr" else _lib.CCC, m, n, k,
                                                     _dev(A, "A"), _dev(B, "B"), _dev(C_, "C"), _stream()))
    return C_


def sdpa_fused(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, *, scale: Optional[float] = None) -> torch.Tensor:
    """softmax(scale * Q.K^T).V per head in one kernel (scores never leave the chip).  Q [..., l, e],
    K [..., s, e], V [..., s, e], f16 or bf16, contiguous, e = 64 or 128.  scale defaults to 1/sqrt(e)."""
    if Q.dtype not in (torch.float16, torch.bfloat16) or K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise TypeError("sdpa_fused needs f16 or bf16 tensors of one dtype")
    lead = tuple(Q.shape[:-2])
    l, e = Q.shape[-2:]
    s = K.shape[-2]
    if tuple(K.shape) != lead + (s, e) or tuple(V.shape) != lead + (s, e):
        raise ValueError("shapes do not match: %s %s %s" % (tuple(Q.shape), tuple(K.shape), tuple(V.shape)))
    pages = 1
    for d in lead:
        pages *= d
    out = torch.empty_like(Q)
    with torch.cuda.device(Q.device):
        check(_lib.load().klas_b200_sdpa_fused(_code(Q), pages, l, s, e, _dev(Q, "Q"), _dev(K, "K"), _dev(V, "V"),
                                               _dev(out, "out"), float(scale if scale is not None else e ** -0.5),
                                               _stream()))
    return out


def sdpa(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, bias: Optional[torch.Tensor] = None, *,
         scale: Optional[float] = None, scores: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax(scale * Q.K^T + bias).V per head.  Q [..., l, e], K [..., s, e], V [..., s, ev] (f16 or
    bf16, contiguous, same leading dimensions); `bias` [..., l, s] is overwritten with the
    probabilities; without it pass `scores` (same shape) to receive them.  With neither, and a head
    dimension of 64 or 128, the fused kernel runs instead (`sdpa_fused`).  scale defaults to 1/sqrt(e)."""
    if Q.dtype not in (torch.float16, torch.bfloat16) or K.dtype != Q.dtype or V.dtype != Q.dtype:
        raise TypeError("sdpa needs f16 or bf16 tensors of one dtype")
    if bias is None and scores is None and Q.shape[-1] in (64, 128) and V.shape[-1] == Q.shape[-1]:
        return sdpa_fused(Q, K, V, scale=scale)      # nobody asked for the probabilities: one kernel, scores on chip
    lead = tuple(Q.shape[:-2])
    l, e = Q.shape[-2:]
    s, e2 = K.shape[-2:]
    s2, ev = V.shape[-2:]
    if tuple(K.shape[:-2]) != lead or tuple(V.shape[:-2]) != lead or e2 != e or s2 != s:
        raise ValueError("shapes do not match: %s %s %s" % (tuple(Q.shape), tuple(K.shape), tuple(V.shape)))
    pages = 1
    for d in lead:
        pages *= d
    buf = bias if bias is not None else scores
    if buf is None:
        buf = torch.empty(lead + (l, s), dtype=Q.dtype, device=Q.device)
    if tuple(buf.shape) != lead + (l, s) or buf.dtype != Q.dtype:
        raise ValueError("bias / scores must have shape %s and dtype %s" % (lead + (l, s), Q.dtype))
    out = torch.empty(lead + (l, ev), dtype=Q.dtype, device=Q.device)
    with torch.cuda.device(Q.device):
        check(_lib.load().klas_b200_sdpa(_code(Q), pages, l, s, e, ev, _dev(Q, "Q"), _dev(K, "K"), _dev(V, "V"),
                                         _dev(buf, "bias"), int(bias is not None), _dev(out, "out"),
                                         float(scale if scale is not None else e ** -0.5), _stream()))
    return out


def csr_from_dense(M: torch.Tensor) -> Csr:
    """CSR form (values != 0 in column order, offsets, longest-first row order) of a dense 2-D f32 or
    32-bit integer CUDA tensor, built on the device.  One 4-byte read-back (nnz) sizes the arrays."""
    code = _code(M)
    if code not in (_lib.F32, _lib.U32) or M.dim() != 2:
        raise TypeError("csr_from_dense needs a 2-D f32 or 32-bit integer tensor")
    rows, cols = M.shape
    lib = _lib.load()
    dense = _dev(M, "M")
    with torch.cuda.device(M.device):
        row_off = torch.empty(rows + 1, dtype=torch.int32, device=M.device)
        check(lib.klas_b200_csr_count(code, rows, cols, dense, row_off.data_ptr(), _stream()))
        nnz = int(row_off[-1].item()) & 0xFFFFFFFF
        elems = torch.empty(nnz, dtype=M.dtype, device=M.device)
        col_ind = torch.empty(nnz, dtype=torch.int32, device=M.device)
        check(lib.klas_b200_csr_fill(code, rows, cols, dense, row_off.data_ptr(), elems.data_ptr() if nnz else None,
                                     col_ind.data_ptr() if nnz else None, _stream()))
        row_indices = torch.empty(rows, dtype=torch.int32, device=M.device)
        need = lib.klas_b200_csr_row_order_scratch_bytes(rows)
        scratch = torch.empty(max(need, 8), dtype=torch.uint8, device=M.device)
        check(lib.klas_b200_csr_row_order(rows, row_off.data_ptr(), row_indices.data_ptr(), scratch.data_ptr(), need, _stream()))
    return Csr(rows, cols, elems, col_ind, row_off, row_indices)


def minplus_u16(A: torch.Tensor, B: torch.Tensor, C_: torch.Tensor) -> torch.Tensor:
    """In place C_ = min(C_, A (min,+) B) on 16-bit path lengths held in int16 / uint16 tensors, 0 = no path."""
    ok = (torch.int16,) + ((torch.uint16,) if hasattr(torch, "uint16") else ())
    if A.dtype not in ok or B.dtype != A.dtype or C_.dtype != A.dtype:
        raise TypeError("minplus_u16 needs three 16-bit integer tensors of one dtype")
    m, k = A.shape
    k2, n = B.shape
    if k2 != k or tuple(C_.shape) != (m, n):
        raise ValueError("shapes do not match")
    with torch.cuda.device(A.device):
        check(_lib.load().klas_b200_minplus_u16(m, n, k, _dev(A, "A"), _dev(B, "B"), _dev(C_, "C"), _stream()))
    return C_


def gemm_strided(A: torch.Tensor, B: torch.Tensor, C_: torch.Tensor, *, alpha=None, beta=None,
                 map_a: Optional[str] = None, map_b: Optional[str] = None, comb: Optional[str] = None) -> torch.Tensor:
    """General batched CUDA-core GEMM on tensor VIEWS: A [batch, m, k], B [batch, k, n], C_ [batch, m, n]
    (or 2-D for one page) whose last dimension is contiguous; row and page strides are taken from the
    views, and an expanded (stride-0) batch dimension of A or B shares one matrix between the pages.
    C_ = comb(C_, map_a(A) . map_b(B)) in place; default comb: "axpby" when alpha/beta are given, else "new"."""
    code = _code(A)
    if B.dtype != A.dtype or C_.dtype != A.dtype:
        raise TypeError("A, B and C dtypes differ")
    if A.dim() == 2:
        A, B, C_ = A[None], B[None], C_[None]
    batch, m, k = A.shape
    if tuple(B.shape) != (batch, k, B.shape[2]) or tuple(C_.shape) != (batch, m, B.shape[2]):
        raise ValueError("shapes do not match: %s %s %s" % (tuple(A.shape), tuple(B.shape), tuple(C_.shape)))
    n = B.shape[2]
    for t, name in ((A, "A"), (B, "B"), (C_, "C")):
        if not t.is_cuda:
            raise ValueError("%s must be a CUDA tensor" % name)
        if t.shape[2] > 1 and t.stride(2) != 1:
            raise ValueError("%s: the last dimension must be contiguous" % name)
    if (alpha is None) != (beta is None):
        raise ValueError("give both alpha and beta or neither")
    try:
        ma, mb = _MAPS[map_a], _MAPS[map_b]
        cb = _COMBS[comb] if comb is not None else (_lib.COMB_AXPBY if alpha is not None else _lib.COMB_NEW)
    except KeyError as e:
        raise ValueError("unknown map or combine rule %s" % e) from None
    pa = pb = None
    if alpha is not None:
        sa_, sb_ = _scalar(code, alpha), _scalar(code, beta)
        pa, pb = C.addressof(sa_), C.addressof(sb_)
    with torch.cuda.device(A.device):
        check(_lib.load().klas_b200_gemm_strided(
            code, batch, m, n, k, pa, pb, A.data_ptr(), A.stride(1), A.stride(0) if batch > 1 else 0,
            B.data_ptr(), B.stride(1), B.stride(0) if batch > 1 else 0,
            C_.data_ptr(), C_.stride(1), C_.stride(0) if batch > 1 else 0, ma, mb, cb, _stream()))
    return C_


_MAPS = {None: _lib.MAP_ID, "id": _lib.MAP_ID, "sqrt": _lib.MAP_SQRT, "abs": _lib.MAP_ABS,
         "square": _lib.MAP_SQUARE, "relu": _lib.MAP_RELU, "neg": _lib.MAP_NEG}
_COMBS = {"new": _lib.COMB_NEW, "axpby": _lib.COMB_AXPBY, "max": _lib.COMB_MAX, "min": _lib.COMB_MIN,
          "mul": _lib.COMB_MUL, "relu": _lib.COMB_RELU, "scaled": _lib.COMB_SCALED}


def gemm_tc(A: torch.Tensor, B: torch.Tensor, *, out_dtype=torch.float32, b_col_major: bool = False,
            C_: Optional[torch.Tensor] = None, D: Optional[torch.Tensor] = None,
            alpha: float = 1.0, beta: float = 0.0, map_a: Optional[str] = None,
            map_b: Optional[str] = None, comb: Optional[str] = None) -> torch.Tensor:
    """Tensor-core GEMM D = out_dtype(alpha*A.B + beta*C) (or A.B when C_ is None).
    A: [batch,] rows x shared; B: [batch,] shared x cols, or [batch,] cols x shared when
    `b_col_major`.  Returns D (allocated when not given; pass D=C_ to accumulate in place).

    Fused hooks: `map_a` / `map_b` in {"sqrt", "abs", "square", "relu", "neg"} are applied to the
    operands inside the kernel; `comb` in {"new", "axpby", "max", "min", "mul", "relu", "scaled"} says how
    the product meets C_ (default: "axpby" with C_, "new" without)."""
    if A.dtype not in (torch.bfloat16, torch.float16) or B.dtype != A.dtype:
        raise TypeError("A and B must both be bf16 or both be f16")
    if A.dim() not in (2, 3) or B.dim() != A.dim() or (A.dim() == 3 and B.shape[0] != A.shape[0]):
        raise ValueError("A and B must both be 2-D, or both 3-D with one page count (A %s, B %s); the kernel reads one "
                         "page of B per page of A" % (tuple(A.shape), tuple(B.shape)))
    batch = A.shape[0] if A.dim() == 3 else 1
    rows, shared = A.shape[-2:]
    if b_col_major:
        cols, k2 = B.shape[-2:]
    else:
        k2, cols = B.shape[-2:]
    if k2 != shared:
        raise ValueError("inner dimensions differ: %d vs %d" % (shared, k2))
    dshape = ((batch,) if A.dim() == 3 else ()) + (rows, cols)
    if D is None:
        D = torch.empty(dshape, dtype=out_dtype, device=A.device)
    if tuple(D.shape) != dshape or D.dtype != out_dtype:
        raise ValueError("D has the wrong shape or dtype")
    pc = None
    if C_ is not None:
        if tuple(C_.shape) != dshape or C_.dtype != out_dtype:
            raise ValueError("C has the wrong shape or dtype")
        pc = _dev(C_, "C")
    lib = _lib.load()
    try:
        ma, mb = _MAPS[map_a], _MAPS[map_b]
        cb = _COMBS[comb] if comb is not None else (_lib.COMB_AXPBY if C_ is not None else _lib.COMB_NEW)
    except KeyError as e:
        raise ValueError("unknown map or combine rule %s" % e) from None
    bmaj = _lib.B_COL_MAJOR if b_col_major else _lib.B_ROW_MAJOR
    with torch.cuda.device(A.device):
        if map_a is None and map_b is None and comb is None:
            check(lib.klas_b200_gemm_tc(_code(A), _DTYPES[out_dtype], bmaj, batch, rows, shared, cols,
                                        _dev(A, "A"), _dev(B, "B"), pc, _dev(D, "D"),
                                        float(alpha), float(beta), None, _stream()))
        else:
            check(lib.klas_b200_gemm_tc_fused(_code(A), _DTYPES[out_dtype], bmaj, batch, rows, shared, cols,
                                              _dev(A, "A"), _dev(B, "B"), pc, _dev(D, "D"),
                                              float(alpha), float(beta), ma, mb, cb, None, _stream()))
    return D


def gemm_tc_strided(A: torch.Tensor, B: torch.Tensor, D: torch.Tensor, *, b_col_major: bool = False,
                    C_: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0,
                    map_a: Optional[str] = None, map_b: Optional[str] = None,
                    comb: Optional[str] = None) -> torch.Tensor:
    """Tensor-core GEMM on tensor VIEWS (windows of larger arrays): A [batch,] rows x shared, B [batch,]
    shared x cols (cols x shared when `b_col_major`), D [batch,] rows x cols, last dimension contiguous;
    row and page strides come from the views and must be multiples of 8 elements.  C_, when given,
    must have D's strides (pass C_=D to accumulate in place).  Hooks as in gemm_tc.  Returns D."""
    if A.dtype not in (torch.bfloat16, torch.float16) or B.dtype != A.dtype:
        raise TypeError("A and B must both be bf16 or both be f16")
    if A.dim() == 2:
        A, B, D3 = A[None], B[None], D[None]
        C3 = None if C_ is None else C_[None]
    else:
        D3, C3 = D, C_
    batch, rows, shared = A.shape
    cols, k2 = (B.shape[1], B.shape[2]) if b_col_major else (B.shape[2], B.shape[1])
    if k2 != shared or B.shape[0] != batch or tuple(D3.shape) != (batch, rows, cols):
        raise ValueError("shapes do not match: %s %s %s" % (tuple(A.shape), tuple(B.shape), tuple(D3.shape)))
    for t, name in ((A, "A"), (B, "B"), (D3, "D")) + (((C3, "C"),) if C3 is not None else ()):
        if not t.is_cuda:
            raise ValueError("%s must be a CUDA tensor" % name)
        if t.shape[2] > 1 and t.stride(2) != 1:
            raise ValueError("%s: the last dimension must be contiguous" % name)
        if batch > 1 and t.stride(0) == 0:
            raise ValueError("%s: pages that share one matrix (stride 0) are not served on this path" % name)
    if C3 is not None and (C3.dtype != D3.dtype or tuple(C3.shape) != tuple(D3.shape) or
                           (rows > 1 and C3.stride(1) != D3.stride(1)) or (batch > 1 and C3.stride(0) != D3.stride(0))):
        raise ValueError("C must have D's dtype, shape and strides")
    try:
        ma, mb = _MAPS[map_a], _MAPS[map_b]
        cb = _COMBS[comb] if comb is not None else (_lib.COMB_AXPBY if C_ is not None else _lib.COMB_NEW)
    except KeyError as e:
        raise ValueError("unknown map or combine rule %s" % e) from None
    page = (lambda t: t.stride(0) if batch > 1 else 0)
    row = (lambda t: t.stride(1) if t.shape[1] > 1 else 0)
    with torch.cuda.device(A.device):
        check(_lib.load().klas_b200_gemm_tc_strided(
            _code(A), _DTYPES[D3.dtype], _lib.B_COL_MAJOR if b_col_major else _lib.B_ROW_MAJOR, batch, rows, shared, cols,
            A.data_ptr(), row(A), page(A), B.data_ptr(), row(B), page(B),
            C3.data_ptr() if C3 is not None else None, D3.data_ptr(), row(D3), page(D3),
            float(alpha), float(beta), ma, mb, cb, None, _stream()))
    return D


_KNOBS = {"tc_mode": (_lib.KNOB_TC_MODE, {"auto": 0, "single": 1, "narrow": 2, "pair": 3, "wide": 4, "slim": 5}),
          "tc_raster": (_lib.KNOB_TC_RASTER, {"auto": 0}), "simt_split_k": (_lib.KNOB_SIMT_SPLIT_K, {"auto": 0}),
          "f64_mode": (_lib.KNOB_F64_MODE, {"auto": 0, "simt": 1}), "simt_tile": (_lib.KNOB_SIMT_TILE, {"auto": -1}),
          "host_grid": (_lib.KNOB_HOST_GRID, {"auto": -1}), "spmm_slab": (_lib.KNOB_SPMM_SLAB, {"auto": 0}),
          "tc_ksplit": (_lib.KNOB_TC_KSPLIT, {"auto": 0, "off": 1}),
          "tc_tail": (_lib.KNOB_TC_TAIL, {"auto": 0, "off": 1, "always": 2})}


def debug_set(knob: str, value="auto") -> None:
    """Forces one variant of a kernel choice the library otherwise makes itself (klas_b200_debug_set):
    knob in {"tc_mode", "tc_raster", "simt_split_k", "f64_mode", "simt_tile", "host_grid", "spmm_slab", "tc_ksplit", "tc_tail"}, value a name
    ("auto" restores the library's choice; tc_mode: "single", "narrow", "slim", "pair", "wide"; f64_mode: "simt") or an int."""
    code, names = _KNOBS[knob]
    check(_lib.load().klas_b200_debug_set(code, names[value] if isinstance(value, str) else int(value)))


def release_workspace() -> None:
    """Frees the device workspace that the host-buffer entry points keep on the current device."""
    check(_lib.load().klas_b200_release_workspace())


def gemm_tc_status() -> int:
    """Raises KlasError(ERR_TIMEOUT) if a bounded device-side wait of the tensor-core kernel
    gave up since the last call (synchronises the device); returns 0 otherwise."""
    site = C.c_int(0)
    check(_lib.load().klas_b200_gemm_tc_status(C.byref(site)))
    return site.value


def spmm(A: Csr, B: torch.Tensor, C_: Optional[torch.Tensor] = None, *,
         use_row_indices: bool = True) -> torch.Tensor:
    """C = CSR(A) . B for f32 (elems float32) or wrapping u32 (elems int32)."""
    code = _code(A.elems)
    if code not in (_lib.F32, _lib.U32) or B.dtype != A.elems.dtype:
        raise TypeError("spmm needs f32 or 32-bit integer elems and a B of the same dtype")
    shared, cols = B.shape
    if shared != A.shared:
        raise ValueError("B has %d rows, the CSR matrix %d columns" % (shared, A.shared))
    if C_ is None:
        C_ = torch.empty((A.rows, cols), dtype=B.dtype, device=B.device)
    elif tuple(C_.shape) != (A.rows, cols) or C_.dtype != B.dtype:
        raise ValueError("C has the wrong shape or dtype")
    ri = _dev(A.row_indices, "row_indices") if use_row_indices and A.row_indices is not None else None
    lib = _lib.load()
    with torch.cuda.device(B.device):
        check(lib.klas_b200_spmm(code, A.rows, shared, cols, A.nnz,
                                 _dev(A.elems, "elems") if A.nnz else None,
                                 _dev(A.col_ind, "col_ind") if A.nnz else None,
                                 _dev(A.row_off, "row_off"), ri, _dev(B, "B"), _dev(C_, "C"),
                                 _stream()))
    return C_


def spmm_gather_probe(A: Csr, B: torch.Tensor) -> None:
    """Issues the reads of B that spmm(A, B) issues (f32, cols % 4 == 0) and nothing else; time it
    to get the gather-rate ceiling of that product."""
    if B.dtype != torch.float32 or A.elems.dtype != torch.float32:
        raise TypeError("spmm_gather_probe needs f32 operands")
    shared, cols = B.shape
    if shared != A.shared:
        raise ValueError("B has %d rows, the CSR matrix %d columns" % (shared, A.shared))
    lib = _lib.load()
    with torch.cuda.device(B.device):
        check(lib.klas_b200_spmm_gather_probe(shared, cols, A.nnz, _dev(A.col_ind, "col_ind") if A.nnz else None,
                                              _dev(B, "B"), _stream()))


def softmax(a: torch.Tensor, *, log: bool = False) -> torch.Tensor:
    """In-place softmax (log-softmax with log=True) of a vector, or of every row of a row-major
    matrix; f16 / bf16 / f32 / f64.  Returns `a`."""
    if a.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64) or a.dim() not in (1, 2):
        raise TypeError("softmax needs a 1-D or 2-D f16/bf16/f32/f64 tensor")
    rows, cols = (1, a.shape[0]) if a.dim() == 1 else a.shape
    lib = _lib.load()
    with torch.cuda.device(a.device):
        need = lib.klas_b200_softmax_scratch_bytes(rows, cols)
        scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=a.device) if need else None
        check(lib.klas_b200_softmax(_code(a), int(log), rows, cols, _dev(a, "a"),
                                    scratch.data_ptr() if need else None, need, _stream()))
    return a


def rowscale(scale: torch.Tensor, b: torch.Tensor, *, col_major: bool = False) -> torch.Tensor:
    """In place b[r][c] = scale[r] * b[r][c].  `b` is m x n row-major, or (col_major) the n x m
    tensor that holds the column-major data of an m x n matrix.  Returns `b`."""
    if b.dtype != scale.dtype or b.dtype not in (torch.float16, torch.float32, torch.float64):
        raise TypeError("rowscale needs matching f16/f32/f64 tensors")
    m, n = (b.shape[1], b.shape[0]) if col_major else b.shape
    if scale.numel() != m:
        raise ValueError("scale has %d entries, the matrix %d rows" % (scale.numel(), m))
    with torch.cuda.device(b.device):
        check(_lib.load().klas_b200_rowscale(_code(b), int(col_major), m, n, _dev(scale, "scale"), _dev(b, "b"), _stream()))
    return b


def reduce_sum(a: torch.Tensor) -> torch.Tensor:
    """Sum of a 1-D tensor (f16/f32/f64 or wrapping 32/64-bit integers) as a 0-D device tensor."""
    lib = _lib.load()
    out = torch.empty((), dtype=a.dtype, device=a.device)
    with torch.cuda.device(a.device):
        need = lib.klas_b200_reduce_scratch_bytes(a.numel())
        scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
        check(lib.klas_b200_reduce_sum(_code(a), a.numel(), _dev(a, "a") if a.numel() else None, out.data_ptr(),
                                       scratch.data_ptr(), need, _stream()))
    return out


# --------------------------------------------------------------------------- reference names
_TORCH_OF = {"f32": torch.float32, "f64": torch.float64, "u32": torch.int32, "u64": torch.int64,
             "bf16": torch.bfloat16, "f16": torch.float16}

_RE_TILED = re.compile(r"^Klas_GEMM_(SHMem|Tiled|BlockTiling1D)_g_(matmul|gemm)_(f32|f64|u32|u64)"
                       r"(?:_tile(16|32))?_rrr$")
_RE_BT2D = re.compile(r"^Klas_GEMM_BlockTiling2D_g_gemm_(f32|bf16)_(\d+)x(\d+)x(\d+)_(\d+)x(\d+)$")
_RE_NAIVE = re.compile(r"^Klas_GEMM_Naive([123])_g_matmul_(bf16|f32|f64|u32|u64)_(rrr|ccc)$")
_RE_NAIVE_B = re.compile(r"^Klas_GEMM_Naive([12])_batched_(matmul|gemm)_f32$")
_RE_TC2D = re.compile(r"^Klas_GEMM_TensorCore2D_g_gemm_(bf16_f32|f16_f16)_(\d+)x(\d+)x(\d+)"
                      r"_16x16x16_(\d+)x(\d+)$")
_RE_TC2D_TO = re.compile(r"^Klas_GEMM_TensorCore2D_To_g_gemm_bf16_f32_bf16_(\d+)x(\d+)x(\d+)"
                         r"_16x16x16_(\d+)x(\d+)$")
_RE_TC1D = re.compile(r"^Klas_GEMM_TensorCore_g_gemm_f16_(f16|f32)_(\d+)x(\d+)x(\d+)_(\d+)x(\d+)x(\d+)$")
_RE_SOFTMAX = re.compile(r"^Klas_(Softmax_softmax|LogSoftmax_log_softmax)_(gpu_)?(n_)?(f16|f32|f64)$")
_RE_ROWSOFTMAX = re.compile(r"^Klas_RowSoftmax_row_softmax_rm_(f32|f64)$")
_RE_ROWSCALE = re.compile(r"^Klas_RowScale_rowscale_(f16|f32|f64)_(rowmajor|colmajor)$")
_RE_REDUCE = re.compile(r"^Klas_(?:HReduce_reduce_(f16|f32|f64|u32|u64)_plus|AtomicReduce_reduce_(u32|u64|f32|f64))$")
_RE_GRAPHDIST = re.compile(r"^Kuiper_GraphDist_(matmul_dist_gpu|uu___is_D)$")
_RE_FUSED = re.compile(r"^Kuiper_Example_Fused_GEMM_gemm_sqrt_fused$")
_RE_SPMM = re.compile(r"^Klas_SPMM_(?:spmm_(f32|u32)|g_spmm_f32_(\d+)x(\d+)x(\d+))$")


def _guard(cond: bool, text: str) -> None:
    if not cond:
        raise KlasGuardError("Guard failed: " + text)


def _view(t: torch.Tensor, dtype, *shape) -> torch.Tensor:
    if t.dtype != dtype:
        raise TypeError("expected %s, got %s" % (dtype, t.dtype))
    n = 1
    for s in shape:
        n *= s
    if t.numel() < n:
        raise ValueError("buffer of %d elements is too small for %s" % (t.numel(), shape))
    return t.reshape(-1)[:n].view(*shape)


def call(name: str, *args):
    """Runs the reference entry point `name` with the reference's positional arguments
    (device tensors where the reference takes device pointers).  Results land in the
    caller's output tensor, as with the reference; returns None."""
    m_ = _RE_TILED.match(name)
    if m_:
        family, kind, dt, tile = m_.groups()
        args = list(args)
        if tile is None:
            if family == "BlockTiling1D":
                raise KeyError(name)
            tile_v = int(args.pop(0))
            _guard(tile_v > 0, "tile > 0U")
        else:
            tile_v = int(tile)
        alpha = beta = None
        if kind == "gemm":
            alpha, beta = args.pop(0), args.pop(0)
        m, n, k, A, B, Cc = args
        if family == "BlockTiling1D":
            for v, nm in ((m, "m"), (k, "k"), (n, "n")):
                _guard(v % tile_v == 0, "%s %% %dU == 0U" % (nm, tile_v))
        t = _TORCH_OF[dt]
        gemm(_view(A, t, m, k), _view(B, t, k, n), _view(Cc, t, m, n), alpha=alpha, beta=beta)
        return None
    m_ = _RE_BT2D.match(name)
    if m_:
        dt, bm, bn, bk = m_.group(1), int(m_.group(2)), int(m_.group(3)), int(m_.group(4))
        alpha, beta, m, n, k, A, B, Cc = args
        _guard(m % bm == 0, "m %% %dU == 0U" % bm)
        _guard(k % bk == 0, "k %% %dU == 0U" % bk)
        _guard(n % bn == 0, "n %% %dU == 0U" % bn)
        t = _TORCH_OF[dt]
        gemm(_view(A, t, m, k), _view(B, t, k, n), _view(Cc, t, m, n), alpha=alpha, beta=beta)
        return None
    m_ = _RE_NAIVE.match(name)
    if m_:
        which, dt, lay = m_.groups()
        m, n, k, A, B, Cc = args
        t = _TORCH_OF[dt]
        mul = gemm_compensated if which == "3" else gemm   # Naive3: the reference's compensated sums
        if lay == "rrr":
            mul(_view(A, t, m, k), _view(B, t, k, n), _view(Cc, t, m, n))
        else:
            mul(_view(A, t, k, m), _view(B, t, n, k), _view(Cc, t, n, m), layout="ccc")
        return None
    m_ = _RE_NAIVE_B.match(name)
    if m_:
        kind = m_.group(2)
        args = list(args)
        alpha = beta = None
        if kind == "gemm":
            alpha, beta = args.pop(0), args.pop(0)
        batch, m, n, k, A, B, Cc = args
        t = torch.float32
        gemm(_view(A, t, batch, m, k), _view(B, t, batch, k, n), _view(Cc, t, batch, m, n),
             alpha=alpha, beta=beta)
        return None
    m_ = _RE_TC2D.match(name)
    if m_:
        dt, bm, bn, bk = m_.group(1), int(m_.group(2)), int(m_.group(3)), int(m_.group(4))
        rows, shared, cols, A, B, Cc = args
        _guard(rows % bm == 0, "rows %% %dU == 0U" % bm)
        _guard(shared % bk == 0, "shared %% %dU == 0U" % bk)
        _guard(cols % bn == 0, "cols %% %dU == 0U" % bn)
        tin, tout = (torch.bfloat16, torch.float32) if dt == "bf16_f32" else (torch.float16, torch.float16)
        gemm_tc(_view(A, tin, rows, shared), _view(B, tin, shared, cols), out_dtype=tout,
                D=_view(Cc, tout, rows, cols))
        return None
    m_ = _RE_TC2D_TO.match(name)
    if m_:
        bm, bn, bk = int(m_.group(1)), int(m_.group(2)), int(m_.group(3))
        rows, shared, cols, A, B, Cc, Dd, alpha, beta = args
        _guard(rows % bm == 0, "rows %% %dU == 0U" % bm)
        _guard(shared % bk == 0, "shared %% %dU == 0U" % bk)
        _guard(cols % bn == 0, "cols %% %dU == 0U" % bn)
        t = torch.bfloat16
        gemm_tc(_view(A, t, rows, shared), _view(B, t, shared, cols), out_dtype=t,
                C_=_view(Cc, t, rows, cols), D=_view(Dd, t, rows, cols), alpha=alpha, beta=beta)
        return None
    m_ = _RE_TC1D.match(name)
    if m_:
        acc = m_.group(1)
        bm, bn, bk, tm, tn, tk = (int(v) for v in m_.groups()[1:])
        if (bm, bn, bk, tm, tn, tk) == (8, 32, 16, 8, 32, 16):
            # This one name guards on 32 in every dimension: its block tile really is
            # 32x32x32 (dist/Klas_GEMM_TensorCore.cu:531-535, src/klas/Klas.GEMM.TensorCore.fst:14).
            bm, bk, bn = 32, 32, 32
        rows, shared, cols, A, B, Cc = args
        _guard(rows % bm == 0, "rows %% %dU == 0U" % bm)
        _guard(shared % bk == 0, "shared %% %dU == 0U" % bk)
        _guard(cols % bn == 0, "cols %% %dU == 0U" % bn)
        tout = torch.float16 if acc == "f16" else torch.float32
        cv = _view(Cc, tout, rows, cols)
        gemm_tc(_view(A, torch.float16, rows, shared), _view(B, torch.float16, shared, cols),
                out_dtype=tout, C_=cv, D=cv, alpha=1.0, beta=1.0)
        return None
    m_ = _RE_SPMM.match(name)
    if m_:
        rows, shared, cols, A, row_indices, B, Cc = args
        dt = torch.int32 if m_.group(1) == "u32" else torch.float32
        csr = Csr(rows, shared, A.elems, A.col_ind, A.row_off, row_indices)
        spmm(csr, _view(B, dt, shared, cols), _view(Cc, dt, rows, cols))
        return None
    m_ = _RE_SOFTMAX.match(name)
    if m_:
        unit, gpu, has_n, dt = m_.groups()
        args = list(args)
        if has_n:
            args.pop(0)                     # thread-count hint
        lena, a = args
        t = _TORCH_OF[dt]
        if gpu:
            softmax(_view(a, t, lena), log=unit.startswith("Log"))
        else:                               # host-pointer variants: the tensor lives on the CPU
            if a.is_cuda or a.dtype != t:
                raise TypeError("%s takes a host tensor of %s" % (name, t))
            check(_lib.load().klas_b200_softmax_host(_DTYPES[t], int(unit.startswith("Log")), 1, lena, a.data_ptr()))
        return None
    m_ = _RE_ROWSOFTMAX.match(name)
    if m_:
        m, n, _nth, a = args
        softmax(_view(a, _TORCH_OF[m_.group(1)], m, n))
        return None
    m_ = _RE_ROWSCALE.match(name)
    if m_:
        m, n, a, b = args
        t = _TORCH_OF[m_.group(1)]
        if m_.group(2) == "rowmajor":
            rowscale(_view(a, t, m), _view(b, t, m, n))
        else:
            rowscale(_view(a, t, m), _view(b, t, n, m), col_major=True)
        return None
    m_ = _RE_REDUCE.match(name)
    if m_:
        a = args[-1]
        count = args[-2]
        t = _TORCH_OF[m_.group(1) or m_.group(2)]
        return reduce_sum(_view(a, t, count)).item()
    if name == "Kuiper_GraphDist_uu___is_D":
        return True
    if name == "Kuiper_GraphDist_matmul_dist_gpu":
        size, a, b = args
        minplus_u16(a.view(-1)[:size * size].view(size, size), a.view(-1)[:size * size].view(size, size),
                    b.view(-1)[:size * size].view(size, size))
        return None
    if _RE_FUSED.match(name):
        m, n, k, A, B, Cc = args
        if n % 8 or k % 8:
            raise KlasGuardError("%s: n and k must be multiples of 8" % name)
        t = torch.float16
        gemm_tc(_view(A, t, m, k), _view(B, t, k, n), out_dtype=t, D=_view(Cc, t, m, n), map_a="sqrt")
        return None
    raise KeyError("unknown Klas entry point: %s" % name)


def gemm_tc_plan(rows: int, shared: int, cols: int, batch: int = 1, sm_count: int = 148) -> dict:
    """What gemm_tc would run for this shape on a device with `sm_count` SMs (klas_b200_gemm_tc_plan;
    needs no GPU): {"kind": "single" | "pair" | "wide", "tile_cols", "k_parts", "tail_cut"}."""
    kind, tile_cols, parts, tail = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    check(_lib.load().klas_b200_gemm_tc_plan(rows, shared, cols, batch, sm_count, C.byref(kind), C.byref(tile_cols),
                                             C.byref(parts), C.byref(tail)))
    return {"kind": ("single", "pair", "wide")[kind.value], "tile_cols": tile_cols.value, "k_parts": parts.value,
            "tail_cut": bool(tail.value)}
