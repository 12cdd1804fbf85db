"""The host-buffer entry points (klas_b200_*_host: H2D copies, kernel, D2H copy inside one call)
give the same results as the device-pointer entry points."""
import numpy as np
import pytest
import torch

from kuiper_b200 import _lib, klas, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,shared,cols,with_c", [(8192, 512, 1024, False), (1000, 264, 520, False),
                                                      (2304, 128, 256, True), (64, 64, 64, True)])
def test_gemm_tc_host_row_chunks(rows, shared, cols, with_c):
    A, Bt = synth.gemm_bf16(5, rows, cols, shared, b_col_major=True)
    C0 = synth.uniform(5, 3, 0, rows * cols, -1, 1, torch.float32).view(rows, cols) if with_c else None
    want = klas.gemm_tc(A.cuda(), Bt.cuda(), b_col_major=True, C_=C0.cuda() if with_c else None,
                        alpha=0.5, beta=2.0).cpu()
    hA, hB, hD = A.pin_memory(), Bt.pin_memory(), torch.empty((rows, cols)).pin_memory()
    hC = C0.pin_memory() if with_c else None
    lib = _lib.load()
    for _ in range(2):     # second call reuses the workspace and the streams
        hD.fill_(-1)
        _lib.check(lib.klas_b200_gemm_tc_host(_lib.BF16, _lib.F32, _lib.B_COL_MAJOR, 1, rows, shared, cols,
                                              hA.data_ptr(), hB.data_ptr(), hC.data_ptr() if with_c else None,
                                              hD.data_ptr(), 0.5, 2.0))
        assert torch.equal(hD, want)


@pytest.mark.parametrize("rows,shared,cols", [(4096, 256, 4096), (4608, 136, 4360), (8192, 64, 4104)])
@pytest.mark.parametrize("b_col_major", [True, False])
def test_gemm_tc_host_two_dimensional_schedule(rows, shared, cols, b_col_major):
    """Large single products without C are sent as alternating row blocks of A and column blocks of B, each
    arrival followed by the products it completes; every element is still one ascending-k accumulation, so
    the result equals the device entry point's bit for bit."""
    A, Bm = synth.gemm_bf16(6, rows, cols, shared, b_col_major=b_col_major)
    want = klas.gemm_tc(A.cuda(), Bm.cuda(), b_col_major=b_col_major).cpu()
    hA, hB, hD = A.pin_memory(), Bm.pin_memory(), torch.empty((rows, cols)).pin_memory()
    lib = _lib.load()
    for _ in range(2):
        hD.fill_(-1)
        _lib.check(lib.klas_b200_gemm_tc_host(_lib.BF16, _lib.F32, _lib.B_COL_MAJOR if b_col_major else _lib.B_ROW_MAJOR,
                                              1, rows, shared, cols, hA.data_ptr(), hB.data_ptr(), None, hD.data_ptr(),
                                              1.0, 0.0))
        assert torch.equal(hD, want)


def test_gemm_tc_host_batched_pages():
    batch, m, n, k = 11, 128, 136, 72
    A, B = synth.gemm_f16_batched(2, batch, m, n, k)
    want = klas.gemm_tc(A.cuda(), B.cuda(), out_dtype=torch.float16).cpu()
    hD = torch.empty((batch, m, n), dtype=torch.float16)
    _lib.check(_lib.load().klas_b200_gemm_tc_host(_lib.F16, _lib.F16, _lib.B_ROW_MAJOR, batch, m, k, n,
                                                  A.data_ptr(), B.data_ptr(), None, hD.data_ptr(), 1.0, 0.0))
    assert torch.equal(hD, want)


def test_gemm_host_u64_and_f32():
    a, b = synth.gemm_u64(3, 200, 96, 72, full_range=True)
    want = klas.gemm(a.cuda(), b.cuda()).cpu()
    out = torch.empty((200, 96), dtype=torch.int64)
    _lib.check(_lib.load().klas_b200_gemm_host(_lib.U64, _lib.RRR, 1, 200, 96, 72, None, None, a.data_ptr(),
                                               b.data_ptr(), out.data_ptr()))
    assert torch.equal(out, want)
    A, B = synth.gemm_f32(0, 128, 64, 32)
    C0 = torch.ones((128, 64))
    import ctypes
    al, be = ctypes.c_float(0.7), ctypes.c_float(0.3)
    want = klas.gemm(A.cuda(), B.cuda(), C0.clone().cuda(), alpha=0.7, beta=0.3).cpu()
    _lib.check(_lib.load().klas_b200_gemm_host(_lib.F32, _lib.RRR, 1, 128, 64, 32, ctypes.addressof(al),
                                               ctypes.addressof(be), A.data_ptr(), B.data_ptr(), C0.data_ptr()))
    assert torch.equal(C0, want)


def test_spmm_host():
    csr = synth.csr_poisson(4, 700, 900, 12.0)
    B = synth.spmm_dense_b(4, 900, 72)
    want = klas.spmm(csr.to("cuda"), B.cuda()).cpu()
    out = torch.empty((700, 72))
    _lib.check(_lib.load().klas_b200_spmm_host(_lib.F32, 700, 900, 72, csr.nnz, csr.elems.data_ptr(),
                                               csr.col_ind.data_ptr(), csr.row_off.data_ptr(),
                                               csr.row_indices.data_ptr(), B.data_ptr(), out.data_ptr()))
    assert torch.equal(out, want)
    assert _lib.load().klas_b200_release_workspace() == 0
