"""Parity at the sizes the benchmark times, on the benchmark's own seeded inputs.

The CPU oracle cannot multiply 8192^3 in a test's time, so each configuration is checked two
ways: a sample of full rows against the oracle (fp64, the drivers' gold loop), and the WHOLE
result against the reference's own kernel for that path compiled for sm_100a (oracle/_ref),
where it is built.  Tolerances are the configurations' own: bf16 -> f32 2e-3, f16 -> f16 1e-2,
f32 SpMM 1e-5, all relative to (|A|.|B|)_ij."""
import numpy as np
import pytest
import torch

from gpu_util import rel_err_componentwise
from kuiper_b200 import klas, synth
from oracle_api import bf16_bits
from ref_gpu import RefGpu

pytestmark = pytest.mark.gpu


def _bits16(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def test_bf16_8192_cubed_seeded_rows_against_the_oracle(oracle):
    """BF16 x BF16 -> F32, M = N = K = 8192, A row-major, B column-major, N(0,1) seed 1 -- the
    headline launch itself: 64 full rows (4.3e9 multiply-adds) against the fp64 oracle."""
    n = 8192
    A, Bt = synth.gemm_bf16(1, n, n, n, b_col_major=True, device="cuda")
    D = klas.gemm_tc(A, Bt, out_dtype=torch.float32, b_col_major=True)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    rows = torch.arange(0, n, n // 64)[:64]
    a_rows = A[rows.cuda()].cpu()
    want = oracle.acc_bf16_bt(bf16_bits(a_rows), bf16_bits(Bt.cpu()))
    scale = (a_rows.double().abs().cuda() @ Bt.double().abs().t()).cpu().numpy()
    err = rel_err_componentwise(D[rows.cuda()].cpu().numpy(), want, scale)
    assert err <= 2e-3, "relative error %.3e" % err
    assert err <= 1e-5      # fp32 accumulation of exact products: far inside the tolerance


def test_bf16_8192_cubed_whole_matrix_against_the_reference_kernel():
    """The same product, every element, against Klas_GEMM_TensorCore2D (row-major B as its API has
    it; this library's row-major entry runs the same inputs)."""
    if not RefGpu.available():
        pytest.skip("oracle/_ref/libklas_ref_gpu.so not built")
    ref = RefGpu()
    n = 8192
    A, B = synth.gemm_bf16(1, n, n, n, b_col_major=False, device="cuda")
    mine = klas.gemm_tc(A, B, out_dtype=torch.float32)
    via_col_major = klas.gemm_tc(A, B.t().contiguous(), out_dtype=torch.float32, b_col_major=True)
    theirs = torch.zeros((n, n), device="cuda")
    ref.mnk("Klas_GEMM_TensorCore2D_g_gemm_bf16_f32_128x128x32_16x16x16_8x4", n, n, n, A, B, theirs)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    assert torch.equal(mine, via_col_major)     # both layouts of B: same tiles, same order, same bits
    worst = 0.0
    for lo in range(0, n, 1024):                # |A|.|B| in fp64, a block of rows at a time
        scale = A[lo:lo + 1024].double().abs() @ B.double().abs()
        worst = max(worst, float(((mine[lo:lo + 1024].double() - theirs[lo:lo + 1024].double()).abs() / scale).max()))
    assert worst <= 2e-3, worst


def test_f16_batched_2048_all_pages(oracle):
    """Batched F16 x F16 -> F16, 2048^3 pages, U[-0.5, 0.5) seed 2: every one of 8 pages -- 8 rows
    of each against the oracle, and each page whole against the reference's kernel."""
    pages, n = 8, 2048
    A, B = synth.gemm_f16_batched(2, pages, n, n, n, device="cuda")
    D = klas.gemm_tc(A, B, out_dtype=torch.float16)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    rows = torch.arange(0, n, n // 8)[:8].cuda()
    for p in range(pages):
        want = oracle.acc(_bits16(A[p][rows]), _bits16(B[p]), kind="f16")
        scale = (A[p][rows].double().abs() @ B[p].double().abs()).cpu().numpy()
        err = rel_err_componentwise(D[p][rows].double().cpu().numpy(), want, scale)
        assert err <= 1e-2, "page %d: %.3e" % (p, err)
    if not RefGpu.available():
        return
    ref = RefGpu()
    theirs = torch.zeros((n, n), dtype=torch.float16, device="cuda")
    for p in range(pages):
        ref.mnk("Klas_GEMM_TensorCore2D_g_gemm_f16_f16_128x128x32_16x16x16_8x4", n, n, n, A[p], B[p], theirs)
        scale = A[p].double().abs() @ B[p].double().abs()
        # the reference rounds its half accumulator after every 16-deep step; both stay within 1e-2
        assert float(((D[p].double() - theirs.double()).abs() / scale).max()) <= 1e-2, p


def test_spmm_131072_rows_against_the_oracle(oracle):
    """SpMM at 131072^2, Poisson(64), 256 columns, seed 4: 256 rows (taken as their own CSR
    matrix) against the oracle's CSR loop; every sampled row also repeats bit for bit on a second call."""
    rows = shared = 131072
    cols = 256
    csr = synth.csr_poisson(4, rows, shared, 64.0, device="cuda")
    B = synth.spmm_dense_b(4, shared, cols, device="cuda")
    C1 = klas.spmm(csr, B)
    C2 = klas.spmm(csr, B)
    assert torch.equal(C1, C2)
    pick = torch.arange(0, rows, rows // 256)[:256]
    ro = csr.row_off.long().cpu()
    lens = (ro[pick + 1] - ro[pick])
    sub_off = torch.zeros(pick.numel() + 1, dtype=torch.int64)
    sub_off[1:] = torch.cumsum(lens, 0)
    idx = torch.cat([torch.arange(int(ro[r]), int(ro[r + 1])) for r in pick.tolist()])
    el = csr.elems.cpu()[idx].numpy()
    ci = csr.col_ind.cpu()[idx].numpy().view(np.uint32)
    want, scale = oracle.spmm_f32(pick.numel(), cols, el, ci, sub_off.to(torch.int32).numpy().view(np.uint32),
                                  B.cpu().numpy(), with_abs=True)
    err = rel_err_componentwise(C1[pick.cuda()].cpu().numpy(), want, scale)
    assert err <= 1e-5, err


def test_spmm_power_law_rows_at_size():
    """The same size with row lengths ~ 1 / rank^0.8 (the first row is dense: 131072 nonzeros):
    sampled rows, the longest included, against an fp64 gather-and-sum."""
    rows = shared = 131072
    cols = 256
    csr = synth.csr_from_counts(4, synth.power_law_counts(rows, shared, 64.0, device="cuda"), shared, device="cuda")
    B = synth.spmm_dense_b(4, shared, cols, device="cuda")
    Cg = klas.spmm(csr, B)
    ro = csr.row_off.long()
    for r in [0, 1, 2, 5, 17, 100, 545, 546, 1000, 5000, 70000, rows - 1]:
        lo, hi = int(ro[r]), int(ro[r + 1])
        prod = csr.elems[lo:hi].double()[:, None] * B[csr.col_ind[lo:hi].long()].double()
        want, scale = prod.sum(0), prod.abs().sum(0)
        err = float(((Cg[r].double() - want).abs() / scale.clamp_min(1e-300)).max()) if hi > lo else float(Cg[r].abs().max())
        assert err <= 1e-5, (r, hi - lo, err)
