"""Parity of the CSR x dense kernel with the CPU oracle."""
import numpy as np
import pytest
import torch

from gpu_util import rel_err_componentwise
from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

TOL_SPMM = 1e-5


def run_f32(oracle, csr, B, **kw):
    Cg = klas.spmm(csr.to("cuda"), B.cuda(), **kw)
    want, scale = oracle.spmm_f32(csr.rows, B.shape[1], csr.elems.numpy(), csr.col_ind.numpy().view(np.uint32),
                                  csr.row_off.numpy().view(np.uint32), B.numpy(), with_abs=True)
    return Cg.cpu().numpy(), want, scale


@pytest.mark.parametrize("rows,shared,cols,mean", [
    (512, 4096, 256, 64.0),    # the benchmark's row statistics, two column slabs
    (300, 1000, 128, 20.0),
    (257, 513, 100, 40.0),     # cols % 4 == 0 but not a multiple of the slab
    (100, 64, 7, 9.0),         # scalar path (cols % 4 != 0)
    (64, 64, 33, 30.0),        # dense-ish rows, scalar path
    (2000, 3000, 512, 3.0),    # many short and empty rows, four slabs
    (40, 5000, 4, 100.0),      # long rows, one vector per row
])
def test_f32_matches_oracle(oracle, rows, shared, cols, mean):
    csr = synth.csr_poisson(4, rows, shared, mean)
    B = synth.spmm_dense_b(4, shared, cols)
    got, want, scale = run_f32(oracle, csr, B)
    assert rel_err_componentwise(got, want, scale) <= TOL_SPMM


def _counts_case(oracle, cnt, shared, cols, seed=21, value_kind="f32"):
    csr = synth.csr_from_counts(seed, cnt, shared, value_kind=value_kind)
    B = synth.spmm_dense_b(seed, shared, cols, value_kind=value_kind)
    got = klas.spmm(csr.to("cuda"), B.cuda()).cpu().numpy()
    if value_kind == "f32":
        want, scale = oracle.spmm_f32(csr.rows, cols, csr.elems.numpy(), csr.col_ind.numpy().view(np.uint32),
                                      csr.row_off.numpy().view(np.uint32), B.numpy(), with_abs=True)
        return rel_err_componentwise(got, want, scale)
    want = oracle.spmm_u32(csr.rows, cols, csr.elems.numpy().view(np.uint32), csr.col_ind.numpy().view(np.uint32),
                           csr.row_off.numpy().view(np.uint32), B.numpy().view(np.uint32))
    return 0.0 if np.array_equal(got.view(np.uint32), want) else 1.0


@pytest.mark.parametrize("cols", [256, 96, 10])
def test_long_rows_are_cut_across_ranges(oracle, cols):
    """Rows far longer than a work range (the kernel cuts rows of more than 1024 nonzeros at range
    boundaries and adds the pieces to C): a power-law matrix whose first rows are dense, a matrix
    that is one long row between runs of empty rows, and long rows back to back."""
    shared = 20000
    assert _counts_case(oracle, synth.power_law_counts(600, shared, 120.0), shared, cols) <= TOL_SPMM
    cnt = torch.zeros(700, dtype=torch.int64)
    cnt[350] = 15000
    assert _counts_case(oracle, cnt, shared, cols) <= TOL_SPMM
    cnt = torch.tensor([5000, 1025, 1024, 0, 0, 9000, 3, 20000, 20000, 1, 0, 2047, 64, 64, 64, 1100])
    assert _counts_case(oracle, cnt, shared, cols) <= TOL_SPMM


def test_long_rows_u32_bit_exact(oracle):
    """Wrapping integer sums are exact whatever the order of the pieces."""
    cnt = torch.tensor([7000, 0, 12000, 5, 1500, 0, 0, 2500, 64])
    assert _counts_case(oracle, cnt, 12000, 136, value_kind="u32") == 0.0


def test_runs_of_empty_rows_and_one_nonzero(oracle):
    cnt = torch.zeros(5000, dtype=torch.int64)
    cnt[4999] = 1
    assert _counts_case(oracle, cnt, 64, 128) <= TOL_SPMM
    cnt = torch.zeros(5000, dtype=torch.int64)
    cnt[0] = 40
    cnt[2500:2510] = 7
    assert _counts_case(oracle, cnt, 64, 36) <= TOL_SPMM


def test_short_rows_repeat_bit_for_bit():
    """Rows that stay on one warp (every row here) are summed in CSR order: two calls agree exactly."""
    csr = synth.csr_poisson(9, 5000, 9000, 64.0, device="cuda")
    B = synth.spmm_dense_b(9, 9000, 256, device="cuda")
    assert torch.equal(klas.spmm(csr, B), klas.spmm(csr, B))


def test_gather_probe_runs_and_writes_nothing():
    csr = synth.csr_poisson(9, 3000, 4000, 30.0, device="cuda")
    B = synth.spmm_dense_b(9, 4000, 200, device="cuda")
    keep = B.clone()
    klas.spmm_gather_probe(csr, B)
    torch.cuda.synchronize()
    assert torch.equal(B, keep)


def test_row_order_does_not_change_results(oracle):
    csr = synth.csr_poisson(6, 333, 777, 25.0)
    B = synth.spmm_dense_b(6, 777, 64)
    a = klas.spmm(csr.to("cuda"), B.cuda())
    b = klas.spmm(csr.to("cuda"), B.cuda(), use_row_indices=False)
    assert torch.equal(a, b)   # CSR-order accumulation per row: bit-identical whatever the schedule


def test_empty_rows_are_overwritten_with_zeros(oracle):
    csr = synth.csr_poisson(8, 128, 256, 0.7)
    B = synth.spmm_dense_b(8, 256, 48)
    Cc = torch.full((128, 48), 99.0, device="cuda")
    klas.spmm(csr.to("cuda"), B.cuda(), Cc)
    lens = np.diff(csr.row_off.numpy())
    assert (lens == 0).any()
    assert bool((Cc[torch.tensor(lens == 0)] == 0).all())


def test_nnz_zero():
    csr = synth.csr_poisson(8, 16, 32, 0.0)
    Cc = torch.full((16, 8), 5.0, device="cuda")
    klas.spmm(csr.to("cuda"), torch.ones((32, 8), device="cuda"), Cc)
    assert bool((Cc == 0).all())


def test_identity_and_single_per_row(oracle):
    """Shapes of the reference's SpMM driver cases (test/Test_Klas_SPMM__F32.cu:76-110)."""
    n, cols = 200, 96
    eye = synth.Csr(n, n, torch.ones(n), torch.arange(n, dtype=torch.int32),
                    torch.arange(n + 1, dtype=torch.int32), torch.arange(n, dtype=torch.int32))
    B = synth.spmm_dense_b(2, n, cols)
    assert torch.equal(klas.spmm(eye.to("cuda"), B.cuda()).cpu(), B)
    g = torch.Generator().manual_seed(0)
    colsel = torch.randint(0, n, (n,), generator=g, dtype=torch.int32)
    vals = torch.randint(1, 100, (n,), generator=g).float()
    one = synth.Csr(n, n, vals, colsel, torch.arange(n + 1, dtype=torch.int32), torch.arange(n, dtype=torch.int32))
    got = klas.spmm(one.to("cuda"), B.cuda()).cpu()
    assert torch.equal(got, vals[:, None] * B[colsel.long()])


@pytest.mark.parametrize("cols", [128, 30])
def test_u32_wraps_bit_exact(oracle, cols):
    csr = synth.csr_poisson(12, 400, 600, 30.0, value_kind="u32")
    csr.elems = (csr.elems.long() * 40000003 % (1 << 32)).to(torch.int64).to(torch.int32)   # force wrap-around
    B = (synth.spmm_dense_b(12, 600, cols, value_kind="u32").long() * 99991 % (1 << 31)).to(torch.int32)
    got = klas.spmm(csr.to("cuda"), B.cuda()).cpu().numpy().view(np.uint32)
    want = oracle.spmm_u32(400, cols, csr.elems.numpy().view(np.uint32), csr.col_ind.numpy().view(np.uint32),
                           csr.row_off.numpy().view(np.uint32), B.numpy().view(np.uint32))
    assert np.array_equal(got, want)


def test_full_size_properties():
    """At the benchmark's size (131072^2, Poisson(64), 256 columns) the oracle is too slow for the
    whole matrix; check (a) a sampled set of rows against an fp64 gather on the GPU, and
    (b) linearity in B, which holds bit for bit when B's entries are small integers."""
    rows = shared = 131072
    cols = 256
    csr = synth.csr_poisson(4, rows, shared, 64.0, device="cuda")
    B = synth.spmm_dense_b(4, shared, cols, device="cuda")
    Cg = klas.spmm(csr, B)
    sample = torch.arange(0, rows, 1021, device="cuda")
    ro = csr.row_off.long()
    for r in sample.tolist()[:64]:
        lo, hi = int(ro[r]), int(ro[r + 1])
        want = (csr.elems[lo:hi].double()[:, None] * B[csr.col_ind[lo:hi].long()].double()).sum(0)
        scale = (csr.elems[lo:hi].double()[:, None] * B[csr.col_ind[lo:hi].long()].double()).abs().sum(0)
        assert float(((Cg[r].double() - want).abs() / scale.clamp_min(1e-300)).max()) <= TOL_SPMM
    ints = csr.to("cuda")
    ints.elems = torch.round(csr.elems * 8)                      # small integers
    B1 = torch.round(B * 8)
    B2 = torch.roll(B1, 1, 0)
    assert torch.equal(klas.spmm(ints, B1 + B2), klas.spmm(ints, B1) + klas.spmm(ints, B2))
