"""Device-side CSR construction and the (min,+) product against the CPU oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu


def dense_matrix(seed, rows, cols, density, dtype):
    u = synth.unit_uniform(seed, 41, 0, rows * cols).reshape(rows, cols)
    vals = (synth.integers_below_2_32(seed, 42, 0, rows * cols).reshape(rows, cols) % 98 + 1)
    M = torch.where(u < density, vals, torch.zeros_like(vals))
    return M.to(torch.float32) if dtype == torch.float32 else M.to(torch.int32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.int32])
@pytest.mark.parametrize("rows,cols,density", [(1, 1, 1.0), (37, 100, 0.3), (300, 33, 0.5), (2049, 64, 0.1),
                                               (5000, 257, 0.02), (64, 64, 0.0), (3, 5000, 0.9)])
def test_csr_from_dense_matches_oracle(oracle, dtype, rows, cols, density):
    M = dense_matrix(rows + cols, rows, cols, density, dtype)
    csr = klas.csr_from_dense(M.cuda())
    torch.cuda.synchronize()
    npM = M.numpy() if dtype == torch.float32 else M.numpy().view(np.uint32)
    row_off, elems, col_ind = oracle.sparsify(npM)
    assert np.array_equal(csr.row_off.cpu().numpy().view(np.uint32), row_off)
    assert np.array_equal(csr.col_ind.cpu().numpy().view(np.uint32), col_ind)
    assert np.array_equal(csr.elems.cpu().numpy().view(np.uint32), elems.view(np.uint32))
    assert np.array_equal(csr.row_indices.cpu().numpy().view(np.uint32), oracle.row_order(row_off))


def test_float_zero_and_nan_rules(oracle):
    M = torch.tensor([[0.0, -0.0, float("nan"), 1e-45, 2.0]], dtype=torch.float32)
    csr = klas.csr_from_dense(M.cuda())
    assert csr.col_ind.cpu().tolist() == [2, 3, 4]        # -0.0 dropped, NaN and the subnormal kept


def test_built_csr_feeds_spmm(oracle):
    M = dense_matrix(9, 500, 700, 0.05, torch.float32)
    B = synth.spmm_dense_b(9, 700, 128)
    csr = klas.csr_from_dense(M.cuda())
    got = klas.spmm(csr, B.cuda()).cpu().double()
    want = M.double() @ B.double()
    scale = M.double().abs() @ B.double().abs()
    assert float(((got - want).abs() / scale.clamp(min=1e-300)).max()) <= 1e-5


def test_row_order_of_a_large_random_matrix(oracle):
    # more rows than one shared-memory run, not a power of two: exercises the global sort steps
    rows = 70001
    lens = (synth.integers_below_2_32(10, 43, 0, rows) % 200).to(torch.int32)
    row_off = torch.zeros(rows + 1, dtype=torch.int32)
    row_off[1:] = torch.cumsum(lens, 0)
    lib = klas._lib.load()
    d_off = row_off.cuda()
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    need = lib.klas_b200_csr_row_order_scratch_bytes(rows)
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    klas.check(lib.klas_b200_csr_row_order(rows, d_off.data_ptr(), out.data_ptr(), scratch.data_ptr(), need, None))
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle.row_order(row_off.numpy().view(np.uint32)))


# ------------------------------------------------------------------ (min,+)
def lengths(seed, rows, cols, density, top):
    u = synth.unit_uniform(seed, 44, 0, rows * cols).reshape(rows, cols)
    v = synth.integers_below_2_32(seed, 45, 0, rows * cols).reshape(rows, cols) % top + 1
    return torch.where(u < density, v, torch.zeros_like(v)).to(torch.int16)      # bit patterns of uint16


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (64, 64, 64), (130, 70, 33), (256, 384, 200), (257, 129, 1026)])
@pytest.mark.parametrize("top", [100, 32767, 32768, 65535])      # the last two force the wrap-exact pass
def test_minplus_matches_oracle(oracle, m, n, k, top):
    A, B, C = lengths(1, m, k, 0.3, top), lengths(2, k, n, 0.3, top), lengths(3, m, n, 0.2, top)
    want = oracle.minplus_u16(A.numpy().view(np.uint16), B.numpy().view(np.uint16), C.numpy().view(np.uint16))
    got = klas.minplus_u16(A.cuda(), B.cuda(), C.cuda().clone())
    assert np.array_equal(got.cpu().numpy().view(np.uint16), want)


def test_path_graph_by_repeated_squaring():
    """The reference driver's scenario (test/Test_Kuiper_GraphDist.cu:55-95) through the Python mirror."""
    n = 1026
    m1 = torch.zeros((n, n), dtype=torch.int16)
    m1[torch.arange(n - 1), torch.arange(1, n)] = 1
    a, b = m1.cuda(), m1.cuda().clone()
    length = 1
    while length < n:
        klas.call("Kuiper_GraphDist_matmul_dist_gpu", n, a, b)
        a, b = b, a
        length *= 2
    idx = torch.arange(n)
    want = torch.triu(idx[None, :] - idx[:, None], 1).to(torch.int16)
    assert torch.equal(a.cpu(), want)
