"""Parity of the row-wise neighbours (softmax, log-softmax, row scaling, sum reduction) with the
CPU oracle, through the typed wrappers and through the reference's entry-point names."""
import numpy as np
import pytest
import torch

from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

# |got - want| bounds.  Softmax outputs lie in [0, 1]; the f32 kernels evaluate expf / logf
# (a few ulp) and sum in f32 over at most ~1e6 terms in a tree of partial sums.
TOL_SOFTMAX = {torch.float64: 1e-13, torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}
# log-softmax values reach a few tens in magnitude (f16 spacing there is 2^-5): absolute bounds.
TOL_LOGSOFTMAX = {torch.float64: 1e-11, torch.float32: 2e-5, torch.float16: 3.2e-2, torch.bfloat16: 0.26}


def values(seed, *shape, dtype=torch.float32, spread=4.0):
    count = int(np.prod(shape))
    x = synth.normal(seed, 11, 0, count, dtype=torch.float64).reshape(shape) * spread
    return x.to(dtype)


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16])
@pytest.mark.parametrize("n", [1, 7, 100, 4097, 16384, 16385, 1 << 20, (1 << 25) + 3])
@pytest.mark.parametrize("log", [False, True])
def test_vector_softmax(oracle, dtype, n, log):
    x = values(n % 97, n, dtype=dtype)
    want = oracle.softmax(x.double().numpy(), log=log)
    got = klas.softmax(x.cuda(), log=log).double().cpu().numpy()
    tol = (TOL_LOGSOFTMAX if log else TOL_SOFTMAX)[dtype]
    assert np.max(np.abs(got - want)) <= tol
    if not log and dtype != torch.float16:
        assert abs(got.sum() - 1.0) <= 1e-4


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 33), (5, 1), (64, 1000), (300, 257), (7, 70000),
                                       # rows held in registers by one warp: 1 to 8 packs per lane, ragged last pack
                                       (3, 8), (1000, 64), (77, 256), (515, 1024), (33, 2048), (9, 1016), (2, 4096),
                                       # rows held in registers by one CTA (2 to 8 packs per thread), then beyond that
                                       (5, 8192), (3, 16384), (2, 12296), (2, 32768), (2, 70008)])
@pytest.mark.parametrize("log", [False, True])
def test_row_softmax(oracle, dtype, rows, cols, log):
    x = values(rows + cols, rows, cols, dtype=dtype)
    want = oracle.softmax(x.double().numpy(), log=log)
    got = klas.softmax(x.cuda(), log=log).double().cpu().numpy()
    assert np.max(np.abs(got - want)) <= (TOL_LOGSOFTMAX if log else TOL_SOFTMAX)[dtype]


def test_softmax_extreme_values(oracle):
    # A huge spread must not overflow: the maximum is subtracted before exp.
    x = torch.tensor([1e4, -1e4, 0.0, 1e4 - 1.0, 88.0], dtype=torch.float32)
    got = klas.softmax(x.cuda()).cpu().double().numpy()
    want = oracle.softmax(x.double().numpy())
    assert np.all(np.isfinite(got)) and np.max(np.abs(got - want)) <= 2e-6
    same = torch.full((50000,), 3.0, dtype=torch.float32)
    got = klas.softmax(same.cuda()).cpu()
    assert torch.allclose(got, torch.full_like(got, 1 / 50000), rtol=1e-5)


@pytest.mark.parametrize("log", [False, True])
def test_masked_entries_contribute_nothing(oracle, log):
    # -inf marks a masked position: leading runs (whole packs, whole threads' shares), scattered ones.
    x = values(17, 70001)
    x[:5000] = -float("inf")
    x[20000:20003] = -float("inf")
    x[-1] = -float("inf")
    want = oracle.softmax(x.double().numpy(), log=log)
    masked = np.isneginf(x.numpy())
    for got in (klas.softmax(x.cuda(), log=log).cpu().double().numpy(),                        # one vector
                klas.softmax(x[:70000].reshape(7, 10000).cuda(), log=log).cpu().double().numpy()):  # rows
        ref = want if got.ndim == 1 else oracle.softmax(x[:70000].reshape(7, 10000).double().numpy(), log=log)
        mk = masked if got.ndim == 1 else masked[:70000].reshape(7, 10000)
        assert np.all(got[mk] == (-np.inf if log else 0.0))
        assert np.max(np.abs(got[~mk] - ref[~mk])) <= (2e-5 if log else 2e-6)


def test_unaligned_rows_and_offsets(oracle):
    # Rows that start off the 16-byte grid (odd column count) and a vector at an odd offset.
    x = values(19, 33, 1001)
    got = klas.softmax(x.cuda()).cpu().double().numpy()
    assert np.max(np.abs(got - oracle.softmax(x.double().numpy()))) <= 2e-6
    for dtype, off in [(torch.float32, 1), (torch.float16, 3), (torch.float64, 1)]:
        base = values(23, 50000 + off, dtype=dtype).cuda()
        view = base[off:]
        want = oracle.softmax(view.double().cpu().numpy())
        klas.softmax(view)
        assert np.max(np.abs(view.double().cpu().numpy() - want)) <= TOL_SOFTMAX[dtype]
        y = values(29, 4099 + off, dtype=dtype, spread=1.0)[off:]
        got = klas.reduce_sum(y.cuda()).item()
        assert abs(got - float(y.double().sum())) <= TOL_SOFTMAX[dtype] * float(y.double().abs().sum())


def test_softmax_empty_is_a_no_op():
    klas.softmax(torch.empty(0, device="cuda"))
    klas.softmax(torch.empty((0, 8), device="cuda"))


@pytest.mark.parametrize("dtype", [torch.float64, torch.float32, torch.float16])
@pytest.mark.parametrize("m,n", [(1, 1), (33, 65), (1000, 17), (5, 4096)])
def test_rowscale_is_the_rounded_product(dtype, m, n):
    s = values(1, m, dtype=dtype, spread=1.0)
    b = values(2, m, n, dtype=dtype, spread=1.0)
    want = (s.cuda()[:, None] * b.cuda())          # one rounding of an exact product: bit-exact
    got = klas.rowscale(s.cuda(), b.cuda().clone())
    assert torch.equal(got, want)
    bt = b.t().contiguous()                          # column-major data of the same matrix
    got = klas.rowscale(s.cuda(), bt.cuda().clone(), col_major=True)
    assert torch.equal(got, want.t().contiguous())


@pytest.mark.parametrize("n", [0, 1, 255, 4096, 100001, 1 << 24])
def test_integer_sums_wrap_exactly(n):
    x64 = synth.integers_u64(5, 12, 0, n)
    want64 = int(np.add.reduce(x64.numpy().view(np.uint64), dtype=np.uint64)) if n else 0
    assert (klas.reduce_sum(x64.cuda()).item() & (2**64 - 1)) == want64
    x32 = x64.to(torch.int32)
    want32 = int(np.add.reduce(x32.numpy().view(np.uint32), dtype=np.uint32)) if n else 0
    assert (klas.reduce_sum(x32.cuda()).item() & (2**32 - 1)) == want32


@pytest.mark.parametrize("dtype,tol", [(torch.float64, 1e-13), (torch.float32, 2e-6)])
@pytest.mark.parametrize("n", [1, 1000, 1 << 20])
def test_float_sums(dtype, tol, n):
    x = values(9, n, dtype=dtype, spread=1.0)
    want = float(np.sum(x.double().numpy()))
    scale = float(np.sum(np.abs(x.double().numpy())))
    got = klas.reduce_sum(x.cuda()).item()
    assert abs(got - want) <= tol * scale
    again = klas.reduce_sum(x.cuda()).item()
    assert got == again                              # fixed fold order: deterministic


def test_f16_sum():
    x = torch.full((4096,), 0.25, dtype=torch.float16)
    assert klas.reduce_sum(x.cuda()).item() == 1024.0   # accumulated in f32, rounded once


# ------------------------------------------------------------------ the reference's names
def test_reference_names_softmax(oracle):
    x = values(3, 5000)
    want = oracle.softmax(x.double().numpy())
    for name, args in [("Klas_Softmax_softmax_gpu_f32", ()), ("Klas_Softmax_softmax_gpu_n_f32", (256,))]:
        d = x.cuda()
        klas.call(name, *args, 5000, d)
        assert np.max(np.abs(d.cpu().double().numpy() - want)) <= 2e-6
    h = x.clone()
    klas.call("Klas_Softmax_softmax_f32", 5000, h)           # host-pointer variant
    assert np.max(np.abs(h.double().numpy() - want)) <= 2e-6
    h = x.double()
    klas.call("Klas_LogSoftmax_log_softmax_n_f64", 128, 5000, h)
    assert np.max(np.abs(h.numpy() - oracle.softmax(x.double().numpy(), log=True))) <= 1e-11


def test_reference_names_rows_and_reductions(oracle):
    x = values(4, 40, 300)
    d = x.cuda()
    klas.call("Klas_RowSoftmax_row_softmax_rm_f32", 40, 300, 128, d)
    assert np.max(np.abs(d.cpu().double().numpy() - oracle.softmax(x.double().numpy()))) <= 2e-6
    s, b = values(5, 40, spread=1.0), values(6, 40, 300, spread=1.0)
    d = b.cuda().clone()
    klas.call("Klas_RowScale_rowscale_f32_rowmajor", 40, 300, s.cuda(), d)
    assert torch.equal(d, s.cuda()[:, None] * b.cuda())
    u = synth.integers_u64(7, 12, 0, 9999)
    want = int(np.add.reduce(u.numpy().view(np.uint64), dtype=np.uint64))
    assert (klas.call("Klas_HReduce_reduce_u64_plus", 256, 9999, u.cuda()) & (2**64 - 1)) == want
    assert (klas.call("Klas_AtomicReduce_reduce_u64", 9999, u.cuda()) & (2**64 - 1)) == want
