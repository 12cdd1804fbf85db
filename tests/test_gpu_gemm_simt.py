"""Parity of the CUDA-core GEMMs (f32 / f64 / u32 / u64 / bf16 storage) with the CPU oracle."""
import numpy as np
import pytest
import torch

from driver_inputs import tiled_inputs
from gpu_util import rel_err_componentwise
from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_F64 = 1e-13

SHAPES = [(1024, 1024, 1024), (128, 128, 16), (64, 64, 64), (257, 129, 65), (1, 1, 1), (33, 7, 1000), (300, 200, 100)]


def as_u(a: np.ndarray):
    return a.view(np.uint32) if a.dtype == np.int32 else a.view(np.uint64)


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_f32_matmul(oracle, m, n, k):
    A, B = synth.gemm_f32(0, m, n, k, device="cuda")
    Cg = klas.gemm(A, B)
    acc = oracle.acc(A.cpu().numpy(), B.cpu().numpy())
    scale = oracle.absacc(A.cpu().numpy(), B.cpu().numpy())
    assert rel_err_componentwise(Cg.cpu().numpy(), acc, scale) <= TOL_F32


@pytest.fixture(params=["tensor", "simt"])
def f64_mode(request):
    """fp64 products run on the FP64 tensor-core kernel by default and on the CUDA-core kernel on request."""
    klas.debug_set("f64_mode", "simt" if request.param == "simt" else "auto")
    yield request.param
    klas.debug_set("f64_mode", "auto")


@pytest.mark.parametrize("m,n,k,batch,layout", [(256, 128, 64, 1, "rrr"), (100, 36, 52, 1, "rrr"), (129, 67, 33, 3, "rrr"),
                                               (384, 192, 160, 2, "rrr"), (70, 130, 45, 1, "ccc"), (1, 1, 1, 1, "rrr"),
                                               (8, 8, 0, 1, "rrr")])
def test_f64_alpha_beta_batched_layouts(oracle, f64_mode, m, n, k, batch, layout):
    shape = lambda r, c: ((batch,) if batch > 1 else ()) + ((r, c) if layout == "rrr" else (c, r))
    gen = lambda seed, r, c: (synth.uniform(seed, 61, 0, batch * r * c, -1, 1, dtype=torch.float64).reshape(shape(r, c))).cuda()
    A, B, C0 = gen(1, m, max(k, 0)), gen(2, max(k, 0), n), gen(3, m, n)
    t = (lambda x: x) if layout == "rrr" else (lambda x: x.transpose(-1, -2))
    acc = t(A).cpu() @ t(B).cpu() if k else torch.zeros(((batch,) if batch > 1 else ()) + (m, n), dtype=torch.float64)
    bound = (t(A).abs().cpu() @ t(B).abs().cpu() if k else torch.zeros_like(acc)) * 0.7 + 0.3 * t(C0).abs().cpu() + 1e-300
    got = klas.gemm(A, B, C0.clone(), alpha=0.7, beta=-0.3, layout=layout)
    assert float(((t(got).cpu() - (0.7 * acc - 0.3 * t(C0).cpu())).abs() / bound).max()) <= TOL_F64
    got = klas.gemm(A, B, layout=layout)
    assert float(((t(got).cpu() - acc).abs() / (bound + 1e-300)).max()) <= TOL_F64


@pytest.mark.parametrize("m,n,k", SHAPES[1:])
def test_f64_matmul(oracle, f64_mode, m, n, k):
    A, B = synth.gemm_f32(5, m, n, k, device="cuda")
    A, B = A.double() + 1e-9, B.double() - 1e-9
    Cg = klas.gemm(A, B)
    acc = oracle.acc(A.cpu().numpy(), B.cpu().numpy())
    scale = oracle.absacc(A.cpu().numpy(), B.cpu().numpy())
    assert rel_err_componentwise(Cg.cpu().numpy(), acc, scale) <= TOL_F64


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (128, 64, 8), (129, 67, 33), (512, 384, 96)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_integer_matmul_wraps_bit_exact(oracle, m, n, k, dtype):
    a, b = synth.gemm_u64(3, m, n, k, full_range=True, device="cuda")
    if dtype == torch.int32:
        a, b = a.to(torch.int32), b.to(torch.int32)   # low 32 bits
    Cg = klas.gemm(a, b)
    want = oracle.gemm_int(as_u(a.cpu().numpy()), as_u(b.cpu().numpy()))
    assert np.array_equal(as_u(Cg.cpu().numpy()), want)


def test_u64_config_inputs_below_2_32(oracle):
    a, b = synth.gemm_u64(3, 512, 512, 512, device="cuda")
    Cg = klas.gemm(a, b)
    want = oracle.gemm_int(as_u(a.cpu().numpy()), as_u(b.cpu().numpy()))
    assert np.array_equal(as_u(Cg.cpu().numpy()), want)


@pytest.mark.parametrize("m,n,k", [(256, 128, 64), (100, 36, 52)])
def test_gemm_alpha_beta(oracle, m, n, k):
    A, B = synth.gemm_f32(8, m, n, k, device="cuda")
    C0 = synth.uniform(8, 6, 0, m * n, -1.0, 1.0, torch.float32, "cuda").view(m, n)
    Cg = klas.gemm(A, B, C0.clone(), alpha=0.7, beta=0.3)
    acc = oracle.acc(A.cpu().numpy(), B.cpu().numpy())
    want = 0.3 * C0.double().cpu().numpy() + 0.7 * acc
    scale = 0.3 * np.abs(C0.double().cpu().numpy()) + 0.7 * oracle.absacc(A.cpu().numpy(), B.cpu().numpy())
    assert rel_err_componentwise(Cg.cpu().numpy(), want, scale) <= TOL_F32
    # integers: beta*C + alpha*A.B mod 2^64
    a, b = synth.gemm_u64(9, m, n, k, full_range=True, device="cuda")
    c0 = synth.integers_u64(9, 5, 0, m * n, "cuda").view(m, n)
    cg = klas.gemm(a, b, c0.clone(), alpha=3, beta=(1 << 64) - 5)
    want = oracle.gemm_int(as_u(a.cpu().numpy()), as_u(b.cpu().numpy()), as_u(c0.cpu().numpy()), 3, (1 << 64) - 5)
    assert np.array_equal(as_u(cg.cpu().numpy()), want)


def test_gemm_reads_c_even_when_beta_is_zero():
    """beta*C + alpha*acc is evaluated as written (dist/Klas_GEMM_SHMem.cu:1079-1081): NaN in C
    survives beta = 0."""
    A, B = synth.gemm_f32(1, 64, 64, 64, device="cuda")
    C0 = torch.full((64, 64), float("nan"), device="cuda")
    assert bool(torch.isnan(klas.gemm(A, B, C0, alpha=1.0, beta=0.0)).all())
    assert not bool(torch.isnan(klas.gemm(A, B)).any())


def test_column_major_layout(oracle):
    m, n, k = 96, 40, 72
    A, B = synth.gemm_f32(2, m, n, k, device="cuda")
    Acm, Bcm = A.t().contiguous(), B.t().contiguous()       # (k, m) and (n, k): column-major data
    Ccm = klas.gemm(Acm, Bcm, layout="ccc")                   # (n, m) = column-major m x n
    acc = oracle.acc(A.cpu().numpy(), B.cpu().numpy())
    scale = oracle.absacc(A.cpu().numpy(), B.cpu().numpy())
    assert rel_err_componentwise(Ccm.t().cpu().numpy(), acc, scale) <= TOL_F32


def test_batched_f32_driver_inputs(oracle):
    """test/Test_Klas_GEMM_Naive1__F32_Batched.cu: batch 4, 64 x 64 x 32, index-formula inputs."""
    batch, m, n, k = 4, 64, 64, 32
    a = np.empty((batch, m, k), np.float32)
    b = np.empty((batch, k, n), np.float32)
    for bi in range(batch):
        a[bi] = 2 * np.arange(m)[:, None] + np.arange(k)[None, :] + bi
        b[bi] = np.arange(k)[:, None] + np.arange(n)[None, :] + bi
    want = oracle.batched_f32(a, b)
    got = klas.gemm(torch.tensor(a).cuda(), torch.tensor(b).cuda()).cpu().numpy()
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30)) <= 1e-3   # the driver's TOLERANCE
    c0 = np.ones((batch, m, n), np.float32)
    got2 = klas.gemm(torch.tensor(a).cuda(), torch.tensor(b).cuda(), torch.tensor(c0).cuda(), alpha=0.5, beta=2.0)
    assert np.allclose(got2.cpu().numpy(), 0.5 * want + 2.0, rtol=1e-5)


@pytest.mark.parametrize("kind,dt,tdt", [("f32", np.float32, torch.float32), ("f64", np.float64, torch.float64),
                                          ("u32", np.uint32, torch.int32), ("u64", np.uint64, torch.int64)])
def test_driver_inputs_by_reference_name(oracle, kind, dt, tdt):
    """The tiled drivers' defaults (1024^3, m1 = 2i+j, m2 = i+j) through the reference's names."""
    n = 1024
    m1, m2, _ = tiled_inputs(dt, n, n, n)
    A = torch.tensor(m1.view(np.int32) if kind == "u32" else m1.view(np.int64) if kind == "u64" else m1).cuda()
    B = torch.tensor(m2.view(np.int32) if kind == "u32" else m2.view(np.int64) if kind == "u64" else m2).cuda()
    gold = oracle.gemm(m1, m2) if kind in ("f32", "f64") else oracle.gemm_int(m1, m2)
    for name, pre in (("Klas_GEMM_SHMem_g_matmul_%s_rrr", (32,)), ("Klas_GEMM_SHMem_g_matmul_%s_tile16_rrr", ()),
                      ("Klas_GEMM_Tiled_g_matmul_%s_tile32_rrr", ()), ("Klas_GEMM_BlockTiling1D_g_matmul_%s_tile32_rrr", ()),
                      ("Klas_GEMM_Naive1_g_matmul_%s_rrr", ()), ("Klas_GEMM_Naive2_g_matmul_%s_rrr", ())):
        Cc = torch.zeros((n, n), dtype=tdt, device="cuda")
        klas.call(name % kind, *pre, n, n, n, A, B, Cc)
        got = Cc.cpu().numpy()
        if kind in ("u32", "u64"):
            assert np.array_equal(got.view(dt), gold), name      # EXACT in the drivers
        else:
            assert np.max(np.abs(got - gold) / np.abs(np.where(gold == 0, 1, gold))) <= 1e-3, name   # drivers' TOLERANCE


def test_bf16_storage_accumulates_in_f32(oracle):
    m, n, k = 128, 128, 256
    A, Bt = synth.gemm_bf16(4, m, n, k, b_col_major=False, device="cuda")
    Cc = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    klas.call("Klas_GEMM_Naive3_g_matmul_bf16_rrr", m, n, k, A, Bt, Cc)
    acc = A.double().cpu().numpy() @ Bt.double().cpu().numpy()
    scale = np.abs(A.double().cpu().numpy()) @ np.abs(Bt.double().cpu().numpy())
    assert rel_err_componentwise(Cc.double().cpu().numpy(), acc, scale) <= 2 ** -8


def test_guards_raise():
    z = torch.zeros(64 * 64, device="cuda")
    with pytest.raises(klas.KlasGuardError):
        klas.call("Klas_GEMM_BlockTiling2D_g_gemm_f32_128x128x32_8x8", 1.0, 0.0, 64, 64, 64, z, z, z)
    with pytest.raises(klas.KlasGuardError):
        klas.call("Klas_GEMM_BlockTiling1D_g_matmul_f32_tile32_rrr", 48, 64, 64, z, z, z)


def test_compensated_f32_keeps_what_cancellation_destroys():
    """Klas_GEMM_Naive3 adds with Kahan's correction (dist/Klas_GEMM_Naive3.cu:17-30).  Rows built to
    cancel -- +3e7, a term of order 1, -3e7, another small term, ... -- lose the small terms in a
    plain f32 sum (the running sum sits at 3e7, where f32 numbers are 2 apart, every other step);
    the compensated entry point (f64 accumulation of the exact products) must return the sum of the
    small terms to the last place, under the reference's name as well."""
    m, n, k = 65, 33, 4096
    g = torch.Generator().manual_seed(11)
    A = torch.rand((m, k), generator=g) + 0.5
    A[:, 0::4] = 3.0e7
    A[:, 2::4] = -3.0e7
    B = torch.ones((k, n))
    want = A.double() @ B.double()            # about 2048: the big terms cancel pair by pair
    ulp = 2.0 ** -12                          # spacing of f32 between 2048 and 4096
    got = klas.gemm_compensated(A.cuda(), B.cuda()).cpu()
    assert float((got.double() - want).abs().max()) <= ulp
    named = torch.zeros((m, n), device="cuda")
    klas.call("Klas_GEMM_Naive3_g_matmul_f32_rrr", m, n, k, A.cuda(), B.cuda(), named)
    assert torch.equal(named.cpu(), got)
    plain = klas.gemm(A.cuda(), B.cuda()).cpu()
    assert float((plain.double() - want).abs().max()) > 1.0     # the uncompensated f32 sum really does lose them


@pytest.mark.parametrize("m,n,k", [(1024, 1024, 1024), (512, 384, 2048), (128, 64, 512)])
def test_two_ctas_per_tile_along_k(oracle, m, n, k):
    """One part-filled wave of tiles is run with two CTAs per tile, each summing half of K and adding
    its half onto a zeroed C.  Against the oracle (f32, 1e-5), equal from call to call (two addends:
    no order dependence), and for wrapping integers bit-equal to the unsplit kernel."""
    A, B = synth.gemm_f32(0, m, n, k, device="cuda")
    try:
        klas.debug_set("simt_split_k", 1)
        whole = klas.gemm(A, B)
        klas.debug_set("simt_split_k", 2)
        split1 = klas.gemm(A, B)
        split2 = klas.gemm(A, B, torch.full((m, n), 7.0, device="cuda"))   # whatever C held before is gone
        klas.debug_set("simt_split_k", "auto")
        auto = klas.gemm(A, B)
        ua, ub = synth.gemm_u64(3, m, n, k, full_range=True, device="cuda")
        klas.debug_set("simt_split_k", 1)
        uw = klas.gemm(ua, ub)
        klas.debug_set("simt_split_k", 2)
        us = klas.gemm(ua, ub)
    finally:
        klas.debug_set("simt_split_k", "auto")
    acc = oracle.acc(A.cpu().numpy(), B.cpu().numpy())
    scale = oracle.absacc(A.cpu().numpy(), B.cpu().numpy())
    for got in (whole, split1, auto):
        assert rel_err_componentwise(got.cpu().numpy(), acc, scale) <= TOL_F32
    assert torch.equal(split1, split2)
    assert torch.equal(uw, us)


@pytest.mark.parametrize("dt", [torch.float32, torch.int32, torch.int64, torch.float64])
@pytest.mark.parametrize("m,n,k,batch", [(1000, 1000, 1000, 1), (130, 260, 36, 3), (1, 8, 8, 1), (515, 132, 2052, 1)])
def test_shapes_of_whole_vectors_but_not_whole_tiles(dt, m, n, k, batch):
    """Rows that are whole 16-byte vectors without being whole tiles take the vector kernel with
    guarded edges: checked against fp64 / wrapping integer arithmetic, with alpha and beta, and
    with sentinels on both sides of C."""
    klas.debug_set("f64_mode", "simt")
    try:
        if dt in (torch.int32, torch.int64):
            A = torch.randint(-2 ** 20, 2 ** 20, (batch, m, k), device="cuda", dtype=dt)
            B = torch.randint(-2 ** 20, 2 ** 20, (batch, k, n), device="cuda", dtype=dt)
            C0 = torch.randint(-2 ** 20, 2 ** 20, (batch, m, n), device="cuda", dtype=dt)
            want = torch.bmm(A.cpu().to(torch.int64), B.cpu().to(torch.int64))
            want_ab = (3 * want + 5 * C0.cpu().to(torch.int64)).to(dt)
            want = want.to(dt)       # wraps
        else:
            A = torch.randn(batch, m, k, device="cuda").to(dt)
            B = torch.randn(batch, k, n, device="cuda").to(dt)
            C0 = torch.randn(batch, m, n, device="cuda").to(dt)
            want = torch.bmm(A.double().cpu(), B.double().cpu())
            want_ab = 3 * want + 5 * C0.double().cpu()
        guard = 4096
        flat = torch.full((guard + batch * m * n + guard,), 7, device="cuda", dtype=dt)
        Cv = flat[guard:guard + batch * m * n].view(batch, m, n)
        klas.gemm(A, B, Cv)
        torch.cuda.synchronize()
        assert bool((flat[:guard] == 7).all()) and bool((flat[-guard:] == 7).all()), "wrote outside C"
        Cab = C0.clone()
        klas.gemm(A, B, Cab, alpha=3, beta=5)
        torch.cuda.synchronize()
        if dt in (torch.int32, torch.int64):
            assert torch.equal(Cv.cpu(), want) and torch.equal(Cab.cpu(), want_ab)
        else:
            scale = torch.bmm(A.double().abs().cpu(), B.double().abs().cpu())
            tol = 1e-5 if dt == torch.float32 else 1e-13
            assert float(((Cv.double().cpu() - want).abs() / scale).max()) <= tol
            assert float(((Cab.double().cpu() - want_ab).abs() / (3 * scale + 5 * C0.double().abs().cpu())).max()) <= tol
    finally:
        klas.debug_set("f64_mode", "auto")
