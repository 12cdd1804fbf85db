"""Parity of the general batched CUDA-core GEMM (row / page strides, shared operands, maps and
combine rules) with float64 and exact-integer restatements of the same formula."""
import numpy as np
import pytest
import torch

from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

MAPS = {None: lambda x: x, "sqrt": torch.sqrt, "abs": torch.abs, "square": lambda x: x * x,
        "relu": lambda x: torch.clamp(x, min=0), "neg": lambda x: -x}


def padded(seed, batch, rows, cols, ld, gap, dtype, positive=False):
    """[batch, rows, cols] view with row stride ld and `gap` unused elements between pages."""
    page = rows * ld + gap
    flat = synth.uniform(seed, 31, 0, batch * page, -1.0, 1.0, dtype=torch.float64)
    if positive:
        flat = flat.abs()
    flat = flat.to(dtype).cuda()
    return flat.as_strided((batch, rows, cols), (page, ld, 1)), flat


def want_f64(A, B, C, map_a, map_b, comb, alpha, beta):
    a, b, c = MAPS[map_a](A.double().cpu()), MAPS[map_b](B.double().cpu()), C.double().cpu()
    acc = a @ b
    scale = a.abs() @ b.abs()
    out = {"new": acc, "axpby": alpha * acc + beta * c, "max": torch.maximum(c, acc), "min": torch.minimum(c, acc),
           "mul": c * acc, "relu": torch.clamp(acc, min=0), "scaled": alpha * acc}[comb]
    bound = {"axpby": abs(alpha) * scale + abs(beta) * c.abs(), "mul": scale * c.abs()}.get(comb, scale + c.abs())
    return out, bound


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.float64, 1e-14)])
@pytest.mark.parametrize("batch,m,n,k,lda,ldb,ldc", [
    (3, 100, 72, 50, 50, 72, 72),       # contiguous rows, ragged tiles
    (2, 100, 72, 50, 67, 91, 80),       # padded rows, unaligned strides -> predicated kernel
    (2, 256, 256, 64, 68, 260, 264),    # tile multiples, 16-byte aligned strides -> vector kernel
    (1, 130, 40, 300, 304, 40, 44),
])
@pytest.mark.parametrize("map_a,map_b,comb", [(None, None, "new"), ("sqrt", "abs", "axpby"), ("square", "neg", "max"),
                                              ("relu", None, "mul"), (None, "relu", "relu"), ("abs", "abs", "min"), (None, None, "scaled")])
def test_float_pages(dtype, tol, batch, m, n, k, lda, ldb, ldc, map_a, map_b, comb):
    A, _ = padded(1, batch, m, k, lda, 8, dtype, positive=map_a == "sqrt")
    B, _ = padded(2, batch, k, n, ldb, 4, dtype)
    C, cflat = padded(3, batch, m, n, ldc, 12, dtype)
    before = cflat.clone()
    want, bound = want_f64(A, B, C, map_a, map_b, comb, 0.75, -1.5)
    klas.gemm_strided(A, B, C, alpha=0.75 if comb in ("axpby", "scaled") else None,
                      beta=-1.5 if comb == "axpby" else 0.0 if comb == "scaled" else None,
                      map_a=map_a, map_b=map_b, comb=comb)
    torch.cuda.synchronize()
    err = ((C.double().cpu() - want).abs() / bound.clamp(min=1e-300)).max()
    assert float(err) <= tol, float(err)
    # nothing between the rows or the pages was touched
    mask = torch.ones_like(cflat, dtype=torch.bool)
    mask.as_strided(C.shape, C.stride())[:] = False
    assert torch.equal(cflat[mask], before[mask])


def test_shared_operand_and_plain_entry_agree():
    """stride 0 on B multiplies every page of A by the same matrix; results equal the plain entry's bit for bit."""
    A = synth.uniform(4, 31, 0, 4 * 96 * 64, -1, 1).reshape(4, 96, 64).cuda()
    B = synth.uniform(5, 31, 0, 64 * 80, -1, 1).reshape(64, 80).cuda()
    C = torch.empty((4, 96, 80), device="cuda")
    klas.gemm_strided(A, B[None].expand(4, -1, -1), C)
    for p in range(4):
        assert torch.equal(C[p], klas.gemm(A[p].contiguous(), B))


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_wrapping_integers_exact(dtype):
    bits = 32 if dtype == torch.int32 else 64
    mask = (1 << bits) - 1
    raw = synth.integers_u64(6, 32, 0, 2 * (70 * 45 + 45 * 52 + 70 * 52)).numpy()
    a = raw[:2 * 70 * 45].reshape(2, 70, 45)
    b = raw[2 * 70 * 45:2 * 70 * 45 + 2 * 45 * 52].reshape(2, 45, 52)
    c = raw[-2 * 70 * 52:].reshape(2, 70, 52)
    to_t = lambda x: torch.from_numpy(x.astype(np.int64)).to(dtype).cuda()
    A, B, C = to_t(a), to_t(b), to_t(c)
    py = lambda x: [[int(v) & mask for v in row] for row in x]
    for map_a, comb in [(None, "new"), ("neg", "axpby"), ("square", "max")]:
        Cg = C.clone()
        klas.gemm_strided(A, B, Cg, alpha=3 if comb == "axpby" else None, beta=5 if comb == "axpby" else None,
                          map_a=map_a, comb=comb)
        got = Cg.cpu().numpy()
        for p in range(2):
            pa, pb, pc = py(A[p].cpu().numpy()), py(B[p].cpu().numpy()), py(C[p].cpu().numpy())
            for i in (0, 33, 69):
                for j in (0, 17, 51):
                    acc = 0
                    for kk in range(45):
                        x = pa[i][kk]
                        x = (-x) & mask if map_a == "neg" else (x * x) & mask if map_a == "square" else x
                        acc = (acc + x * pb[kk][j]) & mask
                    want = {"new": acc, "axpby": (5 * pc[i][j] + 3 * acc) & mask, "max": max(pc[i][j], acc)}[comb]
                    assert (int(got[p][i][j]) & mask) == want


def test_bad_arguments():
    A = torch.zeros((2, 8, 8), device="cuda")
    with pytest.raises(klas.KlasError):
        klas.gemm_strided(A, A, A[:1].expand(2, -1, -1))                 # pages of C overlap
    with pytest.raises(klas.KlasError):
        klas.gemm_strided(A.int(), A.int(), A.int().clone(), map_a="sqrt")   # sqrt on integers
    with pytest.raises(ValueError):
        klas.gemm_strided(A, A, A.clone(), comb="sum")
