"""The tensor-core GEMM on windows of larger arrays (row and page strides in the tensor maps):
parity with the CPU oracle, bit-equality with the packed entry on packed copies of the same
windows, and the surrounding elements (NaN around the operands, a sentinel around D) untouched
and unread."""
import numpy as np
import pytest
import torch

from gpu_util import rel_err_componentwise, tc_reference
from kuiper_b200 import klas, synth
from kuiper_b200._lib import KlasError

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.float16: 1e-2, torch.bfloat16: 2e-2}


@pytest.fixture(autouse=True, params=["single", "narrow", "slim", "wide", "auto"])
def tc_mode(request):
    klas.debug_set("tc_mode", request.param)
    yield request.param
    klas.debug_set("tc_mode", "auto")
    assert klas.gemm_tc_status() == 0


def window(t, pad_rows, pad_cols, fill):
    """A view equal to `t` ([batch, r, c]) inside a larger array whose other elements are `fill`;
    the window starts 8 elements into a row (16 bytes for the 16-bit types) and one row down."""
    batch, r, c = t.shape
    big = torch.full((batch, r + pad_rows + 1, c + pad_cols + 8), fill, dtype=t.dtype, device=t.device)
    view = big[:, 1:1 + r, 8:8 + c]
    view.copy_(t)
    return big, view


CASES = [  # batch, rows, shared, cols
    (1, 128, 64, 256), (1, 200, 72, 136), (3, 192, 80, 328), (2, 512, 512, 512), (1, 1024, 2048, 1280), (5, 8, 8, 8)]


@pytest.mark.parametrize("batch,rows,shared,cols", CASES)
@pytest.mark.parametrize("b_col_major", [False, True])
@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.float16, torch.float16)])
def test_windows_equal_packed_and_oracle(oracle, batch, rows, shared, cols, b_col_major, in_dtype, out_dtype):
    pages = []
    for b in range(batch):                                  # one seeded draw per page
        a, bm = synth.gemm_bf16(21 + b, rows, cols, shared, b_col_major=b_col_major, device="cuda")
        pages.append((a.to(in_dtype) * 0.25, bm.to(in_dtype)))
    A = torch.stack([p[0] for p in pages])
    Bm = torch.stack([p[1] for p in pages])
    _, Av = window(A, 3, 16, float("nan"))
    _, Bv = window(Bm, 2, 24, float("nan"))
    sentinel = 12345.0
    Dbig, Dv = window(torch.zeros((batch, rows, cols), dtype=out_dtype, device="cuda"), 4, 8, sentinel)
    klas.gemm_tc_strided(Av, Bv, Dv, b_col_major=b_col_major)
    packed = klas.gemm_tc(A, Bm, out_dtype=out_dtype, b_col_major=b_col_major)
    torch.cuda.synchronize()
    assert torch.equal(Dv, packed)                         # same tiles, same order: bit for bit
    outside = torch.ones_like(Dbig, dtype=torch.bool)
    outside[:, 1:1 + rows, 8:8 + cols] = False
    assert bool((Dbig[outside] == sentinel).all())
    for b in range(batch):
        acc, scale = tc_reference(oracle, A[b].cpu(), Bm[b].cpu(), b_col_major)
        err = rel_err_componentwise(Dv[b].float().cpu().numpy(), acc, scale)
        assert err <= TOL[out_dtype], "page %d: relative error %.3e" % (b, err)


def test_combine_and_maps_on_windows(oracle):
    """C read and D written through the same window; a map on A."""
    batch, rows, shared, cols = 2, 320, 264, 200
    A, Bm = synth.gemm_bf16(22, rows, cols, shared, b_col_major=False, device="cuda")
    A = torch.stack([A, A.flip(0)])
    Bm = torch.stack([Bm, Bm.flip(1)])
    _, Av = window(A, 1, 8, float("nan"))
    _, Bv = window(Bm, 1, 8, float("nan"))
    C0 = (synth.normal(23, 1, 0, batch * rows * cols, dtype=torch.float32).reshape(batch, rows, cols)).cuda()
    _, Dv = window(C0, 2, 16, float("nan"))
    klas.gemm_tc_strided(Av, Bv, Dv, C_=Dv, alpha=0.5, beta=-2.0, map_a="abs")
    want = klas.gemm_tc(A, Bm, C_=C0, alpha=0.5, beta=-2.0, map_a="abs", comb="axpby")
    torch.cuda.synchronize()
    assert torch.equal(Dv, want)


def test_strides_that_cannot_be_served():
    A = torch.zeros((64, 68), dtype=torch.bfloat16, device="cuda")
    Bm = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    D = torch.zeros((64, 64), dtype=torch.float32, device="cuda")
    with pytest.raises(KlasError):                          # row stride not a multiple of 8 elements
        klas.gemm_tc_strided(A[:, :64], Bm, D)
    Dodd = torch.zeros((64, 68), dtype=torch.float32, device="cuda")
    with pytest.raises(KlasError):
        klas.gemm_tc_strided(Bm, Bm, Dodd[:, :64])
    with pytest.raises(ValueError):                         # a shared (stride-0) page: not on this path
        klas.gemm_tc_strided(Bm[None].expand(2, 64, 64), torch.stack([Bm, Bm]), torch.stack([D, D]))
