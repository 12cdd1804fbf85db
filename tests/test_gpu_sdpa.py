"""Scaled dot-product attention (tensor-core GEMM, row softmax, tensor-core GEMM) against a float64
restatement of the reference's specification, `attention_real_batched`
(src/lib/kernel/Kuiper.Kernel.SDPA.Naive.fst:95-113, 278-310): scores = scale * Q.K^T + bias,
probabilities = row softmax, output = probabilities . V."""
import numpy as np
import pytest
import torch

from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu


def tensor(seed, *shape, dtype, spread=1.0):
    n = int(np.prod(shape))
    return (synth.normal(seed, 51, 0, n, dtype=torch.float64).reshape(shape) * spread).to(dtype)


def attention_f64(Q, K, V, bias, scale, dtype):
    """Float64 attention with the three roundings to `dtype` the kernel sequence makes (S, P, O inputs)."""
    S = scale * (Q.double() @ K.double().transpose(-1, -2))
    if bias is not None:
        S = S + bias.double()
    S = S.to(dtype).double()
    P = torch.softmax(S, dim=-1).to(dtype).double()
    return P @ V.double(), P


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("lead,l,s,e,ev", [((1,), 128, 128, 64, 64), ((2, 3), 200, 264, 40, 72), ((4,), 1024, 1024, 128, 128),
                                           ((1, 2), 77, 2056, 64, 32), ((1,), 64, 4096, 64, 64),
                                           ((1,), 1, 304, 40, 40)])   # one query of one head: a one-row score matrix
@pytest.mark.parametrize("with_bias", [True, False])
def test_matches_float64_attention(dtype, tol, lead, l, s, e, ev, with_bias):
    Q, K, V = (tensor(i, *lead, r, c, dtype=dtype) for i, (r, c) in enumerate([(l, e), (s, e), (s, ev)]))
    bias = tensor(9, *lead, l, s, dtype=dtype, spread=0.5) if with_bias else None
    scale = e ** -0.5
    want, P = attention_f64(Q, K, V, bias, scale, dtype)
    buf = bias.cuda().clone() if with_bias else None
    scratch = None if with_bias else torch.empty(lead + (l, s), dtype=dtype, device="cuda")   # keeps the three-step path
    out = klas.sdpa(Q.cuda(), K.cuda(), V.cuda(), buf, scale=scale, scores=scratch)
    torch.cuda.synchronize()
    # output rows are convex combinations of V's rows: errors are measured against sum_j P_ij |V_jc|
    bound = (P @ V.double().abs()).clamp(min=1e-30)
    err = float(((out.double().cpu() - want).abs() / bound).max())
    assert err <= tol, err
    if with_bias:   # the bias buffer now holds the probabilities
        assert float((buf.double().cpu().sum(-1) - 1).abs().max()) <= 64 * tol


@pytest.mark.parametrize("dtype,tol", [(torch.float16, 2e-3), (torch.bfloat16, 1.6e-2)])
@pytest.mark.parametrize("lead,l,s,e", [((1,), 128, 128, 64), ((1,), 128, 128, 128), ((2, 3), 200, 264, 128), ((4,), 1024, 1024, 128),
                                        ((1, 2), 77, 2056, 64), ((1,), 64, 4096, 64), ((2,), 130, 1, 64), ((1,), 1, 300, 128),
                                        ((3,), 384, 129, 128)])
def test_fused_kernel_matches_float64_attention(dtype, tol, lead, l, s, e):
    """One kernel, scores never in global memory: against plain float64 attention (no intermediate roundings)."""
    Q, K, V = (tensor(10 + i, *lead, r, e, dtype=dtype) for i, r in enumerate([l, s, s]))
    scale = e ** -0.5
    S = scale * (Q.double() @ K.double().transpose(-1, -2))
    P = torch.softmax(S, dim=-1)
    want = P @ V.double()
    out = klas.sdpa_fused(Q.cuda(), K.cuda(), V.cuda(), scale=scale)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    bound = (P @ V.double().abs()).clamp(min=1e-30)
    err = float(((out.double().cpu() - want).abs() / bound).max())
    assert err <= tol, err


def test_fused_kernel_with_a_peaked_distribution():
    # large scores: the running maximum moves from tile to tile and old sums are rescaled
    dtype = torch.float16
    Q, K, V = tensor(20, 2, 256, 64, dtype=dtype, spread=3.0), tensor(21, 2, 1000, 64, dtype=dtype, spread=3.0), tensor(22, 2, 1000, 64, dtype=dtype)
    P = torch.softmax(1.0 * (Q.double() @ K.double().transpose(-1, -2)), dim=-1)
    want = P @ V.double()
    out = klas.sdpa_fused(Q.cuda(), K.cuda(), V.cuda(), scale=1.0)
    bound = (P @ V.double().abs()).clamp(min=1e-30)
    assert float(((out.double().cpu() - want).abs() / bound).max()) <= 2e-3


def test_fused_kernel_rejects_other_head_dimensions():
    Q = torch.zeros((1, 8, 96), dtype=torch.float16, device="cuda")
    with pytest.raises(klas.KlasError):
        klas.sdpa_fused(Q, Q, Q)


def test_probabilities_ignore_masked_keys():
    dtype = torch.float16
    Q, K, V = tensor(1, 2, 64, 64, dtype=dtype), tensor(2, 2, 256, 64, dtype=dtype), tensor(3, 2, 256, 64, dtype=dtype)
    bias = torch.zeros((2, 64, 256), dtype=dtype)
    bias[..., 100:] = -float("inf")                      # only the first 100 keys are visible
    full = klas.sdpa(Q.cuda(), K.cuda(), V.cuda(), bias.cuda().clone())
    cut = klas.sdpa(Q.cuda(), K[:, :104].contiguous().cuda(), V[:, :104].contiguous().cuda(),
                    bias[..., :104].contiguous().cuda())
    assert torch.allclose(full.float(), cut.float(), atol=2e-3, rtol=2e-3)


def test_bad_arguments():
    Q = torch.zeros((1, 8, 12), dtype=torch.float16, device="cuda")
    with pytest.raises(klas.KlasError):
        klas.sdpa(Q, Q, Q)                               # e = 12 is not a multiple of 8
    with pytest.raises(TypeError):
        klas.sdpa(Q.float(), Q.float(), Q.float())
