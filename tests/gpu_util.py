"""Shared helpers of the GPU parity tests."""
import numpy as np
import torch

from oracle_api import bf16_bits


def rel_err_componentwise(got: np.ndarray, want: np.ndarray, scale: np.ndarray) -> float:
    """max |got - want| / (|A|.|B|)_ij  -- the relative error measure the tolerances
    are stated in (entries of N(0,1) or U[-1,1) products cancel, so dividing by the
    result itself would measure cancellation, not the kernel)."""
    s = np.maximum(scale, np.finfo(np.float64).tiny)
    return float(np.max(np.abs(got.astype(np.float64) - want) / s))


def tc_reference(oracle, A: torch.Tensor, B: torch.Tensor, b_col_major: bool):
    """float64 product and |A|.|B| scale of 16-bit inputs (exact conversion to double)."""
    kind = "bf16" if A.dtype == torch.bfloat16 else "f16"
    a = bf16_bits(A)
    bmat = B.t().contiguous() if b_col_major else B
    b = bf16_bits(bmat)
    acc = oracle.acc(a, b, kind=kind)
    scale = oracle.absacc(A.double().cpu().numpy(), bmat.double().cpu().numpy())
    return acc, scale
