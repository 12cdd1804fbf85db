"""The deterministic inputs of the reference's test drivers, restated as numpy formulas.

* tiled / naive / block-tiled drivers (test/tiled_matmul_driver.c.inc:47-61,
  test/tiled_gemm_driver.c.inc:47-61): m1[i][j] = 2i + j, m2[i][j] = i + j, m3[i][j] = i - j;
* tensor-core drivers (test/tensor_core_gemm_alpha_beta_1_driver.c.inc:54-91):
  m1[i][j] = et(.5 + i/100), m2[i][j] = et(.5 + j/100), m3 = 0.0001f (mixed precision) or 0.
"""
import numpy as np
import torch


def tiled_inputs(dtype, rows, shared, cols):
    i = np.arange(rows)[:, None]
    j = np.arange(shared)[None, :]
    m1 = (2 * i + j).astype(dtype)
    i = np.arange(shared)[:, None]
    j = np.arange(cols)[None, :]
    m2 = (i + j).astype(dtype)
    i = np.arange(rows, dtype=np.int64)[:, None]
    j = np.arange(cols, dtype=np.int64)[None, :]
    m3 = (i - j).astype(dtype)   # wraps for unsigned types exactly as the C assignment does
    return m1, m2, m3


def tc_inputs(torch_dtype, rows, shared, cols):
    """Returns torch tensors (bf16 or f16) built as the drivers do: double -> float -> et."""
    a_col = torch.tensor((.5 + np.arange(rows) / 100.0).astype(np.float32)).to(torch_dtype)
    b_row = torch.tensor((.5 + np.arange(cols) / 100.0).astype(np.float32)).to(torch_dtype)
    A = a_col[:, None].expand(rows, shared).contiguous()
    B = b_row[None, :].expand(shared, cols).contiguous()
    return A, B


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)
