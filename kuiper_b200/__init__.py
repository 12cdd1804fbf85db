"""kuiper_b200 -- B200-native implementation of the Klas matrix-multiply hot path
(dense GEMM on tensor cores and CUDA cores, CSR x dense SpMM) behind a C ABI.

The compute library is kuiper_b200/lib/libklas_b200.so (built by
`python -m kuiper_b200.build`); this package is its host-side mirror for
Python callers, tests and benchmarks.
"""
from . import synth  # noqa: F401

__all__ = ["synth", "klas", "sharding", "build"]
__version__ = "1.0"
