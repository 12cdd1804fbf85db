"""Generates tests/golden/klas_golden.npz from the reference's own host gold loops
(oracle/_ref/libklas_ref_cpu.so = test/matmul_common.c.inc and
dist/Kuiper_Example_Sparse_MM.cu compiled from the reference tree).

    python oracle/build.py && python tests/golden/make_golden.py

The fixture holds outputs only; the inputs are the drivers' index formulas
(tests/driver_inputs.py) and seeded synthetic CSR matrices (kuiper_b200.synth).
"""
import hashlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path[:0] = [str(REPO), str(REPO / "oracle"), str(REPO / "tests")]

from driver_inputs import bits16, tc_inputs, tiled_inputs  # noqa: E402
from oracle_api import RefCpu  # noqa: E402
from kuiper_b200 import synth  # noqa: E402

SMALL = (24, 40, 16)       # rows, shared, cols of the full-matrix fixtures
TC_SMALL = (32, 48, 24)
BIG = (1024, 1024, 1024)   # the drivers' default size: stored as digest + strided samples
STRIDE = 4099


def digest(a: np.ndarray) -> np.ndarray:
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


def main():
    ref = RefCpu()
    out = {}
    for kind, dt in (("f32", np.float32), ("f64", np.float64), ("u32", np.uint32), ("u64", np.uint64)):
        m1, m2, m3 = tiled_inputs(dt, *SMALL)
        out["mul_%s_small" % kind] = ref.cpu_mul(kind, m1, m2)
        if kind in ("f32", "f64"):
            out["sgemm_%s_small" % kind] = ref.cpu_sgemm(kind, m1, m2, m3, 0.7, 0.3)
        m1, m2, m3 = tiled_inputs(dt, *BIG)
        big = ref.cpu_mul(kind, m1, m2)
        out["mul_%s_big_sha256" % kind] = digest(big)
        out["mul_%s_big_samples" % kind] = big.reshape(-1)[::STRIDE].copy()
    for kind, tdt in (("bf16_f32", torch.bfloat16), ("f16_f16", torch.float16)):
        A, B = tc_inputs(tdt, *TC_SMALL)
        out["mul_%s_small" % kind] = ref.cpu_mul(kind, bits16(A), bits16(B))
        A, B = tc_inputs(tdt, *BIG)
        big = ref.cpu_mul(kind, bits16(A), bits16(B))
        out["mul_%s_big_sha256" % kind] = digest(big)
        out["mul_%s_big_samples" % kind] = big.reshape(-1)[::STRIDE].copy()
        if kind == "f16_f16":
            out["mul_f16_f16_big_inf_count"] = np.array([int((big == 0x7c00).sum())])
    # u32 CSR x dense through the reference's verified host loop
    csr = synth.csr_poisson(11, 96, 80, 6.0, value_kind="u32")
    Bd = synth.spmm_dense_b(11, 80, 24, value_kind="u32")
    out["spmm_u32_small"] = ref.mmsd_u32_rr(96, 80, 24, csr.elems.numpy().view(np.uint32),
                                            csr.col_ind.numpy().view(np.uint32),
                                            csr.row_off.numpy().view(np.uint32),
                                            Bd.numpy().view(np.uint32))
    # softmax drivers' gold functions on their ramp pattern (test/softmax_test_common.c.inc:66-72)
    ramp = (np.arange(100) % 16) * 0.5 - 4.0
    out["softmax_ramp"] = ref.cpu_softmax(ramp)
    out["logsoftmax_ramp"] = ref.cpu_softmax(ramp, log=True)
    np.savez_compressed(HERE / "klas_golden.npz", **out)
    print("wrote", HERE / "klas_golden.npz", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
