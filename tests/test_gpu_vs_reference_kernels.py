"""Same seeded inputs through this library and through the reference's own kernels (dist/Klas_*.cu
compiled for sm_100a, oracle/_ref): results must agree -- bit for bit for integers, within the
float tolerances otherwise.  The timings of both are written to the file named by the
KLAS_TIMINGS_OUT environment variable, when it is set."""
import ctypes as C
import json
import os
import time
from pathlib import Path

import numpy as np
import pytest
import torch

from kuiper_b200 import klas, synth
from ref_gpu import RefGpu

pytestmark = pytest.mark.gpu

TIMINGS = {}


@pytest.fixture(scope="module")
def ref():
    if not RefGpu.available():
        pytest.skip("oracle/_ref/libklas_ref_gpu.so not built")
    yield RefGpu()
    if os.environ.get("KLAS_TIMINGS_OUT"):
        out = Path(os.environ["KLAS_TIMINGS_OUT"])
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(TIMINGS, indent=1))


def wall_ms(fn, reps=3):
    """Per-call wall time of a blocking call, as the reference's drivers measure it."""
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / reps * 1e3


def event_ms(fn, reps=5):
    fn()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def test_f32_1024(ref):
    n = 1024
    A, B = synth.gemm_f32(0, n, n, n, device="cuda")
    mine, theirs = torch.zeros((n, n), device="cuda"), torch.zeros((n, n), device="cuda")
    klas.call("Klas_GEMM_SHMem_g_matmul_f32_tile32_rrr", n, n, n, A, B, mine)
    ref.mnk("Klas_GEMM_SHMem_g_matmul_f32_tile32_rrr", n, n, n, A, B, theirs)
    scale = (A.abs().double() @ B.abs().double())
    assert float(((mine.double() - theirs.double()).abs() / scale).max()) <= 2e-5
    TIMINGS["f32_1024"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm(A, B, mine)),
        "ref_SHMem_tile32_call_ms": wall_ms(lambda: ref.mnk("Klas_GEMM_SHMem_g_matmul_f32_tile32_rrr", n, n, n, A, B, theirs)),
        "ref_BlockTiling2D_128x128x32_8x8_call_ms": wall_ms(lambda: ref.mnk(
            "Klas_GEMM_BlockTiling2D_g_gemm_f32_128x128x32_8x8", n, n, n, A, B, theirs,
            pre=((C.c_float, 1.0), (C.c_float, 0.0)))),
        "flop": 2 * n ** 3}


def test_fused_sqrt_gemm_against_the_reference_demo(ref):
    """Kuiper_Example_Fused_GEMM_gemm_sqrt_fused: the reference's one-thread-per-element kernel vs
    the tensor-core GEMM with sqrt applied to the staged A tiles (f16 in and out)."""
    n = 2048
    A, B = synth.gemm_f16_batched(21, 1, n, n, n, device="cuda")
    A, B = A[0].abs(), B[0]
    mine = torch.zeros((n, n), dtype=torch.float16, device="cuda")
    theirs = torch.zeros_like(mine)
    klas.call("Kuiper_Example_Fused_GEMM_gemm_sqrt_fused", n, n, n, A, B, mine)
    ref.mnk("Kuiper_Example_Fused_GEMM_gemm_sqrt_fused", n, n, n, A, B, theirs)
    scale = A.double().sqrt() @ B.double().abs()
    # theirs multiplies the unrounded f32 sqrt, mine rounds it to f16 first; both round the result
    assert float(((mine.double() - theirs.double()).abs() / scale).max()) <= 2 ** -9
    TIMINGS["fused_sqrt_f16_2048"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm_tc(A, B, out_dtype=torch.float16, D=mine, map_a="sqrt")),
        "ref_call_ms": wall_ms(lambda: ref.mnk("Kuiper_Example_Fused_GEMM_gemm_sqrt_fused", n, n, n, A, B, theirs)),
        "flop": 2 * n ** 3}


@pytest.mark.parametrize("top", [200, 65535])
def test_graph_distance_step_bit_exact(ref, top):
    """Kuiper_GraphDist_matmul_dist_gpu on random weights (top = 65535: sums wrap at 2^16 as in the reference)."""
    n = 1026
    u = synth.unit_uniform(31, 44, 0, n * n).reshape(n, n)
    v = synth.integers_below_2_32(31, 45, 0, n * n).reshape(n, n) % top + 1
    a = torch.where(u < 0.05, v, torch.zeros_like(v)).to(torch.int16).cuda()
    mine, theirs = a.clone(), a.clone()
    klas.call("Kuiper_GraphDist_matmul_dist_gpu", n, a, mine)
    f = ref.fn("Kuiper_GraphDist_matmul_dist_gpu", [C.c_uint32, C.c_void_p, C.c_void_p])
    f(n, a.data_ptr(), theirs.data_ptr())
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)
    if top == 200:
        TIMINGS["graphdist_1026"] = {
            "ours_kernel_ms": event_ms(lambda: klas.minplus_u16(a, a, mine)),
            "ref_call_ms": wall_ms(lambda: f(n, a.data_ptr(), theirs.data_ptr())),
            "ring_ops": 2 * n ** 3}


def test_row_wise_neighbours_against_the_reference_kernels(ref):
    """Vector softmax, row softmax, row scale and sum: same inputs through both libraries."""
    n = 1 << 22
    x = (synth.normal(41, 11, 0, n, dtype=torch.float32, device="cuda") * 4.0)
    mine, theirs = x.clone(), x.clone()
    klas.softmax(mine)
    f = ref.fn("Klas_Softmax_softmax_gpu_f32", [C.c_uint32, C.c_void_p])
    f(n, theirs.data_ptr())
    torch.cuda.synchronize()
    # the reference sums 4M exponentials in f32, one long chain per thread: its own denominator is only good to ~1e-5
    assert float((mine - theirs).abs().max()) <= 2e-5 * float(theirs.max())
    TIMINGS["softmax_f32_4M"] = {"ours_kernel_ms": event_ms(lambda: klas.softmax(mine)),
                                 "ref_call_ms": wall_ms(lambda: f(n, theirs.data_ptr())), "elements": n}

    rows, cols = 4096, 1024
    m = synth.normal(42, 11, 0, rows * cols, dtype=torch.float32, device="cuda").reshape(rows, cols) * 3.0
    mine, theirs = m.clone(), m.clone()
    klas.softmax(mine)
    g = ref.fn("Klas_RowSoftmax_row_softmax_rm_f32", [C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p])
    g(rows, cols, 256, theirs.data_ptr())
    torch.cuda.synchronize()
    assert float((mine - theirs).abs().max()) <= 2e-6
    TIMINGS["row_softmax_f32_4096x1024"] = {"ours_kernel_ms": event_ms(lambda: klas.softmax(mine)),
                                            "ref_call_ms": wall_ms(lambda: g(rows, cols, 256, theirs.data_ptr()))}

    sc = synth.normal(43, 11, 0, rows, dtype=torch.float32, device="cuda")
    mine, theirs = m.clone(), m.clone()
    klas.rowscale(sc, mine)
    h = ref.fn("Klas_RowScale_rowscale_f32_rowmajor", [C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p])
    h(rows, cols, sc.data_ptr(), theirs.data_ptr())
    torch.cuda.synchronize()
    assert torch.equal(mine, theirs)

    r = ref.fn("Klas_HReduce_reduce_f32_plus", [C.c_uint32, C.c_uint32, C.c_void_p])
    r.restype = C.c_float
    total_ref = r(256, n, x.data_ptr())
    total = klas.reduce_sum(x).item()
    assert abs(total - total_ref) <= 2e-6 * float(x.abs().sum())


def test_u64_bit_exact(ref):
    n = 1024
    a, b = synth.gemm_u64(3, n, n, n, full_range=True, device="cuda")
    mine, theirs = torch.zeros((n, n), dtype=torch.int64, device="cuda"), torch.zeros((n, n), dtype=torch.int64, device="cuda")
    klas.call("Klas_GEMM_SHMem_g_matmul_u64_tile32_rrr", n, n, n, a, b, mine)
    ref.mnk("Klas_GEMM_SHMem_g_matmul_u64_tile32_rrr", n, n, n, a, b, theirs)
    assert torch.equal(mine, theirs)
    n = 4096
    a, b = synth.gemm_u64(3, n, n, n, device="cuda")
    mine, theirs = torch.zeros((n, n), dtype=torch.int64, device="cuda"), torch.zeros((n, n), dtype=torch.int64, device="cuda")
    t_ref = wall_ms(lambda: ref.mnk("Klas_GEMM_SHMem_g_matmul_u64_tile32_rrr", n, n, n, a, b, theirs), reps=1)
    t_ours = event_ms(lambda: klas.gemm(a, b, mine), reps=2)
    assert torch.equal(mine, theirs)          # the 4096^3 benchmark configuration, bit for bit
    TIMINGS["u64_4096"] = {"ours_kernel_ms": t_ours, "ref_SHMem_tile32_call_ms": t_ref, "ops": 2 * n ** 3}


@pytest.mark.parametrize("n", [1024, 4096])
def test_bf16_f32(ref, n):
    A, B = synth.gemm_bf16(1, n, n, n, b_col_major=False, device="cuda")
    mine, theirs = torch.zeros((n, n), device="cuda"), torch.zeros((n, n), device="cuda")
    name = "Klas_GEMM_TensorCore2D_g_gemm_bf16_f32_128x128x32_16x16x16_8x4"
    klas.call(name, n, n, n, A, B, mine)
    ref.mnk(name, n, n, n, A, B, theirs)
    scale = (A.abs().double() @ B.abs().double())
    assert float(((mine.double() - theirs.double()).abs() / scale).max()) <= 2e-3
    TIMINGS["bf16_f32_%d" % n] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm_tc(A, B, D=mine)),
        "ours_call_ms": wall_ms(lambda: (klas.gemm_tc(A, B, D=mine), torch.cuda.synchronize())),
        "ref_TensorCore2D_128x128x32_8x4_call_ms": wall_ms(lambda: ref.mnk(name, n, n, n, A, B, theirs)),
        "flop": 2 * n ** 3}


def test_f16_f16(ref):
    n = 2048
    A, B = synth.gemm_f16_batched(2, 1, n, n, n, device="cuda")
    mine = torch.zeros((n, n), dtype=torch.float16, device="cuda")
    theirs = torch.zeros_like(mine)
    name = "Klas_GEMM_TensorCore2D_g_gemm_f16_f16_128x128x32_16x16x16_8x4"
    klas.call(name, n, n, n, A[0], B[0], mine)
    ref.mnk(name, n, n, n, A[0], B[0], theirs)
    scale = (A[0].abs().double() @ B[0].abs().double())
    # the reference rounds its half accumulator after every 16-deep step; both stay within 1e-2
    assert float(((mine.double() - theirs.double()).abs() / scale).max()) <= 1e-2
    TIMINGS["f16_f16_2048"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm_tc(A[0], B[0], out_dtype=torch.float16, D=mine)),
        "ref_TensorCore2D_128x128x32_8x4_call_ms": wall_ms(lambda: ref.mnk(name, n, n, n, A[0], B[0], theirs)),
        "flop": 2 * n ** 3}


def test_spmm_f32(ref):
    rows = shared = 8192      # the reference's wrappers abort at 10000 and above (dist/Klas_SPMM.cu:196-198)
    cols = 256
    csr = synth.csr_poisson(4, rows, shared, 64.0, device="cuda")
    B = synth.spmm_dense_b(4, shared, cols, device="cuda")
    mine, theirs = torch.zeros((rows, cols), device="cuda"), torch.zeros((rows, cols), device="cuda")
    klas.spmm(csr, B, mine)
    ref.spmm_f32("Klas_SPMM_spmm_f32", rows, shared, cols, csr, B, theirs)
    assert torch.equal(mine, theirs)      # both add each row's products in CSR order with one FMA each
    TIMINGS["spmm_8192_p64_c256"] = {
        "ours_kernel_ms": event_ms(lambda: klas.spmm(csr, B, mine)),
        "ref_spmm_f32_call_ms": wall_ms(lambda: ref.spmm_f32("Klas_SPMM_spmm_f32", rows, shared, cols, csr, B, theirs)),
        "nnz": csr.nnz}


def test_vendor_library_comparison_rows(ref):
    """cuBLAS (through torch.matmul) and cuSPARSE (through torch.sparse) on the benchmark shapes:
    recorded for the comparison table only; nothing in the product calls them."""
    n = 8192
    A, Bt = synth.gemm_bf16(1, n, n, n, b_col_major=True, device="cuda")
    D = torch.empty((n, n), device="cuda")
    TIMINGS["bf16_f32_8192_colmajorB"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm_tc(A, Bt, b_col_major=True, D=D), reps=10),
        "cublas_bf16_out_bf16_ms": event_ms(lambda: torch.matmul(A, Bt.t()), reps=10),
        "flop": 2 * n ** 3}
    Brm = Bt.t().contiguous()
    TIMINGS["bf16_f32_8192_rowmajorB"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm_tc(A, Brm, D=D), reps=10),
        "cublas_bf16_out_bf16_ms": event_ms(lambda: torch.matmul(A, Brm), reps=10),
        "flop": 2 * n ** 3}
    del A, Bt, Brm, D
    n = 4096
    a32, b32 = synth.gemm_f32(0, n, n, n, device="cuda")
    c32 = torch.empty((n, n), device="cuda")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        TIMINGS["f32_4096"] = {
            "ours_kernel_ms": event_ms(lambda: klas.gemm(a32, b32, c32), reps=3),
            "cublas_sgemm_ms": event_ms(lambda: torch.matmul(a32, b32), reps=3),
            "ref_BlockTiling2D_128x128x32_8x8_call_ms": wall_ms(lambda: ref.mnk(
                "Klas_GEMM_BlockTiling2D_g_gemm_f32_128x128x32_8x8", n, n, n, a32, b32, c32,
                pre=((C.c_float, 1.0), (C.c_float, 0.0))), reps=2),
            "flop": 2 * n ** 3}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    a64, b64 = a32[:2048, :2048].double().contiguous(), b32[:2048, :2048].double().contiguous()
    c64 = torch.empty((2048, 2048), dtype=torch.float64, device="cuda")
    TIMINGS["f64_2048"] = {
        "ours_kernel_ms": event_ms(lambda: klas.gemm(a64, b64, c64), reps=3),
        "cublas_dgemm_ms": event_ms(lambda: torch.matmul(a64, b64), reps=3),
        "flop": 2 * 2048 ** 3}
    rows = shared = 131072
    cols = 256
    csr = synth.csr_poisson(4, rows, shared, 64.0, device="cuda")
    Bd = synth.spmm_dense_b(4, shared, cols, device="cuda")
    Cd = torch.empty((rows, cols), device="cuda")
    sp = torch.sparse_csr_tensor(csr.row_off.long(), csr.col_ind.long(), csr.elems, size=(rows, shared))
    got = klas.spmm(csr, Bd, Cd)
    want = torch.sparse.mm(sp, Bd)
    assert float((got - want).abs().max()) <= 1e-4
    TIMINGS["spmm_131072_p64_c256"] = {
        "ours_kernel_ms": event_ms(lambda: klas.spmm(csr, Bd, Cd), reps=5),
        "cusparse_csr_spmm_ms": event_ms(lambda: torch.sparse.mm(sp, Bd), reps=5),
        "nnz": csr.nnz}
