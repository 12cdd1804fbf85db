"""Parity of the tcgen05 tensor-core GEMM (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from driver_inputs import bits16, tc_inputs
from gpu_util import rel_err_componentwise, tc_reference
from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

TOL_BF16_F32 = 2e-3   # bf16 x bf16 -> f32, relative to fp64, component-wise scale
TOL_F16_F16 = 1e-2    # f16 x f16 -> f16


@pytest.fixture(autouse=True, params=["single", "narrow", "slim", "pair", "wide", "auto"])
def tc_mode(request):
    """Every test runs with the single-CTA tiles (256, 128 and 64 columns wide), the CTA-pair tiles, the wide
    pair tiles and the library's own choice."""
    klas.debug_set("tc_mode", request.param)
    yield request.param
    klas.debug_set("tc_mode", "auto")
    assert klas.gemm_tc_status() == 0


SHAPES = [
    (128, 64, 256),     # one tile, one k-block
    (128, 256, 256),    # one tile, pipeline wraps (4 k-blocks = ring depth)
    (256, 512, 512),    # 2x2 tiles, ring wraps twice
    (64, 16, 64),       # smallest legacy guard multiple: partial tile in M, N and K
    (192, 80, 328),     # ragged everywhere (multiples of 8 only)
    (1024, 1024, 1024), # the reference drivers' default size
    (640, 2048, 1280),  # more tiles than fit one wave of a small grid; deep K
]


@pytest.mark.parametrize("rows,shared,cols", SHAPES)
@pytest.mark.parametrize("b_col_major", [False, True])
def test_bf16_f32_matches_oracle(oracle, rows, shared, cols, b_col_major):
    A, Bm = synth.gemm_bf16(1, rows, cols, shared, b_col_major=b_col_major, device="cuda")
    D = klas.gemm_tc(A, Bm, out_dtype=torch.float32, b_col_major=b_col_major)
    torch.cuda.synchronize()
    acc, scale = tc_reference(oracle, A.cpu(), Bm.cpu(), b_col_major)
    err = rel_err_componentwise(D.cpu().numpy(), acc, scale)
    assert err <= TOL_BF16_F32, "relative error %.3e" % err
    # fp32 accumulation of exact bf16 products: far inside the tolerance
    assert err <= 1e-5


@pytest.mark.parametrize("rows,shared,cols", SHAPES[:6])
def test_f16_f16_matches_oracle(oracle, rows, shared, cols):
    A, B = synth.gemm_f16_batched(2, 1, rows, cols, shared, device="cuda")
    D = klas.gemm_tc(A[0], B[0], out_dtype=torch.float16)
    torch.cuda.synchronize()
    acc, scale = tc_reference(oracle, A[0].cpu(), B[0].cpu(), False)
    err = rel_err_componentwise(D.double().cpu().numpy(), acc, scale)
    assert err <= TOL_F16_F16, "relative error %.3e" % err


def test_f16_driver_inputs_overflow_pattern(oracle):
    """The six F16_F16 drivers' inputs: ~13 % of the results overflow to +inf in the gold;
    the kernel must overflow too (never saturate to 65504)."""
    A, B = tc_inputs(torch.float16, 1024, 1024, 1024)
    gold = oracle.gemm(bits16(A), bits16(B), kind="f16")
    D = klas.gemm_tc(A.cuda(), B.cuda(), out_dtype=torch.float16)
    got = bits16(D.cpu())
    inf_gold, inf_got = gold == 0x7c00, got == 0x7c00
    assert inf_gold.sum() > 100000
    # entries within rounding distance of the 65520 threshold may differ; the driver's own
    # comparison tolerates up to 9 mismatching cells (test/matmul_common.c.inc:106-112)
    assert int((inf_gold != inf_got).sum()) <= 9
    fin = ~inf_gold & ~inf_got
    g64, d64 = oracle.f16_bits_to_f64(gold[fin]), oracle.f16_bits_to_f64(got[fin])
    assert np.max(np.abs(g64 - d64) / np.abs(g64)) <= 0.02   # the drivers' TOLERANCE


def test_bf16_driver_inputs(oracle):
    A, B = tc_inputs(torch.bfloat16, 1024, 1024, 1024)
    gold = oracle.gemm(bits16(A), bits16(B), kind="bf16")
    D = klas.gemm_tc(A.cuda(), B.cuda(), out_dtype=torch.float32).cpu().numpy()
    assert np.max(np.abs(D - gold) / np.abs(gold)) <= 1e-5


def test_alpha_beta_bf16_out(oracle):
    """D = bf16(beta*C + alpha*A.B) with distinct C and D (the TensorCore2D_To contract,
    src/klas/Klas.GEMM.TensorCore2D.To.Inst.fsti:65-66)."""
    rows, shared, cols = 256, 320, 384
    A, B = synth.gemm_bf16(7, rows, cols, shared, b_col_major=False, device="cuda")
    Cin = synth.normal(7, 9, 0, rows * cols, torch.bfloat16, "cuda").view(rows, cols)
    Cin_copy = Cin.clone()
    D = klas.gemm_tc(A, B, out_dtype=torch.bfloat16, C_=Cin, alpha=0.7, beta=0.3)
    acc, scale = tc_reference(oracle, A.cpu(), B.cpu(), False)
    want = 0.3 * Cin.double().cpu().numpy() + 0.7 * acc
    bound = 0.3 * np.abs(Cin.double().cpu().numpy()) + 0.7 * scale
    # one bf16 rounding of the result (2^-9 relative) on top of the accumulation error
    assert rel_err_componentwise(D.double().cpu().numpy(), want, bound) <= 2 ** -8
    assert torch.equal(Cin, Cin_copy)


@pytest.mark.parametrize("out_dtype", [torch.float16, torch.float32])
def test_accumulate_in_place(oracle, out_dtype):
    """C += A.B (dist/Klas_GEMM_TensorCore.cu:28-33): D aliases C, alpha = beta = 1."""
    rows, shared, cols = 128, 192, 128
    A, B = synth.gemm_f16_batched(5, 1, rows, cols, shared, device="cuda")
    C0 = synth.uniform(5, 7, 0, rows * cols, -1.0, 1.0, out_dtype, "cuda").view(rows, cols)
    Cio = C0.clone()
    klas.gemm_tc(A[0], B[0], out_dtype=out_dtype, C_=Cio, D=Cio, alpha=1.0, beta=1.0)
    acc, scale = tc_reference(oracle, A[0].cpu(), B[0].cpu(), False)
    want = C0.double().cpu().numpy() + acc
    tol = 1e-2 if out_dtype == torch.float16 else 1e-5
    assert rel_err_componentwise(Cio.double().cpu().numpy(), want, scale + np.abs(C0.double().cpu().numpy())) <= tol


def test_batched_pages(oracle):
    batch, m, n, k = 3, 192, 264, 136
    A, B = synth.gemm_f16_batched(2, batch, m, n, k, device="cuda")
    D = klas.gemm_tc(A, B, out_dtype=torch.float16)
    for b in range(batch):
        acc, scale = tc_reference(oracle, A[b].cpu(), B[b].cpu(), False)
        assert rel_err_componentwise(D[b].double().cpu().numpy(), acc, scale) <= TOL_F16_F16


def test_never_writes_outside_the_output(oracle):
    """Canary rows around D stay intact for a ragged shape."""
    rows, shared, cols = 200, 72, 136
    A, B = synth.gemm_bf16(3, rows, cols, shared, b_col_major=True, device="cuda")
    buf = torch.full((rows + 16, cols), 12345.0, device="cuda")
    D = buf[8:8 + rows]
    klas.gemm_tc(A, B, out_dtype=torch.float32, b_col_major=True, D=D)
    torch.cuda.synchronize()
    assert bool((buf[:8] == 12345.0).all()) and bool((buf[8 + rows:] == 12345.0).all())


def test_linearity_at_full_size():
    """Size-independent property at the benchmark's size (8192^3): (A1 + A2).B == A1.B + A2.B
    when the sums are exact -- rows of small integers keep every product and partial sum
    exactly representable, so the identity must hold bit for bit."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    A1 = torch.randint(-3, 4, (n, n), device="cuda", generator=g).to(torch.bfloat16)
    A2 = torch.randint(-3, 4, (n, n), device="cuda", generator=g).to(torch.bfloat16)
    Bt = torch.randint(-3, 4, (n, n), device="cuda", generator=g).to(torch.bfloat16)
    d1 = klas.gemm_tc(A1, Bt, b_col_major=True)
    d2 = klas.gemm_tc(A2, Bt, b_col_major=True)
    d12 = klas.gemm_tc((A1 + A2), Bt, b_col_major=True)
    assert torch.equal(d12, d1 + d2)
    # and a sampled exact check against an fp64 product of the same small integers
    rows = torch.tensor([0, 1, 127, 128, 4095, 8191], device="cuda")
    want = A1[rows].double() @ Bt.double().t()   # exact: every partial sum is a small integer
    assert torch.equal(d1[rows].double(), want)


def test_rejects_unsupported_shapes():
    A = torch.zeros((64, 60), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((60, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(klas.KlasError) as e:
        klas.gemm_tc(A, B)
    assert e.value.status == 2   # KLAS_ERR_UNSUPPORTED: shared % 8 != 0


def test_zero_inner_dimension():
    A = torch.zeros((64, 0), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((0, 64), dtype=torch.bfloat16, device="cuda")
    D = torch.full((64, 64), 7.0, device="cuda")
    klas.gemm_tc(A, B, D=D)
    assert bool((D == 0).all())


@pytest.mark.parametrize("rows,cols,expect", [
    (2048, 2048, "one round of single tiles"), (2560, 2048, "40 wide tiles, one round"),
    (3072, 3072, "72 wide tiles, one round"), (3584, 3072, "84 wide tiles would take two rounds: pairs"),
    (3000, 2056, "ragged edges"), (1024, 1024, "64 narrow tiles instead of 32"), (1536, 1480, "narrow, ragged")])
def test_tile_choice_does_not_change_results(oracle, rows, cols, expect, tc_mode):
    """The library picks single, pair or wide tiles from the shape.  Every element is accumulated
    over k in the same order whatever the tile, so the three kernels and the library's own choice
    must agree bit for bit; a sample of rows is checked against the oracle."""
    if tc_mode != "auto":
        return   # the modes are set below; one pass is enough
    shared = 192
    A, Bt = synth.gemm_bf16(31, rows, cols, shared, b_col_major=True, device="cuda")
    results = {}
    for mode in ("auto", "single", "narrow", "slim", "pair", "wide"):
        klas.debug_set("tc_mode", mode)
        results[mode] = klas.gemm_tc(A, Bt, out_dtype=torch.float32, b_col_major=True)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    for mode in ("single", "narrow", "slim", "pair", "wide"):
        assert torch.equal(results["auto"], results[mode]), "%s differs (%s)" % (mode, expect)
    pick = torch.arange(0, rows, 97, device="cuda")
    acc, scale = tc_reference(oracle, A[pick].cpu(), Bt.cpu(), True)
    err = rel_err_componentwise(results["auto"][pick].cpu().numpy(), acc, scale)
    assert err <= 1e-5, "relative error %.3e" % err


@pytest.mark.parametrize("parts", [2, 3, 8])
@pytest.mark.parametrize("rows,cols,shared", [(256, 512, 1024), (328, 200, 1160), (1024, 1024, 4096)])
def test_k_split_parts_are_added_in_fixed_order(oracle, rows, cols, shared, parts, tc_mode):
    """A tile's K range cut into parts (the single-CTA and pair kernels; the wide kernel has no
    split and ignores the knob): the parts' f32 products are added in index order by a second
    kernel, so the result equals the unsplit product up to fp32 re-association, is the same from
    run to run, and goes through every output rule: plain, alpha/beta with an old C, 16-bit
    output, relu."""
    A, Bt = synth.gemm_bf16(17, rows, cols, shared, b_col_major=True, device="cuda")
    C0 = torch.randn(rows, cols, device="cuda")
    klas.debug_set("tc_ksplit", "off")
    whole = klas.gemm_tc(A, Bt, b_col_major=True)
    whole_ab = klas.gemm_tc(A, Bt, b_col_major=True, C_=C0, alpha=0.5, beta=-1.25)
    whole_bf = klas.gemm_tc(A, Bt, b_col_major=True, out_dtype=torch.bfloat16)
    try:
        klas.debug_set("tc_ksplit", parts)
        split = [klas.gemm_tc(A, Bt, b_col_major=True) for _ in range(3)]
        split_ab = klas.gemm_tc(A, Bt, b_col_major=True, C_=C0, alpha=0.5, beta=-1.25)
        split_bf = klas.gemm_tc(A, Bt, b_col_major=True, out_dtype=torch.bfloat16)
        split_relu = klas.gemm_tc(A, Bt, b_col_major=True, comb="relu")
    finally:
        klas.debug_set("tc_ksplit", "auto")
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    assert torch.equal(split[0], split[1]) and torch.equal(split[0], split[2]), "run-to-run difference"
    scale = (A.float().abs() @ Bt.float().abs().t()).clamp_min(1e-30)
    assert float(((split[0] - whole).abs() / scale).max()) <= 1e-6
    assert float(((split_ab - whole_ab).abs() / (scale + C0.abs())).max()) <= 1e-6
    assert float(((split_bf.float() - whole_bf.float()).abs() / scale).max()) <= 2 ** -8
    assert torch.equal(split_relu, split[0].clamp_min(0.0))
    pick = torch.arange(0, rows, 37, device="cuda")
    acc, sc = tc_reference(oracle, A[pick].cpu(), Bt.cpu(), True)
    assert rel_err_componentwise(split[0][pick].cpu().numpy(), acc, sc) <= 1e-5


def test_k_split_chosen_for_small_outputs_with_long_k(oracle, tc_mode):
    """1024 x 1024 x 4096 fills a quarter of the SMs with 128 x 256 tiles: the library cuts K by
    itself.  The result is checked against the oracle on sampled rows and against the unsplit
    product."""
    if tc_mode != "auto":
        return
    A, Bt = synth.gemm_bf16(19, 1024, 1024, 4096, b_col_major=True, device="cuda")
    auto = klas.gemm_tc(A, Bt, b_col_major=True)
    klas.debug_set("tc_ksplit", "off")
    whole = klas.gemm_tc(A, Bt, b_col_major=True)
    klas.debug_set("tc_ksplit", "auto")
    torch.cuda.synchronize()
    pick = torch.arange(0, 1024, 61, device="cuda")
    acc, sc = tc_reference(oracle, A[pick].cpu(), Bt.cpu(), True)
    assert rel_err_componentwise(auto[pick].cpu().numpy(), acc, sc) <= 1e-5
    scale = (A.float().abs() @ Bt.float().abs().t())
    assert float(((auto - whole).abs() / scale).max()) <= 1e-6


def test_k_split_with_pages_and_row_major_b(tc_mode):
    """The split's workspace holds parts x pages partial products; checked against the unsplit
    product of the same pages (f16, row-major B, 16-bit output)."""
    A, B = synth.gemm_f16_batched(23, 3, 200, 264, 1096, device="cuda")
    klas.debug_set("tc_ksplit", "off")
    whole = klas.gemm_tc(A, B, out_dtype=torch.float16)
    try:
        klas.debug_set("tc_ksplit", 5)
        split = klas.gemm_tc(A, B, out_dtype=torch.float16)
        again = klas.gemm_tc(A, B, out_dtype=torch.float16)
    finally:
        klas.debug_set("tc_ksplit", "auto")
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    assert torch.equal(split, again)
    scale = torch.bmm(A.float().abs(), B.float().abs())
    assert float(((split.float() - whole.float()).abs() / scale).max()) <= 2 ** -9


def test_k_split_does_not_allocate_while_a_graph_records(tc_mode):
    """A split launch needs a buffer for its parts.  On a stream that has none yet and is recording a
    CUDA graph the library must not allocate (that would invalidate the capture): the launch runs
    in one pass, the graph records and replays, and the result matches the eager one."""
    if tc_mode != "auto":
        return
    A, Bt = synth.gemm_bf16(29, 1024, 1024, 4096, b_col_major=True, device="cuda")
    eager = klas.gemm_tc(A, Bt, b_col_major=True)          # split, on the current stream
    D = torch.empty_like(eager)
    fresh = torch.cuda.Stream()
    fresh.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(fresh):
        with torch.cuda.graph(g, stream=fresh):
            klas.gemm_tc(A, Bt, b_col_major=True, D=D)      # first call on this stream: no buffer yet
    g.replay()
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    scale = A.float().abs() @ Bt.float().abs().t()
    assert float(((D - eager).abs() / scale).max()) <= 1e-6


def test_k_split_on_two_streams_at_once(tc_mode):
    """Split launches on different streams may overlap, so each stream has its own buffer for the
    parts: two streams running different products at the same time must both get their own result."""
    if tc_mode != "auto":
        return
    A1, B1 = synth.gemm_bf16(41, 1024, 1024, 4096, b_col_major=True, device="cuda")
    A2, B2 = synth.gemm_bf16(43, 1024, 1024, 4096, b_col_major=True, device="cuda")
    klas.debug_set("tc_ksplit", "off")
    want1, want2 = klas.gemm_tc(A1, B1, b_col_major=True), klas.gemm_tc(A2, B2, b_col_major=True)
    klas.debug_set("tc_ksplit", "auto")
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    got1, got2 = torch.empty_like(want1), torch.empty_like(want2)
    for _ in range(20):
        with torch.cuda.stream(s1):
            klas.gemm_tc(A1, B1, b_col_major=True, D=got1)
        with torch.cuda.stream(s2):
            klas.gemm_tc(A2, B2, b_col_major=True, D=got2)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    scale1 = A1.float().abs() @ B1.float().abs().t()
    scale2 = A2.float().abs() @ B2.float().abs().t()
    assert float(((got1 - want1).abs() / scale1).max()) <= 1e-6
    assert float(((got2 - want2).abs() / scale2).max()) <= 1e-6


@pytest.mark.parametrize("rows,cols,shared", [(2560, 2048, 1024), (2500, 2040, 1032), (4096, 4096, 512)])
def test_last_round_cut_along_k(oracle, rows, cols, shared, tc_mode):
    """More tiles than CTA groups with a part-filled last round: the full rounds run as one launch,
    the last round's tiles with their K range cut into parts as a second one, and a third kernel
    adds the parts (restricted to those tiles).  Forced here for every tile shape that has the
    path; the result must match the one-launch product (the tiles of the full rounds bit for
    bit, the others to fp32 re-association), through every output rule."""
    A, Bt = synth.gemm_bf16(37, rows, cols, shared, b_col_major=True, device="cuda")
    C0 = torch.randn(rows, cols, device="cuda")
    klas.debug_set("tc_tail", "off")
    whole = klas.gemm_tc(A, Bt, b_col_major=True)
    whole_ab = klas.gemm_tc(A, Bt, b_col_major=True, C_=C0, alpha=0.5, beta=-1.25)
    whole_bf = klas.gemm_tc(A, Bt, b_col_major=True, out_dtype=torch.bfloat16)
    try:
        klas.debug_set("tc_tail", "always")
        cut = [klas.gemm_tc(A, Bt, b_col_major=True) for _ in range(2)]
        cut_ab = klas.gemm_tc(A, Bt, b_col_major=True, C_=C0, alpha=0.5, beta=-1.25)
        cut_bf = klas.gemm_tc(A, Bt, b_col_major=True, out_dtype=torch.bfloat16)
        inplace = C0.clone()
        klas.gemm_tc(A, Bt, b_col_major=True, C_=inplace, D=inplace, alpha=0.5, beta=-1.25)
    finally:
        klas.debug_set("tc_tail", "auto")
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    assert torch.equal(cut[0], cut[1]), "run-to-run difference"
    scale = (A.float().abs() @ Bt.float().abs().t()).clamp_min(1e-30)
    assert float(((cut[0] - whole).abs() / scale).max()) <= 1e-6
    assert float(((cut_ab - whole_ab).abs() / (scale + C0.abs())).max()) <= 1e-6
    assert torch.equal(inplace, cut_ab)
    assert float(((cut_bf.float() - whole_bf.float()).abs() / scale).max()) <= 2 ** -8
    if tc_mode not in ("wide", "auto"):
        # most of the matrix belongs to the full rounds and is untouched by the cut
        assert float((cut[0] == whole).float().mean()) >= 0.5
    pick = torch.arange(0, rows, 111, device="cuda")
    acc, sc = tc_reference(oracle, A[pick].cpu(), Bt.cpu(), True)
    assert rel_err_componentwise(cut[0][pick].cpu().numpy(), acc, sc) <= 1e-5
