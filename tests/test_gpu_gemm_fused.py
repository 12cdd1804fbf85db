"""Parity of the tensor-core GEMM's fused element-wise hooks (operand maps applied in shared
memory, combine rules in the epilogue) with the CPU oracle: the maps are applied to the 16-bit
bit patterns by the oracle (float evaluation, one rounding), then the product is accumulated
in float64 exactly as for the plain GEMM."""
import numpy as np
import pytest
import torch

from driver_inputs import bits16
from gpu_util import rel_err_componentwise, tc_reference
from kuiper_b200 import klas, synth

pytestmark = pytest.mark.gpu

# One mapped element in a few thousand may differ by one 16-bit ulp from the oracle's (sqrt is
# the hardware approximation, <= 1 ulp of f32 before the rounding), hence looser than the
# plain GEMM's 1e-5 for bf16 -> f32.
TOL_F32_OUT = 5e-5
TOL_F16_OUT = 1e-2
MAP_CODE = {None: 0, "sqrt": 1, "abs": 2, "square": 3, "relu": 4, "neg": 5}


@pytest.fixture(autouse=True, params=["single", "narrow", "slim", "wide", "auto"])
def tc_mode(request):
    """Single-CTA tiles, wide pair tiles, and the library's own choice (the 256 x 256 pair tiles
    carry no mapping warps and are never chosen for a mapped product)."""
    klas.debug_set("tc_mode", request.param)
    yield request.param
    klas.debug_set("tc_mode", "auto")
    assert klas.gemm_tc_status() == 0


def mapped(oracle, t, op):
    """The oracle's image of tensor `t` under map `op`, as a tensor of the same dtype."""
    if op is None:
        return t.cpu()
    kind = "bf16" if t.dtype == torch.bfloat16 else "f16"
    bits = oracle.map16(bits16(t.cpu()), kind, MAP_CODE[op])
    return torch.from_numpy(bits.view(np.int16).reshape(tuple(t.shape))).view(t.dtype)


def positive(t):
    return t.abs() + 0.0   # sqrt wants non-negative operands


SHAPES = [(128, 64, 256), (256, 512, 512), (192, 80, 328), (1024, 1024, 1024), (640, 2048, 1280)]


@pytest.mark.parametrize("rows,shared,cols", SHAPES)
@pytest.mark.parametrize("map_a,map_b", [("sqrt", None), (None, "abs"), ("square", "relu"), ("neg", "sqrt")])
@pytest.mark.parametrize("b_col_major", [False, True])
def test_bf16_operand_maps(oracle, rows, shared, cols, map_a, map_b, b_col_major):
    A, Bm = synth.gemm_bf16(11, rows, cols, shared, b_col_major=b_col_major, device="cuda")
    if map_a == "sqrt":
        A = positive(A)
    if map_b == "sqrt":
        Bm = positive(Bm)
    D = klas.gemm_tc(A, Bm, out_dtype=torch.float32, b_col_major=b_col_major, map_a=map_a, map_b=map_b)
    torch.cuda.synchronize()
    acc, scale = tc_reference(oracle, mapped(oracle, A, map_a), mapped(oracle, Bm, map_b), b_col_major)
    err = rel_err_componentwise(D.cpu().numpy(), acc, scale)
    assert err <= TOL_F32_OUT, "relative error %.3e" % err


@pytest.mark.parametrize("rows,shared,cols", SHAPES[:4])
def test_f16_sqrt_a_is_the_reference_demo(oracle, rows, shared, cols):
    """C = sqrt(A).B in f16 with f32 accumulation: dist/Kuiper_Example_Fused_GEMM.cu:8-43.  The
    demo takes sqrt in f32 and does not round it to f16 before multiplying, so against ITS
    arithmetic the error bound is the f16 rounding of the mapped operand plus that of the result."""
    A, B = synth.gemm_f16_batched(12, 1, rows, cols, shared, device="cuda")
    A, B = positive(A[0]), B[0]
    D = klas.gemm_tc(A, B, out_dtype=torch.float16, map_a="sqrt")
    torch.cuda.synchronize()
    acc, scale = tc_reference(oracle, mapped(oracle, A, "sqrt"), B.cpu(), False)
    assert rel_err_componentwise(D.double().cpu().numpy(), acc, scale) <= TOL_F16_OUT
    demo = torch.sqrt(A.double().cpu()) @ B.double().cpu()                 # unrounded sqrt, float64
    demo_scale = (torch.sqrt(A.double().cpu()) @ B.double().abs().cpu()).numpy()
    assert rel_err_componentwise(D.double().cpu().numpy(), demo.numpy(), demo_scale) <= 2 ** -10


@pytest.mark.parametrize("comb", ["max", "min", "mul", "relu", "axpby", "new", "scaled"])
@pytest.mark.parametrize("rows,shared,cols", [(192, 80, 328), (1024, 256, 512)])
def test_combine_rules(oracle, comb, rows, shared, cols):
    A, Bm = synth.gemm_bf16(13, rows, cols, shared, b_col_major=False, device="cuda")
    C = synth.normal(14, 3, 0, rows * cols, dtype=torch.float32, device="cuda").reshape(rows, cols) * 10
    acc, scale = tc_reference(oracle, A.cpu(), Bm.cpu(), False)
    c = C.double().cpu().numpy()
    want = {"max": np.maximum(c, acc), "min": np.minimum(c, acc), "mul": c * acc, "relu": np.maximum(acc, 0),
            "axpby": 0.5 * acc - 2.0 * c, "new": acc, "scaled": 0.5 * acc}[comb]
    bound = {"mul": scale * np.abs(c), "axpby": 0.5 * scale + 2.0 * np.abs(c)}.get(comb, scale + (np.abs(c) if comb in ("max", "min") else 0))
    D = klas.gemm_tc(A, Bm, out_dtype=torch.float32, C_=C, D=torch.empty_like(C), alpha=0.5, beta=-2.0, comb=comb)
    torch.cuda.synchronize()
    assert rel_err_componentwise(D.cpu().numpy(), want, bound) <= 1e-5
    if comb in ("new", "relu", "scaled"):
        if comb == "scaled":
            assert klas.gemm_tc(A, Bm, out_dtype=torch.float32, alpha=0.5, comb=comb).equal(D)
            return
        assert klas.gemm_tc(A, Bm, out_dtype=torch.float32, comb=comb).equal(D)   # C is not read


def test_map_and_combine_together_in_place(oracle):
    A, Bm = synth.gemm_bf16(15, 512, 768, 256, b_col_major=False, device="cuda")
    C = torch.ones((512, 768), dtype=torch.float32, device="cuda")
    acc, scale = tc_reference(oracle, mapped(oracle, A, "abs"), mapped(oracle, Bm, "square"), False)
    klas.gemm_tc(A, Bm, out_dtype=torch.float32, C_=C, D=C, map_a="abs", map_b="square", comb="max")
    torch.cuda.synchronize()
    assert rel_err_componentwise(C.cpu().numpy(), np.maximum(1.0, acc), scale + 1.0) <= 1e-5


def test_batched_pages_with_a_map(oracle):
    A, B = synth.gemm_f16_batched(16, 3, 256, 256, 128, device="cuda")
    D = klas.gemm_tc(A, B, out_dtype=torch.float16, map_b="abs")
    torch.cuda.synchronize()
    for i in range(3):
        acc, scale = tc_reference(oracle, A[i].cpu(), mapped(oracle, B[i], "abs"), False)
        assert rel_err_componentwise(D[i].double().cpu().numpy(), acc, scale) <= TOL_F16_OUT


def test_bad_arguments():
    A = torch.zeros((128, 64), dtype=torch.bfloat16, device="cuda")
    B = torch.zeros((64, 128), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        klas.gemm_tc(A, B, map_a="exp")
    with pytest.raises(klas.KlasError):
        klas.gemm_tc(A, B, comb="max")          # needs C
