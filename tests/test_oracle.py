"""Pins the CPU oracle (oracle/klas_oracle.c): bit-for-bit against the golden values
produced by the reference's own host loops (tests/golden/klas_golden.npz) and, where
oracle/_ref is built, against those loops run live on further inputs."""
import hashlib
from pathlib import Path

import numpy as np
import pytest
import torch

from driver_inputs import bits16, tc_inputs, tiled_inputs
from kuiper_b200 import synth

GOLD = np.load(Path(__file__).parent / "golden" / "klas_golden.npz")
SMALL = (24, 40, 16)
TC_SMALL = (32, 48, 24)
BIG = (1024, 1024, 1024)
STRIDE = 4099


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8)


@pytest.mark.parametrize("kind,dt", [("f32", np.float32), ("f64", np.float64)])
def test_float_gold_small_and_driver_size(oracle, kind, dt):
    m1, m2, m3 = tiled_inputs(dt, *SMALL)
    assert np.array_equal(oracle.gemm(m1, m2), GOLD["mul_%s_small" % kind])
    m1, m2, _ = tiled_inputs(dt, *BIG)
    big = oracle.gemm(m1, m2, threads=0)
    assert np.array_equal(sha(big), GOLD["mul_%s_big_sha256" % kind])
    assert np.array_equal(big.reshape(-1)[::STRIDE], GOLD["mul_%s_big_samples" % kind])


def test_sgemm_f32_gold(oracle):
    m1, m2, m3 = tiled_inputs(np.float32, *SMALL)
    got = oracle.sgemm_f32(0.7, 0.3, m1, m2, m3)
    assert np.array_equal(got, GOLD["sgemm_f32_small"])


@pytest.mark.parametrize("kind,dt", [("u32", np.uint32), ("u64", np.uint64)])
def test_integer_gold(oracle, kind, dt):
    m1, m2, _ = tiled_inputs(dt, *SMALL)
    assert np.array_equal(oracle.gemm_int(m1, m2), GOLD["mul_%s_small" % kind])
    m1, m2, _ = tiled_inputs(dt, *BIG)
    big = oracle.gemm_int(m1, m2)
    if kind == "u64":
        # every sum of the driver's inputs stays below 2^53, where the reference's
        # double-accumulating gold loop is exact: bit-for-bit agreement
        assert np.array_equal(sha(big), GOLD["mul_u64_big_sha256"])
        assert np.array_equal(big.reshape(-1)[::STRIDE], GOLD["mul_u64_big_samples"])
    else:
        # u32 at the driver's size: sums reach ~3.6e9 < 2^32, still exact
        assert np.array_equal(sha(big), GOLD["mul_u32_big_sha256"])


def test_integer_wraparound_matches_python_bigints(oracle):
    rng = np.random.default_rng(5)
    for dt, bits in ((np.uint32, 32), (np.uint64, 64)):
        A = rng.integers(0, 1 << bits, size=(5, 7), dtype=dt)
        B = rng.integers(0, 1 << bits, size=(7, 3), dtype=dt)
        Cin = rng.integers(0, 1 << bits, size=(5, 3), dtype=dt)
        alpha, beta = (1 << bits) - 3, 12345
        got = oracle.gemm_int(A, B)
        got2 = oracle.gemm_int(A, B, Cin, alpha, beta)
        for i in range(5):
            for j in range(3):
                s = sum(int(A[i, l]) * int(B[l, j]) for l in range(7))
                assert int(got[i, j]) == s % (1 << bits)
                assert int(got2[i, j]) == (beta * int(Cin[i, j]) + alpha * s) % (1 << bits)


@pytest.mark.parametrize("kind,tdt", [("bf16_f32", torch.bfloat16), ("f16_f16", torch.float16)])
def test_tensor_core_driver_gold(oracle, kind, tdt):
    sub = "bf16" if kind == "bf16_f32" else "f16"
    A, B = tc_inputs(tdt, *TC_SMALL)
    assert np.array_equal(oracle.gemm(bits16(A), bits16(B), kind=sub), GOLD["mul_%s_small" % kind])
    A, B = tc_inputs(tdt, *BIG)
    big = oracle.gemm(bits16(A), bits16(B), kind=sub)
    assert np.array_equal(sha(big), GOLD["mul_%s_big_sha256" % kind])
    if kind == "f16_f16":
        # fp16 overflow to +inf is part of the drivers' gold
        assert int((big == 0x7c00).sum()) == int(GOLD["mul_f16_f16_big_inf_count"][0]) > 0


def test_f16_conversion_single_rounding(oracle):
    # every finite half value round-trips; ties go to even; 65520 overflows
    allbits = np.arange(0, 0x7c00, dtype=np.uint16)
    vals = oracle.f16_bits_to_f64(allbits)
    assert np.array_equal(oracle.to_f16_bits(vals), allbits)
    assert np.array_equal(oracle.to_f16_bits(-vals[1:]), allbits[1:] | 0x8000)
    assert np.array_equal(vals, torch.tensor(allbits.view(np.int16)).view(torch.float16).double().numpy())
    mid = (vals[:-1] + vals[1:]) / 2     # exact midpoints: must pick the even neighbour
    r = oracle.to_f16_bits(mid)
    assert np.array_equal(r, np.where(allbits[:-1] % 2 == 0, allbits[:-1], allbits[1:]))
    assert oracle.to_f16_bits(np.array([65519.999, 65520.0, 1e9, -65520.0])).tolist() == [0x7bff, 0x7c00, 0x7c00, 0xfc00]
    # double rounding trap: 1 + 2^-11 + 2^-30 must round up in one step
    x = np.array([1.0 + 2.0 ** -11 + 2.0 ** -30])
    assert oracle.to_f16_bits(x)[0] == 0x3c01


def test_bf16_conversion(oracle):
    x = torch.randn(4096, dtype=torch.float64) * 37.0
    ref = bits16(x.float().to(torch.bfloat16))   # float -> bf16 is a single rounding of the float
    got = oracle.to_bf16_bits(x.float().double().numpy())
    assert np.array_equal(got, ref)


def test_spmm_u32_gold(oracle):
    csr = synth.csr_poisson(11, 96, 80, 6.0, value_kind="u32")
    Bd = synth.spmm_dense_b(11, 80, 24, value_kind="u32")
    got = oracle.spmm_u32(96, 24, csr.elems.numpy().view(np.uint32), csr.col_ind.numpy().view(np.uint32),
                          csr.row_off.numpy().view(np.uint32), Bd.numpy().view(np.uint32))
    assert np.array_equal(got, GOLD["spmm_u32_small"])


def test_spmm_f32_matches_dense_product(oracle):
    csr = synth.csr_poisson(4, 64, 50, 5.0)
    Bd = synth.spmm_dense_b(4, 50, 12)
    dense = np.zeros((64, 50), np.float32)
    ro = csr.row_off.numpy()
    for r in range(64):
        dense[r, csr.col_ind.numpy()[ro[r]:ro[r + 1]]] = csr.elems.numpy()[ro[r]:ro[r + 1]]
    got, ab = oracle.spmm_f32(64, 12, csr.elems.numpy(), csr.col_ind.numpy().view(np.uint32),
                              ro.view(np.uint32), Bd.numpy(), with_abs=True)
    want = dense.astype(np.float64) @ Bd.numpy().astype(np.float64)
    assert np.allclose(got, want, rtol=0, atol=1e-12)
    assert np.all(ab >= np.abs(got) - 1e-12)
    # the drivers' float gold loop agrees within float rounding
    assert np.allclose(oracle.dense_matmul_f32(dense, Bd.numpy()), want, rtol=1e-5, atol=1e-5)


def test_softmax_gold(oracle):
    ramp = (np.arange(100) % 16) * 0.5 - 4.0
    assert np.array_equal(oracle.softmax(ramp), GOLD["softmax_ramp"])
    assert np.array_equal(oracle.softmax(ramp, log=True), GOLD["logsoftmax_ramp"])
    x = np.random.default_rng(1).normal(size=(5, 37)) * 4
    sm = oracle.softmax(x)
    assert np.allclose(sm.sum(axis=1), 1.0, atol=1e-14)
    assert np.allclose(np.log(sm), oracle.softmax(x, log=True), atol=1e-12)


def test_live_reference_softmax(oracle, refcpu):
    x = np.random.default_rng(2).normal(size=4097) * 5
    assert np.array_equal(oracle.softmax(x), refcpu.cpu_softmax(x))
    assert np.array_equal(oracle.softmax(x, log=True), refcpu.cpu_softmax(x, log=True))


def test_minplus_squaring_reaches_all_path_lengths(oracle):
    """The graph-distance driver's own check (test/Test_Kuiper_GraphDist.cu:55-95): on the path graph
    0 -> 1 -> ... -> n-1, repeated squaring ends with dist[i][j] = j - i above the diagonal, 0 elsewhere."""
    n = 70
    m1 = np.zeros((n, n), dtype=np.uint16)
    m1[np.arange(n - 1), np.arange(1, n)] = 1
    m2 = m1.copy()
    length = 1
    while length < n:
        m2 = oracle.minplus_u16(m1, m1, m2)
        m1, m2 = m2, m1
        length *= 2
    want = np.triu(np.arange(n)[None, :] - np.arange(n)[:, None], 1).astype(np.uint16)
    assert np.array_equal(m1, want)


def test_minplus_ring_laws(oracle):
    # 0 is absorbing for mult and neutral for add; x + y wraps at 2^16 as the reference's uint16 return does
    a = np.array([[0, 5, 40000]], dtype=np.uint16)
    b = np.array([[7], [0], [30000]], dtype=np.uint16)
    assert oracle.minplus_u16(a, b, np.zeros((1, 1), np.uint16))[0, 0] == (40000 + 30000) % 65536
    assert oracle.minplus_u16(a, b, np.array([[3]], np.uint16))[0, 0] == 3
    assert oracle.minplus_u16(a[:, :2], b[:2], np.array([[9]], np.uint16))[0, 0] == 9


def test_sparsify_and_row_order(oracle):
    M = np.array([[0, 1.5, -0.0, 2], [0, 0, 0, 0], [3, 0, 0, np.nan], [1, 1, 1, 1]], dtype=np.float32)
    row_off, elems, col_ind = oracle.sparsify(M)
    assert row_off.tolist() == [0, 2, 2, 4, 8]
    assert col_ind.tolist() == [1, 3, 0, 3, 0, 1, 2, 3]
    assert elems[:3].tolist() == [1.5, 2.0, 3.0] and np.isnan(elems[3])
    assert oracle.row_order(row_off).tolist() == [3, 0, 2, 1]      # longest first, ties by row


def test_live_reference_sparsify(oracle, refcpu):
    rng = np.random.default_rng(3)
    for dtype in (np.float32, np.uint32):
        M = (rng.integers(1, 99, size=(57, 83)) * (rng.random((57, 83)) < 0.2)).astype(dtype)
        got, want = oracle.sparsify(M), refcpu.sparsify(M)
        for g, w in zip(got, want):
            assert np.array_equal(g, w)
        # the reference's order is any permutation with non-increasing lengths; ours is one of them
        lens = np.diff(want[0].astype(np.int64))
        ref_order, our_order = refcpu.mk_row_indices(want[0]), oracle.row_order(want[0])
        assert sorted(ref_order.tolist()) == list(range(57)) == sorted(our_order.tolist())
        assert np.array_equal(lens[ref_order], lens[our_order])


# ------------------------------------------------------------------ live checks against oracle/_ref
@pytest.mark.parametrize("shape", [(7, 5, 3), (33, 65, 17), (128, 96, 64)])
def test_live_reference_loops(oracle, refcpu, shape):
    rng = np.random.default_rng(shape[0])
    A = rng.uniform(-1, 1, size=shape[:2]).astype(np.float32)
    B = rng.uniform(-1, 1, size=shape[1:]).astype(np.float32)
    Cin = rng.uniform(-1, 1, size=(shape[0], shape[2])).astype(np.float32)
    assert np.array_equal(oracle.gemm(A, B), refcpu.cpu_mul("f32", A, B))
    assert np.array_equal(oracle.sgemm_f32(0.7, 0.3, A, B, Cin), refcpu.cpu_sgemm("f32", A, B, Cin, 0.7, 0.3))
    Ad, Bd = A.astype(np.float64), B.astype(np.float64)
    assert np.array_equal(oracle.gemm(Ad, Bd), refcpu.cpu_mul("f64", Ad, Bd))
    for dt in (np.uint32, np.uint64):
        Ai = rng.integers(0, 3000, size=shape[:2]).astype(dt)
        Bi = rng.integers(0, 3000, size=shape[1:]).astype(dt)
        assert np.array_equal(oracle.gemm_int(Ai, Bi), refcpu.cpu_mul("u32" if dt == np.uint32 else "u64", Ai, Bi))
    Ah = torch.tensor(A).to(torch.float16)
    Bh = (torch.tensor(B) * 300).to(torch.float16)
    assert np.array_equal(oracle.gemm(bits16(Ah), bits16(Bh), kind="f16"),
                          refcpu.cpu_mul("f16_f16", bits16(Ah), bits16(Bh)))
    Ab, Bb = torch.tensor(A).to(torch.bfloat16), torch.tensor(B).to(torch.bfloat16)
    assert np.array_equal(oracle.gemm(bits16(Ab), bits16(Bb), kind="bf16"),
                          refcpu.cpu_mul("bf16_f32", bits16(Ab), bits16(Bb)))


def test_live_reference_csr_loop(oracle, refcpu):
    csr = synth.csr_poisson(21, 200, 150, 9.0, value_kind="u32")
    Bd = synth.spmm_dense_b(21, 150, 33, value_kind="u32")
    e, c, r, b = (csr.elems.numpy().view(np.uint32), csr.col_ind.numpy().view(np.uint32),
                  csr.row_off.numpy().view(np.uint32), Bd.numpy().view(np.uint32))
    assert np.array_equal(oracle.spmm_u32(200, 33, e, c, r, b), refcpu.mmsd_u32_rr(200, 150, 33, e, c, r, b))
