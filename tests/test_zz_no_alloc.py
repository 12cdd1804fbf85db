"""klas_b200_softmax_static: the vector softmax whose per-chunk statistics live in a fixed array
inside the library, for callers that can neither pass scratch nor allocate.  Called through the
C ABI and compared with klas_b200_softmax (caller scratch) on the same inputs.

The file name sorts last on purpose: the entry point must work after everything else has used
the device, and equally as the first call of a fresh process (run this file alone)."""
import numpy as np
import pytest
import torch

from kuiper_b200 import _lib, synth

pytestmark = pytest.mark.gpu

MAX_COLS = 16777216          # KLAS_B200_SOFTMAX_STATIC_MAX_COLS in include/klas_b200.h
TOL = {torch.float64: 1e-13, torch.float32: 2e-6, torch.float16: 1e-3}   # as in test_gpu_rowops.py
CODE = {torch.float64: _lib.F64, torch.float32: _lib.F32, torch.float16: _lib.F16}


def vector(seed, n, dtype):
    return (synth.normal(seed, 11, 0, n, dtype=torch.float64) * 4.0).to(dtype).cuda()


def with_caller_scratch(lib, x, log):
    out = x.clone()
    need = lib.klas_b200_softmax_scratch_bytes(1, out.numel())
    scratch = torch.empty(need, dtype=torch.uint8, device="cuda")
    _lib.check(lib.klas_b200_softmax(CODE[x.dtype], int(log), 1, out.numel(), out.data_ptr(),
                                     scratch.data_ptr(), need, torch.cuda.current_stream().cuda_stream))
    return out


def static(lib, x, log):
    out = x.clone()
    _lib.check(lib.klas_b200_softmax_static(CODE[x.dtype], int(log), out.numel(), out.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream))
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16])
def test_two_calls_in_a_row_match_the_scratch_entry_point(dtype):
    lib = _lib.load()
    # Second call is shorter and of other values: whatever the first left in the array must not leak.
    for seed, n, log in [(1, 3_000_001, False), (2, 40_000, True)]:
        x = vector(seed, n, dtype)
        want = with_caller_scratch(lib, x, log)
        got = static(lib, x, log)
        torch.cuda.synchronize()
        tol = TOL[dtype] * (32.0 if log else 1.0)        # log-softmax values are tens, not <= 1
        assert float((got.double() - want.double()).abs().max()) <= tol
        assert torch.equal(got, want)                     # same kernels, same chunking: bit-identical


def test_largest_size_and_one_beyond():
    lib = _lib.load()
    x = vector(3, MAX_COLS, torch.float32)
    want = with_caller_scratch(lib, x, False)
    got = static(lib, x, False)
    torch.cuda.synchronize()
    assert float((got - want).abs().max()) <= TOL[torch.float32]
    assert abs(float(got.double().sum()) - 1.0) <= 1e-4
    y = torch.zeros(MAX_COLS + 1, device="cuda")
    rc = lib.klas_b200_softmax_static(_lib.F32, 0, MAX_COLS + 1, y.data_ptr(), None)
    assert rc == _lib.ERR_TOO_LARGE
    assert b"at most" in lib.klas_b200_last_error()
    assert bool((y == 0).all())                           # refused before touching the data


def test_makes_no_device_allocation():
    lib = _lib.load()
    x = vector(4, 100_000, torch.float32)
    static(lib, x, False)                                 # set-up call for this device
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    out = x.clone()
    free_mid, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        _lib.check(lib.klas_b200_softmax_static(_lib.F32, 0, out.numel(), out.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_mid <= free_before          # the driver's free-memory figure did not move


def test_empty_vector_and_bad_dtype():
    lib = _lib.load()
    assert lib.klas_b200_softmax_static(_lib.F32, 0, 0, None, None) == _lib.OK
    y = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert lib.klas_b200_softmax_static(_lib.U32, 0, 8, y.data_ptr(), None) == _lib.ERR_INVALID
