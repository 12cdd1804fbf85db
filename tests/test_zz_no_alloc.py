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
TOL = {torch.float64: 1e-13, torch.float32: 2e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}   # as in test_gpu_rowops.py
CODE = {torch.float64: _lib.F64, torch.float32: _lib.F32, torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}


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


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.float16, torch.bfloat16])
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


def test_against_the_oracle_directly(oracle):
    """Not only through its sibling: the fixed-array entry point against the CPU oracle's float64
    softmax and log-softmax (the reference drivers' gold functions), two calls in a row."""
    lib = _lib.load()
    for seed, n, log in [(5, 1_000_003, False), (6, 70_001, True)]:
        x = vector(seed, n, torch.float32)
        got = static(lib, x, log)
        torch.cuda.synchronize()
        want = oracle.softmax(x.double().cpu().numpy(), log=log)
        tol = TOL[torch.float32] * (32.0 if log else 1.0)
        assert float(np.abs(got.double().cpu().numpy() - want).max()) <= tol


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
    reserved_mid = torch.cuda.memory_reserved()
    for _ in range(3):
        _lib.check(lib.klas_b200_softmax_static(_lib.F32, 0, out.numel(), out.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    # The device-wide free-memory figure must not drop by an allocation of ours.  It is shared with
    # whatever else runs on the GPU, so allow a little noise instead of demanding equality; any
    # allocation the entry point made (the driver hands out 2 MiB granules) would show.
    assert free_mid - free_after < (1 << 20) and free_mid <= free_before
    # and torch's own allocator, which the entry point must not go through either, did not grow
    assert torch.cuda.memory_reserved() == reserved_mid


def test_empty_vector_and_bad_dtype():
    lib = _lib.load()
    assert lib.klas_b200_softmax_static(_lib.F32, 0, 0, None, None) == _lib.OK
    y = torch.zeros(8, dtype=torch.int32, device="cuda")
    assert lib.klas_b200_softmax_static(_lib.U32, 0, 8, y.data_ptr(), None) == _lib.ERR_INVALID
