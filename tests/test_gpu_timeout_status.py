"""Failure detection without a GPU fault: a device-side wait that runs out returns an error
status the host reads, and the context stays usable (no trap, no hang, no bad address)."""
import time

import numpy as np
import pytest
import torch

from gpu_util import rel_err_componentwise, tc_reference
from kuiper_b200 import _lib, klas, synth

pytestmark = pytest.mark.gpu


def matches_oracle(oracle, A, Bt, D):
    acc, scale = tc_reference(oracle, A.cpu(), Bt.cpu(), True)
    return rel_err_componentwise(D.cpu().numpy(), acc, scale) <= 2e-3


def test_bounded_wait_gives_up_and_reports(oracle):
    lib = _lib.load()
    assert klas.gemm_tc_status() == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    t0 = time.perf_counter()
    _lib.check(lib.klas_b200_debug_wait_probe(50, gave_up.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.04 <= elapsed < 1.0                      # waited about the 50 ms limit, then returned
    assert int(gave_up.item()) == 1
    assert lib.klas_b200_gemm_tc_status_peek() == 0x7F   # visible to the host without a device round trip
    with pytest.raises(klas.KlasError) as e:
        klas.gemm_tc_status()
    assert e.value.status == _lib.ERR_TIMEOUT and "0x7f" in str(e.value)
    assert klas.gemm_tc_status() == 0                 # reading the status clears it

    # the context is still usable and the next GEMM is correct
    A, Bt = synth.gemm_bf16(1, 256, 256, 128, device="cuda")
    D = klas.gemm_tc(A, Bt, b_col_major=True)
    torch.cuda.synchronize()
    assert lib.klas_b200_gemm_tc_status_peek() == 0   # the host-visible mirror agrees
    assert matches_oracle(oracle, A, Bt, D)
    assert klas.gemm_tc_status() == 0


def test_stale_status_makes_launches_drain_until_cleared(oracle):
    """While the status word is non-zero the pipeline's waits give up at once, so a GEMM launched
    before the host has looked returns promptly; after the status is read, results are right."""
    lib = _lib.load()
    _lib.check(lib.klas_b200_debug_wait_probe(5, None, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    A, Bt = synth.gemm_bf16(2, 1024, 512, 512, device="cuda")
    t0 = time.perf_counter()
    klas.gemm_tc(A, Bt, b_col_major=True)             # drains: output undefined
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0
    with pytest.raises(klas.KlasError):
        klas.gemm_tc_status()
    D = klas.gemm_tc(A, Bt, b_col_major=True)
    torch.cuda.synchronize()
    assert klas.gemm_tc_status() == 0
    assert matches_oracle(oracle, A, Bt, D)


def test_probe_rejects_bad_limits():
    lib = _lib.load()
    assert lib.klas_b200_debug_wait_probe(0, None, None) == _lib.ERR_INVALID
    assert lib.klas_b200_debug_wait_probe(5000, None, None) == _lib.ERR_INVALID
