"""The tensor-core GEMM's choice of kernel, tile width and K split is host arithmetic on the shape
and the SM count (klas_b200_gemm_tc_plan): checked here without a GPU against what the tuning run
(python -m kuiper_b200.tune_tc) measured fastest on 148 SMs."""
import ctypes as C

import pytest

from kuiper_b200 import _lib, klas


@pytest.fixture(autouse=True)
def knobs_at_rest():
    lib = _lib.load()
    for knob in (_lib.KNOB_TC_MODE, _lib.KNOB_TC_KSPLIT, _lib.KNOB_TC_TAIL):
        assert lib.klas_b200_debug_set(knob, 0) == _lib.OK
    yield
    for knob in (_lib.KNOB_TC_MODE, _lib.KNOB_TC_KSPLIT, _lib.KNOB_TC_TAIL):
        lib.klas_b200_debug_set(knob, 0)


# rows, cols, shared -> what measured fastest (profiles/gemm_umma_tile_shapes_tuning.md)
GRID = [
    ((1024, 1024, 1024), dict(kind="single", tile_cols=64, k_parts=1, tail_cut=False)),
    ((2048, 2048, 2048), dict(kind="single", tile_cols=256, k_parts=1, tail_cut=False)),
    ((2560, 2048, 4096), dict(kind="pair", tile_cols=256, k_parts=1, tail_cut=True)),
    ((3072, 3072, 3072), dict(kind="wide", tile_cols=256, k_parts=1, tail_cut=False)),
    ((3584, 3072, 4096), dict(kind="pair", tile_cols=256, k_parts=1, tail_cut=False)),
    ((4096, 4096, 4096), dict(kind="wide", tile_cols=256, k_parts=1, tail_cut=False)),
    ((8192, 8192, 8192), dict(kind="wide", tile_cols=256, k_parts=1, tail_cut=False)),
    ((8192, 1024, 8192), dict(kind="wide", tile_cols=256, k_parts=1, tail_cut=False)),
    ((8192, 8192, 512), dict(kind="single", tile_cols=256, k_parts=1, tail_cut=False)),
    ((8192, 8192, 2048), dict(kind="pair", tile_cols=256, k_parts=1, tail_cut=False)),
    ((1024, 1024, 4096), dict(kind="single", tile_cols=256, k_parts=4, tail_cut=False)),
    ((512, 512, 8192), dict(kind="single", tile_cols=256, k_parts=8, tail_cut=False)),
    ((1536, 1536, 512), dict(kind="single", tile_cols=128, k_parts=1, tail_cut=False)),
    ((2560, 2048, 8192), dict(kind="pair", tile_cols=256, k_parts=1, tail_cut=True)),
]


@pytest.mark.parametrize("shape,want", GRID)
def test_plan_on_148_sms(shape, want):
    rows, cols, shared = shape
    assert klas.gemm_tc_plan(rows, shared, cols, sm_count=148) == want


def test_batched_f16_configuration_takes_pair_tiles():
    # 64 pages of 2048^3: the wide tile's unhidden drain costs more than the pair tile's lower rate at K = 2048
    assert klas.gemm_tc_plan(2048, 2048, 2048, batch=64)["kind"] == "pair"
    # pages are never cut along K together with a tail launch
    assert klas.gemm_tc_plan(2560, 2048, 8192, batch=2)["tail_cut"] is False


def test_knobs_force_the_plan():
    lib = _lib.load()
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_MODE, 4) == _lib.OK          # wide
    assert klas.gemm_tc_plan(1024, 1024, 1024)["kind"] == "wide"
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_MODE, 5) == _lib.OK          # 128 x 64
    assert klas.gemm_tc_plan(8192, 8192, 8192) == dict(kind="single", tile_cols=64, k_parts=1, tail_cut=False)
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_MODE, 0) == _lib.OK
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_KSPLIT, 1) == _lib.OK        # never split
    assert klas.gemm_tc_plan(1024, 4096, 1024)["k_parts"] == 1
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_KSPLIT, 3) == _lib.OK        # three parts where the kernel can
    assert klas.gemm_tc_plan(2048, 2048, 2048)["k_parts"] == 3
    assert klas.gemm_tc_plan(8192, 8192, 8192)["k_parts"] == 1               # the wide tile is never cut
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_KSPLIT, 0) == _lib.OK
    assert lib.klas_b200_debug_set(_lib.KNOB_TC_TAIL, 1) == _lib.OK          # no tail launch
    assert klas.gemm_tc_plan(2560, 8192, 2048)["tail_cut"] is False


def test_small_devices_and_bad_arguments():
    # one SM: no CTA pairs, so never pair or wide tiles
    assert klas.gemm_tc_plan(8192, 8192, 8192, sm_count=1)["kind"] == "single"
    lib = _lib.load()
    kind = C.c_int()
    assert lib.klas_b200_gemm_tc_plan(128, 128, 128, 1, 0, C.byref(kind), None, None, None) == _lib.ERR_INVALID
    assert lib.klas_b200_gemm_tc_plan(128, 128, 128, 1, 148, None, None, None, None) == _lib.OK
