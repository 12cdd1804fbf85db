"""Runs the reference's own test drivers -- compiled unchanged from the reference tree and linked
against this library (oracle/_ref/drivers, built by oracle/build.py) -- and compares their stdout
with the reference's golden stdout, byte for byte (the rule of the reference's `make test`,
nvcc.mk:32-41 and scripts/diff.sh)."""
import json
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent
DRIVERS = REPO / "oracle" / "_ref" / "drivers"
EXPECTED = json.loads((Path(__file__).parent / "golden" / "driver_expected.json").read_text())


@pytest.mark.parametrize("name", sorted(EXPECTED))
def test_driver_prints_its_expected_output(name):
    exe = DRIVERS / (name + ".exe")
    if not exe.exists():
        pytest.skip("driver not built (the reference tree was not available at build time)")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=180)   # nvcc.mk:33 allows 180 s
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout == EXPECTED[name], r.stderr[-2000:]


def test_all_hot_path_drivers_are_covered():
    assert len(EXPECTED) == 51   # 37 GEMM + 2 SpMM + 6 softmax / log-softmax + 5 reductions + graph distances
    if DRIVERS.exists():
        built = {p.stem for p in DRIVERS.glob("*.exe")}
        assert built == set(EXPECTED)


@pytest.mark.parametrize("name,args,stem", [
    ("Tune_Klas_GEMM_BlockTiling2D", ["3", "1024", "1024", "1024", "1"], "Klas_GEMM_BlockTiling2D_g_gemm_f32_128x128x32_8x8"),
    # check flag 0, as tuning/tune_tc2d.sh runs it: this driver's own gold applies alpha = 0.7, which the
    # alpha-free TensorCore2D entry points do not take
    ("Tune_Klas_GEMM_TensorCore2D", ["3", "1024", "1024", "1024", "0"], "Klas_GEMM_TensorCore2D_g_gemm_f16_f16_128x128x32_16x16x16_2x2"),
    ("Tune_Klas_SPMM", ["3", "2048", "2048", "512", "5"], "Klas_SPMM_g_spmm_f32_16x16x16"),
])
def test_tuning_driver_runs_unchanged(name, args, stem):
    """The reference's tuning harness (test/Tune_*.cu, compiled with -Dstem=<entry point> as tuning/*.sh do)
    against this library: exits 0 and reports a timing line for the entry point."""
    exe = REPO / "oracle" / "_ref" / "tune" / (name + ".exe")
    if not exe.exists():
        pytest.skip("tuning driver not built (the reference tree was not available at build time)")
    r = subprocess.run([str(exe)] + args, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, (r.stdout[-1000:], r.stderr[-1000:])
    assert ">> RES" in r.stderr + r.stdout and stem in r.stderr + r.stdout
