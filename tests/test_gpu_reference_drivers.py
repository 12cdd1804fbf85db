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
