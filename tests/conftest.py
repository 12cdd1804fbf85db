import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
for p in (REPO, REPO / "oracle", REPO / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    import build as oracle_build  # oracle/build.py
    oracle_build.build_oracle()
    from oracle_api import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def refcpu():
    from oracle_api import RefCpu
    if not RefCpu.available():
        pytest.skip("oracle/_ref/libklas_ref_cpu.so not built (reference tree not mounted)")
    return RefCpu()
