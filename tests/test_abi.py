"""The C-ABI library builds for sm_100a, loads without a GPU, and exports every symbol
include/klas_b200.h declares (no compute calls here)."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "klas_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(klas_b200_\w+)\s*\(", text)))


@pytest.fixture(scope="module")
def libpath():
    from kuiper_b200 import build
    return build.build_library()


def test_header_is_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "klas_b200.h"\nint main(void) { return klas_b200_version() == 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", str(REPO / "include"), str(src)],
                   check=True)


def test_library_exports_every_declared_symbol(libpath):
    lib = ctypes.CDLL(str(libpath))
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), "missing export: " + n


def test_python_binding_covers_the_header(libpath):
    from kuiper_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()
    lib = _lib.load()
    assert lib.klas_b200_version() == 1000
    assert lib.klas_b200_last_error() == b""


def test_exports_have_c_linkage(libpath):
    out = subprocess.run(["nm", "-D", "--defined-only", str(libpath)], capture_output=True, text=True, check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    for n in declared_functions():
        assert n in exported


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from kuiper_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError):
        _lib.load()


def test_wrappers_reject_mismatched_page_counts_before_any_launch():
    """A 3-D A with a 2-D B, or operands with different page counts, would make the kernel read
    pages of B that do not exist: the wrappers must raise on the host (no GPU is touched here)."""
    import torch
    from kuiper_b200 import klas
    a3 = torch.zeros((4, 64, 32), dtype=torch.bfloat16)
    b2 = torch.zeros((32, 64), dtype=torch.bfloat16)
    b3 = torch.zeros((2, 32, 64), dtype=torch.bfloat16)
    for bad in (b2, b3):
        with pytest.raises(ValueError):
            klas.gemm_tc(a3, bad)
    f3 = torch.zeros((4, 8, 8))
    with pytest.raises(ValueError):
        klas.gemm(f3, torch.zeros((8, 8)))
    with pytest.raises(ValueError):
        klas.gemm(f3, torch.zeros((3, 8, 8)))
