"""The multi-GPU entry points through a C program (tests/mg_driver.c) that links libklas_b200.so the
way a C or C++ consumer would: sharded bf16 GEMM, u64 GEMM and SpMM, gathered through NCCL, compared
bit for bit with the single-GPU product.  Runs on as many GPUs as the box has (up to 4); on one GPU
the shard and gather code still runs, with one shard."""
import shutil
import subprocess
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    from kuiper_b200 import build
    lib = build.build_library()
    cuda = Path(shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc").resolve().parent.parent
    exe = tmp_path_factory.mktemp("mg") / "mg_driver"
    subprocess.run(["gcc", "-std=c99", "-O1", "-Wall", "-o", str(exe), str(REPO / "tests" / "mg_driver.c"),
                    "-I", str(REPO / "include"), "-I", str(cuda / "include"), "-L", str(lib.parent), "-lklas_b200",
                    "-L", str(cuda / "lib64"), "-lcudart", "-Wl,-rpath," + str(lib.parent), "-Wl,-rpath," + str(cuda / "lib64")],
                   check=True)
    return exe


@pytest.mark.parametrize("devices", [1, 2, 4])
def test_c_consumer(driver, devices):
    if torch.cuda.device_count() < devices:
        pytest.skip("needs %d GPUs" % devices)
    r = subprocess.run([str(driver), str(devices)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.strip().endswith("OK")
    assert "DIFFERENT" not in r.stdout
