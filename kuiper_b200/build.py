"""In-tree nvcc build of libklas_b200.so (sm_100a only).

`python -m kuiper_b200.build` (re)builds the shared library next to the
package; the library has no Python or torch dependency and is what a C, C++
or FFI caller links against.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libklas_b200.so"
INCLUDE_DIR = REPO_DIR / "include"

SOURCES = ["abi.cu", "gemm_umma.cu", "gemm_simt.cu", "spmm.cu", "rowops.cu", "minplus.cu", "csr_build.cu", "gemm_dmma.cu", "attention.cu", "multi_gpu.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def nvcc_path() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: cannot build libklas_b200.so")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every .cu of the package into one shared library; returns its path."""
    srcs = [CSRC / s for s in SOURCES]
    deps = srcs + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [INCLUDE_DIR / "klas_b200.h"]
    if not force and not _stale(LIB_PATH, deps):
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    objs = []
    procs = []
    for s in srcs:
        obj = LIB_DIR / (s.stem + ".o")
        objs.append(obj)
        cmd = [nvcc_path(), *NVCC_FLAGS, "-I", str(INCLUDE_DIR), "-I", str(CSRC), "-c", str(s), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), out))
    link = [nvcc_path(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
            "-o", str(LIB_PATH), *map(str, objs), "-ldl"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed: %s\n%s" % (" ".join(link), r.stdout))
    return LIB_PATH


COMPAT_DIR = CSRC / "compat"
COMPAT_OUT = LIB_DIR / "compat"
COMPAT_LIB = LIB_DIR / "libklas_compat.so"


def build_compat(force: bool = False) -> Path:
    """Compiles one object per reference header (lib/compat/Klas_*.o, to be linked where the
    reference links its own Klas_*.o) and bundles them into lib/libklas_compat.so."""
    build_library(force=False)
    COMPAT_OUT.mkdir(parents=True, exist_ok=True)
    hdrs = sorted((INCLUDE_DIR / "klas").rglob("*.h")) + sorted((INCLUDE_DIR / "klas").rglob("*.inc")) + \
        [COMPAT_DIR / "compat_common.h", INCLUDE_DIR / "klas_b200.h"]
    procs, objs = [], []
    for src in sorted(COMPAT_DIR.glob("Klas_*.cu")) + sorted(COMPAT_DIR.glob("Kuiper_*.cu")):
        obj = COMPAT_OUT / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + hdrs):
            cmd = [nvcc_path(), "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC",
                   "-I", str(INCLUDE_DIR), "-I", str(INCLUDE_DIR / "klas"), "-I", str(COMPAT_DIR), "-c", str(src), "-o", str(obj)]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: %s\n%s" % (" ".join(cmd), out))
    if procs or not COMPAT_LIB.exists():
        link = [nvcc_path(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(COMPAT_LIB), *map(str, objs),
                "-L", str(LIB_DIR), "-lklas_b200", "-Xlinker", "-rpath=$ORIGIN"]
        r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s" % (" ".join(link), r.stdout))
    return COMPAT_LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_compat(force="--force" in sys.argv))
