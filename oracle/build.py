"""Builds the checkers: oracle/libklas_oracle.so (the CPU restatement, gcc) and --
only where the FStarLang/kuiper tree is mounted -- oracle/_ref/: the reference's own
host loops, GPU kernels and test drivers compiled from where they lie.

    KUIPER_REF_ROOT=/path/to/kuiper python oracle/build.py [--ref-root /path/to/kuiper] [--no-ref-gpu]

Outputs are git-ignored build products; nothing here is part of the product library.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
REPO_DIR = ORACLE_DIR.parent
if str(REPO_DIR) not in sys.path:
    sys.path.insert(0, str(REPO_DIR))
ORACLE_LIB = ORACLE_DIR / "libklas_oracle.so"
REF_DIR = ORACLE_DIR / "_ref"
def ref_root_from_env():
    """Where the FStarLang/kuiper tree is mounted: the KUIPER_REF_ROOT environment variable (or pass
    --ref-root on the command line).  None when it is not set or holds no dist/ directory."""
    v = os.environ.get("KUIPER_REF_ROOT")
    return Path(v) if v and (Path(v) / "dist").is_dir() else None
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

REF_GPU_UNITS = [
    "Klas_GEMM_SHMem", "Klas_GEMM_Tiled", "Klas_GEMM_BlockTiling1D", "Klas_GEMM_BlockTiling2D",
    "Klas_GEMM_Naive1", "Klas_GEMM_Naive2", "Klas_GEMM_Naive3", "Klas_GEMM_TensorCore",
    "Klas_GEMM_TensorCore2D", "Klas_GEMM_TensorCore2D_To", "Klas_SPMM",
    "Klas_Softmax", "Klas_LogSoftmax", "Klas_RowSoftmax", "Klas_RowScale", "Klas_HReduce", "Klas_AtomicReduce",
    "Kuiper_Example_Fused_GEMM", "Kuiper_GraphDist",
]


def _run(cmd, **kw):
    r = subprocess.run(list(map(str, cmd)), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, **kw)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s" % (" ".join(map(str, cmd)), r.stdout))
    return r.stdout


def _newer(target: Path, *deps: Path) -> bool:
    return target.exists() and all(target.stat().st_mtime >= d.stat().st_mtime for d in deps if d.exists())


def build_oracle(force: bool = False) -> Path:
    src = ORACLE_DIR / "klas_oracle.c"
    if not force and _newer(ORACLE_LIB, src):
        return ORACLE_LIB
    _run(["gcc", "-O3", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-o", ORACLE_LIB, src, "-lm"])
    return ORACLE_LIB


def build_ref_cpu(ref_root: Path, force: bool = False) -> Path:
    """The reference's host gold loops (test/matmul_common.c.inc, dist/Kuiper_Example_Sparse_MM.cu)."""
    out = REF_DIR / "libklas_ref_cpu.so"
    wrap = ORACLE_DIR / "ref_wrap" / "ref_cpu.cu"
    wrap2 = ORACLE_DIR / "ref_wrap" / "ref_softmax.cu"
    wrap3 = ORACLE_DIR / "ref_wrap" / "ref_csr.cu"
    if not force and _newer(out, wrap, wrap2, wrap3):
        return out
    REF_DIR.mkdir(exist_ok=True)
    _run(["nvcc", "-O3", "-std=c++17", *ARCH, "-Xcompiler", "-fPIC", "-shared",
          "-I", ref_root / "include", "-I", ref_root / "test", "-I", ref_root / "dist",
          "-o", out, wrap, wrap2, wrap3, ref_root / "dist" / "Kuiper_Example_Sparse_MM.cu"])
    return out


def build_ref_gpu(ref_root: Path, force: bool = False) -> Path:
    """The reference's extracted kernels (dist/Klas_*.cu and the fused-map demo) for sm_100a, one shared library,
    plus symbols.json mapping each entry-point name to its mangled symbol."""
    out = REF_DIR / "libklas_ref_gpu.so"
    if not force and out.exists() and (REF_DIR / "symbols.json").exists() and \
            all((REF_DIR / "obj" / (u + ".o")).exists() for u in REF_GPU_UNITS):
        return out
    obj_dir = REF_DIR / "obj"
    obj_dir.mkdir(parents=True, exist_ok=True)

    def compile_unit(unit):
        obj = obj_dir / (unit + ".o")
        if force or not obj.exists():
            _run(["nvcc", "-O3", *ARCH, "-Xcompiler", "-fPIC", "-I", ref_root / "include",
                  "-I", ref_root / "dist", "-DKUIPER_CFG_TENSORCORES=1",
                  "-c", ref_root / "dist" / (unit + ".cu"), "-o", obj])
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_unit, REF_GPU_UNITS))
    _run(["nvcc", "-shared", *ARCH, "-o", out, *objs])
    names = {}
    for line in _run(["nm", "-D", "--defined-only", out]).splitlines():
        parts = line.split()
        if len(parts) == 3 and parts[1] == "T" and any(t in parts[2] for t in ("Klas_", "Kuiper_Example_Fused_GEMM", "Kuiper_GraphDist")):
            demangled = _run(["c++filt", parts[2]]).strip()
            names[demangled.split("(")[0]] = parts[2]
    (REF_DIR / "symbols.json").write_text(json.dumps(names, indent=0, sort_keys=True))
    return out


def build_ref_spmm_noguard(ref_root: Path, force: bool = False) -> Path:
    """The reference's SpMM unit with its `< 10000` size guards compiled out (oracle/ref_wrap/
    ref_spmm_noguard.cu): lets the benchmark time the reference's own kernel at 131072^2."""
    out = REF_DIR / "libklas_ref_spmm_noguard.so"
    wrap = ORACLE_DIR / "ref_wrap" / "ref_spmm_noguard.cu"
    if not force and _newer(out, wrap):
        return out
    REF_DIR.mkdir(exist_ok=True)
    _run(["nvcc", "-O3", *ARCH, "-Xcompiler", "-fPIC", "-shared", "-I", ref_root / "include", "-I", ref_root / "dist",
          "-o", out, wrap])
    return out


HOT_PATH_DRIVER_GLOBS = ("Test_Kuiper_GraphDist.cu", "Test_Klas_GEMM_*.cu", "Test_Klas_SPMM__*.cu", "Test_Klas_Softmax__*.cu",
                         "Test_Klas_LogSoftmax__*.cu", "Test_Klas_HReduce__*.cu", "Test_Klas_AtomicReduce__*.cu")


def build_ref_drivers(ref_root: Path, force: bool = False) -> Path:
    """The reference's own hot-path test drivers (test/Test_Klas_GEMM_*.cu, test/Test_Klas_SPMM__*.cu),
    compiled UNCHANGED from where they lie, against this repository's headers (include/klas) and linked
    with this repository's compatibility objects and libklas_b200.so -- the reference's link rule
    Test_X__Y.exe = Test_X__Y.o + X.o (nvcc.mk:13,22-26) with X.o replaced.  Also writes
    expected/<driver>.txt = the reference's golden stdout (test/*.output.expected)."""
    from kuiper_b200 import build as lib_build
    lib_build.build_compat()
    out_dir = REF_DIR / "drivers"
    out_dir.mkdir(parents=True, exist_ok=True)
    inc = REPO_DIR / "include"
    srcs = sorted(p for g in HOT_PATH_DRIVER_GLOBS for p in (ref_root / "test").glob(g))

    def one(src: Path):
        exe = out_dir / (src.stem + ".exe")
        if not force and exe.exists() and exe.stat().st_mtime >= (lib_build.COMPAT_LIB.stat().st_mtime):
            return exe
        unit = src.stem[len("Test_"):].split("__")[0]          # Test_Klas_GEMM_SHMem__F32 -> Klas_GEMM_SHMem
        obj = lib_build.COMPAT_OUT / (unit + ".o")
        _run(["nvcc", "-O3", *ARCH, "-DKUIPER_CFG_TENSORCORES=1", "-I", inc / "klas", "-I", ref_root / "test",
              "-o", exe, src, obj, "-L", lib_build.LIB_DIR, "-lklas_b200",
              "-Xlinker", "-rpath=$ORIGIN/../../../kuiper_b200/lib"])
        return exe

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        exes = list(ex.map(one, srcs))
    build_ref_tuning_drivers(ref_root, force)
    return out_dir if exes else out_dir


# The reference's tuning drivers (test/Tune_*.cu) take the entry point to time as -Dstem=<name>
# (tuning/tune_b2d.sh, tune_tc2d.sh, tune_spmm.sh); one representative stem each is enough to show
# that they build and run against this library unchanged.
TUNING_DRIVERS = {
    "Tune_Klas_GEMM_BlockTiling2D": ("Klas_GEMM_BlockTiling2D", "Klas_GEMM_BlockTiling2D_g_gemm_f32_128x128x32_8x8"),
    "Tune_Klas_GEMM_TensorCore2D": ("Klas_GEMM_TensorCore2D", "Klas_GEMM_TensorCore2D_g_gemm_f16_f16_128x128x32_16x16x16_2x2"),
    "Tune_Klas_SPMM": ("Klas_SPMM", "Klas_SPMM_g_spmm_f32_16x16x16"),
}


def build_ref_tuning_drivers(ref_root: Path, force: bool = False) -> Path:
    from kuiper_b200 import build as lib_build
    out_dir = REF_DIR / "tune"
    out_dir.mkdir(parents=True, exist_ok=True)
    inc = REPO_DIR / "include"
    for name, (unit, stem) in TUNING_DRIVERS.items():
        src, exe = ref_root / "test" / (name + ".cu"), out_dir / (name + ".exe")
        if not src.exists() or (not force and exe.exists() and exe.stat().st_mtime >= lib_build.COMPAT_LIB.stat().st_mtime):
            continue
        _run(["nvcc", "-O3", *ARCH, "-DKUIPER_CFG_TENSORCORES=1", "-Dstem=" + stem, "-Dtile_sizes=", "-Dtc_tile_sizes=",
              "-Dregch_sizes=", "-Det_lbl=", "-I", inc / "klas", "-I", ref_root / "test", "-o", exe, src,
              lib_build.COMPAT_OUT / (unit + ".o"), "-L", lib_build.LIB_DIR, "-lklas_b200",
              "-Xlinker", "-rpath=$ORIGIN/../../../kuiper_b200/lib"])
    return out_dir


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", type=Path, default=ref_root_from_env(),
                    help="the FStarLang/kuiper tree (default: $KUIPER_REF_ROOT)")
    ap.add_argument("--no-ref-gpu", action="store_true")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args(argv)
    print(build_oracle(a.force))
    if a.ref_root is not None and (a.ref_root / "dist").is_dir():
        print(build_ref_cpu(a.ref_root, a.force))
        if not a.no_ref_gpu:
            print(build_ref_gpu(a.ref_root, a.force))
            print(build_ref_spmm_noguard(a.ref_root, a.force))
        print(build_ref_drivers(a.ref_root, a.force))
    else:
        print("reference tree not found (--ref-root / KUIPER_REF_ROOT): oracle/_ref not (re)built")
    return 0


if __name__ == "__main__":
    sys.exit(main())
