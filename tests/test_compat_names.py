"""The reference-name layer: the compatibility objects export exactly the reference's mangled
symbols, the instance grids match, and the public headers still compile as the reference's do."""
import subprocess
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def compat():
    from kuiper_b200 import build
    build.build_compat()
    return build


def exported(path):
    out = subprocess.run(["nm", "--defined-only", str(path)], capture_output=True, text=True, check=True).stdout
    return {p[2] for p in (line.split() for line in out.splitlines()) if len(p) == 3 and p[1] == "T"}


def test_every_reference_symbol_is_exported(compat):
    want = set((GOLD / "klas_symbols.txt").read_text().split())
    assert len(want) == 598
    got = set()
    for obj in sorted(compat.COMPAT_OUT.glob("K*.o")):
        got |= exported(obj)
    assert want <= got, sorted(want - got)[:5]
    assert got == want            # and nothing else with external linkage


def test_one_object_per_reference_header(compat):
    units = {p.stem for p in compat.COMPAT_OUT.glob("K*.o")}
    assert units == {"Klas_GEMM_SHMem", "Klas_GEMM_Tiled", "Klas_GEMM_BlockTiling1D", "Klas_GEMM_BlockTiling2D",
                     "Klas_GEMM_Naive1", "Klas_GEMM_Naive2", "Klas_GEMM_Naive3", "Klas_GEMM_TensorCore",
                     "Klas_GEMM_TensorCore2D", "Klas_GEMM_TensorCore2D_To", "Klas_SPMM", "Klas_Softmax",
                     "Klas_LogSoftmax", "Klas_RowSoftmax", "Klas_RowScale", "Klas_HReduce", "Klas_AtomicReduce",
                     "Kuiper_Example_Fused_GEMM", "Kuiper_GraphDist"}
    for u in units:
        assert (REPO / "include" / "klas" / (u + ".h")).exists()


def test_grids_regenerate_identically(tmp_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen_grids", REPO / "kuiper_b200" / "csrc" / "compat" / "gen_grids.py")
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    assert len(list(gen.tc2d())) == 72 and len(list(gen.bt2d())) == 72 and len(list(gen.spmm())) == 91
    gen.OUT = tmp_path
    gen.main()
    for name in ("tc2d.inc", "bt2d.inc", "spmm.inc"):
        assert (tmp_path / name).read_text() == (REPO / "include" / "klas" / "grids" / name).read_text()


def test_python_mirror_knows_every_reference_name():
    """kuiper_b200.klas.call() parses every exported entry-point name."""
    from kuiper_b200 import klas
    names = [n.split("(")[0] for n in subprocess.run(["c++filt"], input=(GOLD / "klas_symbols.txt").read_text(),
                                                      capture_output=True, text=True, check=True).stdout.split("\n") if n]
    assert len(names) == 598
    pats = [klas._RE_TILED, klas._RE_BT2D, klas._RE_NAIVE, klas._RE_NAIVE_B, klas._RE_TC2D, klas._RE_TC2D_TO,
            klas._RE_TC1D, klas._RE_SPMM, klas._RE_SOFTMAX, klas._RE_ROWSOFTMAX, klas._RE_ROWSCALE, klas._RE_REDUCE, klas._RE_FUSED, klas._RE_GRAPHDIST]
    for n in names:
        assert any(p.match(n) for p in pats), n


def test_shim_header_serves_kuiper_h_users(tmp_path):
    src = tmp_path / "t.cu"
    src.write_text('#include <kuiper.h>\n#include "Klas_SPMM.h"\n#include "Klas_GEMM_TensorCore2D_To.h"\n'
                   '__global__ void k(int *p) { char *s = (char *)KPR_SHMEM_AT(4); p[0] = s[0]; }\n'
                   'int main() { void *p = KPR_GPU_ALLOC(4, 1); cudaStream_t s = KPR_FRESH_STREAM();\n'
                   '  KPR_KCALL(k, 0, 32, 16, s, (int *)p); KPR_GUARD(1 == 1); KPR_ASSERT(2 > 1); KPR_SHMEM_FITS(100);\n'
                   '  MUST(cudaStreamDestroy(s)); Kuiper_Sparse_Matrix_smatrix__float m; m.nnz = 0; return (int)m.nnz; }\n')
    subprocess.run(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(REPO / "include" / "klas"),
                    "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


SHIM_USER = r"""
#include <kuiper.h>
__global__ void k(half *h, __nv_bfloat16 *b, float *f, double *d, uint32_t *u, uint64_t *w, float4 *v) {
    h[0] = kpr_hfma(kpr_hsqrt(h[1]), kpr_htanh(h[2]), kpr_hpow(h[3], h[4]));
    h[5] = kpr_hfabs(kpr_hexp2(kpr_hlog2(__hrcp(h[6]))));
    b[0] = kpr_bf16fma(kpr_bf16add(b[1], b[2]), kpr_bf16mul(b[3], b[4]), kpr_bf16exp(kpr_bf16tanh(b[5])));
    b[6] = kpr_bf16atan2(kpr_bf16div(b[1], b[2]), kpr_bf16sub(b[3], b[4]));
    atomic_add_f32(f, 1.f); atomic_add_f64(d, 1.0); atomic_add_u32(u, 1u); atomic_add_u64(w, 1ull);
    vec_memcpy(v, v + 1);
    kpr_fragment(wmma::matrix_a, 16, 16, 16, half, wmma::row_major) fa;
    kpr_fragment(wmma::accumulator, 16, 16, 16, float) acc;
    wmma::fill_fragment(acc, 0.f);
    KPR_LOAD_MAP(h, fa, 16, kpr_hsqrt(_kpr_in_v));
    KPR_STORE_COMB(f, acc, 16, _kpr_old_v + 2.f * _kpr_new_v);
}
int main() { INFO(); half x = kpr_hsqrt(HLF_MAX); (void)x; MUST(cudaDeviceSynchronize()); return 0; }
"""


def test_runtime_shim_provides_the_sub_headers(tmp_path):
    """<kuiper.h> of the reference pulls in kuiper/atomics.h, vectorops.h, math.h and tensorcores.h and
    defines INFO() (include/kuiper.h:12-19,111-123): a translation unit that uses a name from each
    must compile against this repository's include directory (nvcc cross-compiles without a GPU)."""
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = tmp_path / "shim_user.cu"
    src.write_text(SHIM_USER)
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I", str(REPO / "include" / "klas"),
                    "-c", str(src), "-o", str(tmp_path / "shim_user.o")], check=True)
