// Builds the reference's own host-side gold loops, from where they lie in the
// FStarLang/kuiper tree (test/matmul_common.c.inc, dist/Kuiper_Example_Sparse_MM.cu),
// into a shared library with C entry points.  Used only to pin oracle/klas_oracle.c.
// Compile with: -I <kuiper>/include -I <kuiper>/test -I <kuiper>/dist
#include <unistd.h>
#include <inttypes.h>
#include <math.h>
#include "test-common.h"
#include "Kuiper_Example_Sparse_MM.h"

// Each namespace gets its own copy of cpu_mul / cpu_sgemm for one element type.
#define TOLERANCE 0.0f

namespace ref_f32 {
#define et float
#include "matmul_common.c.inc"
#undef et
}
namespace ref_f64 {
#define et double
#include "matmul_common.c.inc"
#undef et
}
namespace ref_u32 {
#define et uint32_t
#include "matmul_common.c.inc"
#undef et
}
namespace ref_u64 {
#define et uint64_t
#include "matmul_common.c.inc"
#undef et
}
#undef cet
namespace ref_bf16_f32 {
#define et __nv_bfloat16
#define et_is_bf16 1
#define mix_prec 1
#define cet float
#include "matmul_common.c.inc"
#undef et
#undef et_is_bf16
#undef mix_prec
#undef cet
}
namespace ref_f16_f16 {
#define et half
#define et_is_half 1
#include "matmul_common.c.inc"
#undef et
#undef et_is_half
#undef cet
}

#define EXPORT_MUL(NS, ET, CET)                                                              \
    extern "C" void ref_cpu_mul_##NS(size_t rows, size_t shared, size_t cols, ET *m1, ET *m2, \
                                     CET *out) {                                             \
        CET *r = ref_##NS::cpu_mul(rows, shared, cols, m1, m2);                              \
        memcpy(out, r, rows * cols * sizeof(CET));                                           \
        free(r);                                                                             \
    }                                                                                        \
    extern "C" void ref_cpu_sgemm_##NS(size_t rows, size_t shared, size_t cols, ET *m1,      \
                                       ET *m2, CET *m3, const CET *alpha, const CET *beta,   \
                                       CET *out) {                                           \
        CET *r = ref_##NS::cpu_sgemm(rows, shared, cols, m1, m2, m3, *alpha, *beta);         \
        memcpy(out, r, rows * cols * sizeof(CET));                                           \
        free(r);                                                                             \
    }

EXPORT_MUL(f32, float, float)
EXPORT_MUL(f64, double, double)
EXPORT_MUL(u32, uint32_t, uint32_t)
EXPORT_MUL(u64, uint64_t, uint64_t)
EXPORT_MUL(bf16_f32, __nv_bfloat16, float)
EXPORT_MUL(f16_f16, half, half)

extern "C" void ref_mmsd_u32_rr(uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                                uint32_t *elems, uint32_t *col_ind, uint32_t *row_off,
                                uint32_t *B, uint32_t *C) {
    Kuiper_Sparse_Matrix_smatrix__uint32_t a;
    a.nnz = nnz;
    a.elems = elems;
    a.col_ind = col_ind;
    a.row_off = row_off;
    Kuiper_Example_Sparse_MM__mmsd_u32_rr(rows, shared, cols, a, B, C);
}
