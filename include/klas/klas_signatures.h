/*
 * klas_signatures.h -- the reference's Klas entry points as X-macro lists.
 *
 * Every list expands to a sequence of
 *     KLAS_ENTRY(name, (parameter list), KIND, extra...)
 * items.  The public headers (Klas_GEMM_*.h, Klas_SPMM.h) define KLAS_ENTRY to emit a
 * prototype; the compatibility sources define it to emit a definition whose body is
 * chosen by KIND.  Names, parameter order and parameter types are those of
 * FStarLang/kuiper dist/Klas_GEMM_*.h and dist/Klas_SPMM.h (C++ linkage, as there).
 */
#ifndef KLAS_SIGNATURES_H
#define KLAS_SIGNATURES_H 1

#include <stdint.h>

/* ---- element types of the CUDA-core families: X(FAMILY, label, C type) ------------------ */
#define KLAS_NUM_TYPES(X, F) X(F, f32, float) X(F, f64, double) X(F, u32, uint32_t) X(F, u64, uint64_t)

/* ---- SHMem / Tiled (dist/Klas_GEMM_SHMem.h:8-187, dist/Klas_GEMM_Tiled.h) ----------------
 * dynamic tile, tile32 and tile16; matmul (C = A.B) and gemm (C = beta*C + alpha*A.B). */
#define KLAS_MNK_ABC(T) uint32_t m, uint32_t n, uint32_t k, T *gA, T *gB, T *gC
#define KLAS_TILED_ENTRIES(F, L, T)                                                                     \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_rrr, (uint32_t tile, KLAS_MNK_ABC(T)), MATMUL_DYNTILE, L, T, 0)   \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_tile32_rrr, (KLAS_MNK_ABC(T)), MATMUL, L, T, 0)          \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_tile16_rrr, (KLAS_MNK_ABC(T)), MATMUL, L, T, 0)          \
    KLAS_ENTRY(Klas_GEMM_##F##_g_gemm_##L##_rrr, (uint32_t tile, T alpha, T beta, KLAS_MNK_ABC(T)), GEMM_DYNTILE, L, T, 0) \
    KLAS_ENTRY(Klas_GEMM_##F##_g_gemm_##L##_tile32_rrr, (T alpha, T beta, KLAS_MNK_ABC(T)), GEMM, L, T, 0) \
    KLAS_ENTRY(Klas_GEMM_##F##_g_gemm_##L##_tile16_rrr, (T alpha, T beta, KLAS_MNK_ABC(T)), GEMM, L, T, 0)

/* ---- BlockTiling1D (dist/Klas_GEMM_BlockTiling1D.h:8-131): static tiles, guarded ---------- */
#define KLAS_BT1D_ENTRIES(F, L, T)                                                                      \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_tile32_rrr, (KLAS_MNK_ABC(T)), MATMUL, L, T, 32)         \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_tile16_rrr, (KLAS_MNK_ABC(T)), MATMUL, L, T, 16)         \
    KLAS_ENTRY(Klas_GEMM_##F##_g_gemm_##L##_tile32_rrr, (T alpha, T beta, KLAS_MNK_ABC(T)), GEMM, L, T, 32) \
    KLAS_ENTRY(Klas_GEMM_##F##_g_gemm_##L##_tile16_rrr, (T alpha, T beta, KLAS_MNK_ABC(T)), GEMM, L, T, 16)

/* ---- Naive1 / Naive2 (dist/Klas_GEMM_Naive1.h:8-65): any m, n, k; rrr and ccc; batched f32 - */
#define KLAS_NAIVE_ENTRIES(F, L, T)                                                                     \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_rrr, (KLAS_MNK_ABC(T)), MATMUL, L, T, 0)                 \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_ccc, (KLAS_MNK_ABC(T)), MATMUL_CCC, L, T, 0)
#define KLAS_NAIVE_BATCHED_ENTRIES(F)                                                                   \
    KLAS_ENTRY(Klas_GEMM_##F##_batched_matmul_f32,                                                      \
               (uint32_t batch, uint32_t m, uint32_t n, uint32_t k, float *a, float *b, float *c),     \
               BATCHED_MATMUL, f32, float, 0)                                                           \
    KLAS_ENTRY(Klas_GEMM_##F##_batched_gemm_f32,                                                        \
               (float alpha, float beta, uint32_t batch, uint32_t m, uint32_t n, uint32_t k, float *a, \
                float *b, float *c),                                                                    \
               BATCHED_GEMM, f32, float, 0)

/* ---- Naive3 (dist/Klas_GEMM_Naive3.h:8-41): compensated sums; bf16, f32, f64 --------------- */
#define KLAS_NAIVE3_TYPES(X, F) X(F, bf16, __nv_bfloat16) X(F, f32, float) X(F, f64, double)
#define KLAS_NAIVE3_ENTRIES(F, L, T)                                                                    \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_rrr, (KLAS_MNK_ABC(T)), COMPENSATED, L, T, 0)            \
    KLAS_ENTRY(Klas_GEMM_##F##_g_matmul_##L##_ccc, (KLAS_MNK_ABC(T)), COMPENSATED_CCC, L, T, 0)

/* ---- BlockTiling2D (dist/Klas_GEMM_BlockTiling2D.h:8-1376): f32 and bf16 per tile instance - */
#define KLAS_BT2D_INSTANCE(bm, bn, bk, tm, tn)                                                          \
    KLAS_ENTRY(Klas_GEMM_BlockTiling2D_g_gemm_f32_##bm##x##bn##x##bk##_##tm##x##tn,                     \
               (float alpha, float beta, KLAS_MNK_ABC(float)), BT2D, f32, float, bm, bn, bk)            \
    KLAS_ENTRY(Klas_GEMM_BlockTiling2D_g_gemm_bf16_##bm##x##bn##x##bk##_##tm##x##tn,                    \
               (__nv_bfloat16 alpha, __nv_bfloat16 beta, KLAS_MNK_ABC(__nv_bfloat16)), BT2D, bf16,      \
               __nv_bfloat16, bm, bn, bk)

/* ---- TensorCore2D (dist/Klas_GEMM_TensorCore2D.h:8-1220): f16->f16 and bf16->f32 ----------- */
#define KLAS_RSC_ABC(TA, TC) uint32_t rows, uint32_t shared, uint32_t cols, TA *gA, TA *gB, TC *gC
#define KLAS_TC2D_PLAIN_INSTANCE(bm, bn, bk, wm, wn)                                                    \
    KLAS_ENTRY(Klas_GEMM_TensorCore2D_g_gemm_f16_f16_##bm##x##bn##x##bk##_16x16x16_##wm##x##wn,         \
               (KLAS_RSC_ABC(half, half)), TC2D, KLAS_F16, KLAS_F16, bm, bn, bk)                        \
    KLAS_ENTRY(Klas_GEMM_TensorCore2D_g_gemm_bf16_f32_##bm##x##bn##x##bk##_16x16x16_##wm##x##wn,        \
               (KLAS_RSC_ABC(__nv_bfloat16, float)), TC2D, KLAS_BF16, KLAS_F32, bm, bn, bk)

/* ---- TensorCore2D_To (dist/Klas_GEMM_TensorCore2D_To.h): D = bf16(beta*C + alpha*A.B) ------ */
#define KLAS_TC2D_TO_INSTANCE(bm, bn, bk, wm, wn)                                                       \
    KLAS_ENTRY(Klas_GEMM_TensorCore2D_To_g_gemm_bf16_f32_bf16_##bm##x##bn##x##bk##_16x16x16_##wm##x##wn, \
               (uint32_t rows, uint32_t shared, uint32_t cols, __nv_bfloat16 *gA, __nv_bfloat16 *gB,    \
                __nv_bfloat16 *gC, __nv_bfloat16 *gD, float alpha, float beta),                         \
               TC2D_TO, KLAS_BF16, KLAS_BF16, bm, bn, bk)

/* ---- TensorCore (dist/Klas_GEMM_TensorCore.h:8-85): C += A.B, eleven names -----------------
 * KLAS_TC1D(accumulator label, accumulator type, name tail, rows guard, shared guard, cols guard).
 * The guards are those of dist/Klas_GEMM_TensorCore.cu (e.g. :99-102, :424-427, :531-535): they
 * follow the real block tile, which for 8x32x16_8x32x16 is 32x32x32, not the name. */
#define KLAS_TC1D_ENTRIES(X)                        \
    X(f16, half, 64x64x16_16x16x16, 64, 16, 64)     \
    X(f16, half, 32x32x32_32x8x16, 32, 32, 32)      \
    X(f16, half, 32x32x32_8x32x16, 32, 32, 32)      \
    X(f16, half, 32x8x16_32x8x16, 32, 16, 8)        \
    X(f16, half, 8x32x16_8x32x16, 32, 32, 32)       \
    X(f16, half, 64x64x64_16x16x16, 64, 64, 64)     \
    X(f16, half, 64x64x64_32x8x16, 64, 64, 64)      \
    X(f16, half, 64x64x64_8x32x16, 64, 64, 64)      \
    X(f16, half, 32x32x32_16x16x16, 32, 32, 32)     \
    X(f16, half, 16x16x16_16x16x16, 16, 16, 16)     \
    X(f32, float, 32x32x32_16x16x16, 32, 32, 32)
#define KLAS_TC1D_ENTRY(L, TC, TAIL, GR, GS, GC)                                                        \
    KLAS_ENTRY(Klas_GEMM_TensorCore_g_gemm_f16_##L##_##TAIL, (KLAS_RSC_ABC(half, TC)), TC1D, L, TC, GR, GS, GC)

/* ---- SpMM (dist/Klas_SPMM.h:7-673) ----------------------------------------------------------- */
#define KLAS_SPMM_PARAMS(ST, T) \
    uint32_t rows, uint32_t shared, uint32_t cols, ST gA, uint32_t *row_indices, T *gB, T *gC
#define KLAS_SPMM_INSTANCE(kk, xx, ww)                                                                  \
    KLAS_ENTRY(Klas_SPMM_g_spmm_f32_##kk##x##xx##x##ww,                                                 \
               (KLAS_SPMM_PARAMS(Kuiper_Sparse_Matrix_smatrix__float, float)), SPMM, KLAS_F32, float, 0)
#define KLAS_SPMM_FIXED_ENTRIES                                                                         \
    KLAS_ENTRY(Klas_SPMM_spmm_u32, (KLAS_SPMM_PARAMS(Kuiper_Sparse_Matrix_smatrix__uint32_t, uint32_t)), \
               SPMM, KLAS_U32, uint32_t, 0)                                                             \
    KLAS_ENTRY(Klas_SPMM_spmm_f32, (KLAS_SPMM_PARAMS(Kuiper_Sparse_Matrix_smatrix__float, float)), SPMM, \
               KLAS_F32, float, 0)

/* ---- Softmax / LogSoftmax (dist/Klas_Softmax.h, dist/Klas_LogSoftmax.h): in-place vector ------
 * softmax; _gpu names take a device pointer, the others a host pointer; _n names carry a
 * thread-count hint.  X(unit, function stem, label, C type). */
#define KLAS_SOFTMAX_TYPES(X, U, F) X(U, F, f16, half) X(U, F, f32, float) X(U, F, f64, double)
#define KLAS_SOFTMAX_ENTRIES(U, F, L, T)                                                                \
    KLAS_ENTRY(Klas_##U##_##F##_gpu_n_##L, (uint32_t nth, uint32_t lena, T *a), SOFTMAX_DEV, U, L)      \
    KLAS_ENTRY(Klas_##U##_##F##_gpu_##L, (uint32_t lena, T *a), SOFTMAX_DEV, U, L)                      \
    KLAS_ENTRY(Klas_##U##_##F##_n_##L, (uint32_t nth, uint32_t lena, T *a), SOFTMAX_HOST, U, L)         \
    KLAS_ENTRY(Klas_##U##_##F##_##L, (uint32_t lena, T *a), SOFTMAX_HOST, U, L)

/* ---- RowSoftmax (dist/Klas_RowSoftmax.h:7-11): rows of a row-major m x n device matrix ------- */
#define KLAS_ROWSOFTMAX_ENTRIES                                                                          \
    KLAS_ENTRY(Klas_RowSoftmax_row_softmax_rm_f32, (uint32_t m, uint32_t n, uint32_t nth, float *a), ROWSOFTMAX, f32) \
    KLAS_ENTRY(Klas_RowSoftmax_row_softmax_rm_f64, (uint32_t m, uint32_t n, uint32_t nth, double *a), ROWSOFTMAX, f64)

/* ---- RowScale (dist/Klas_RowScale.h:7-23): b[r][c] = a[r] * b[r][c] --------------------------- */
#define KLAS_ROWSCALE_TYPES(X) X(f16, half) X(f32, float) X(f64, double)
#define KLAS_ROWSCALE_ENTRIES(L, T)                                                                     \
    KLAS_ENTRY(Klas_RowScale_rowscale_##L##_rowmajor, (uint32_t m, uint32_t n, T *a, T *b), ROWSCALE, L, 0) \
    KLAS_ENTRY(Klas_RowScale_rowscale_##L##_colmajor, (uint32_t m, uint32_t n, T *a, T *b), ROWSCALE, L, 1)

/* ---- HReduce / AtomicReduce (dist/Klas_HReduce.h:7-20, dist/Klas_AtomicReduce.h:7-13) ---------
 * return the sum of a device vector to the host: KLAS_RENTRY(return type, name, params, label). */
#define KLAS_HREDUCE_ENTRIES                                                                            \
    KLAS_RENTRY(half, Klas_HReduce_reduce_f16_plus, (uint32_t nth, uint32_t lena, half *a), f16, lena)  \
    KLAS_RENTRY(float, Klas_HReduce_reduce_f32_plus, (uint32_t nth, uint32_t lena, float *a), f32, lena) \
    KLAS_RENTRY(double, Klas_HReduce_reduce_f64_plus, (uint32_t nth, uint32_t lena, double *a), f64, lena) \
    KLAS_RENTRY(uint32_t, Klas_HReduce_reduce_u32_plus, (uint32_t nth, uint32_t lena, uint32_t *a), u32, lena) \
    KLAS_RENTRY(uint64_t, Klas_HReduce_reduce_u64_plus, (uint32_t nth, uint32_t lena, uint64_t *a), u64, lena)
#define KLAS_ATOMICREDUCE_ENTRIES                                                                       \
    KLAS_RENTRY(uint32_t, Klas_AtomicReduce_reduce_u32, (uint32_t n, uint32_t *a), u32, n)              \
    KLAS_RENTRY(uint64_t, Klas_AtomicReduce_reduce_u64, (uint32_t n, uint64_t *a), u64, n)              \
    KLAS_RENTRY(float, Klas_AtomicReduce_reduce_f32, (uint32_t n, float *a), f32, n)                    \
    KLAS_RENTRY(double, Klas_AtomicReduce_reduce_f64, (uint32_t n, double *a), f64, n)

#endif /* KLAS_SIGNATURES_H */
