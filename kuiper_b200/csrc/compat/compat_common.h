// Bodies of the reference-named entry points: each one checks the reference's guards,
// forwards to the C ABI of libklas_b200.so on the legacy default stream, and returns
// only when the result is visible to every stream -- the blocking, void-returning
// contract of the reference's wrappers (dist/Klas_GEMM_SHMem.cu:50-72,
// include/kuiper.h:132-143).  Any failure prints the runtime's banner and ends the
// process, as the reference's MUST / KPR_GUARD do.
#pragma once

#include <kuiper.h>

#include "klas_b200.h"
#include "klas_signatures.h"

namespace klas_compat {

static inline void finish(int status, const char *entry, bool tensor_core) {
    if (status != KLAS_OK) {
        fprintf(stderr, "*** ABORTING ***\n %s failed: %s\n", entry, klas_b200_last_error());
        exit(1);
    }
    __MUST(cudaStreamSynchronize(0), "cudaStreamSynchronize", entry, __FILE__, __LINE__);
    // the kernels mirror a wait that gave up into host-visible memory: one load, no device round trip
    if (tensor_core && klas_b200_gemm_tc_status_peek() != 0 && klas_b200_gemm_tc_status(NULL) != KLAS_OK) {
        fprintf(stderr, "*** ABORTING ***\n %s failed: %s\n", entry, klas_b200_last_error());
        exit(1);
    }
}

}  // namespace klas_compat

// dtype code of an element-type label
#define KLAS_CODE_f32 KLAS_F32
#define KLAS_CODE_f64 KLAS_F64
#define KLAS_CODE_u32 KLAS_U32
#define KLAS_CODE_u64 KLAS_U64
#define KLAS_CODE_bf16 KLAS_BF16
#define KLAS_CODE_f16 KLAS_F16

#define KLAS_DIVIDES(TILE, V) KPR_GUARD((V) % (TILE) == 0U)

// Guards of the statically tiled families (m, k, n in the reference's order); tile 0: none.
#define KLAS_TILE_GUARDS_0
#define KLAS_TILE_GUARDS_16 KLAS_DIVIDES(16U, m); KLAS_DIVIDES(16U, k); KLAS_DIVIDES(16U, n);
#define KLAS_TILE_GUARDS_32 KLAS_DIVIDES(32U, m); KLAS_DIVIDES(32U, k); KLAS_DIVIDES(32U, n);
#define KLAS_TILE_GUARDS(TILE) KLAS_TILE_GUARDS_##TILE

#define KLAS_BODY_MATMUL(NAME, L, T, TILE)                                                        \
    KLAS_TILE_GUARDS(TILE)                                                                        \
    klas_compat::finish(klas_b200_gemm(KLAS_CODE_##L, KLAS_RRR, 1, m, n, k, NULL, NULL, gA, gB, gC, NULL), NAME, false);

#define KLAS_BODY_MATMUL_DYNTILE(NAME, L, T, TILE) \
    KPR_ASSERT(tile > 0U);                         \
    KLAS_BODY_MATMUL(NAME, L, T, 0)

#define KLAS_BODY_MATMUL_CCC(NAME, L, T, TILE) \
    klas_compat::finish(klas_b200_gemm(KLAS_CODE_##L, KLAS_CCC, 1, m, n, k, NULL, NULL, gA, gB, gC, NULL), NAME, false);

// Naive3: the reference's compensated sums (f32 accumulated in f64 here)
#define KLAS_BODY_COMPENSATED(NAME, L, T, TILE) \
    klas_compat::finish(klas_b200_gemm_compensated(KLAS_CODE_##L, KLAS_RRR, m, n, k, gA, gB, gC, NULL), NAME, false);
#define KLAS_BODY_COMPENSATED_CCC(NAME, L, T, TILE) \
    klas_compat::finish(klas_b200_gemm_compensated(KLAS_CODE_##L, KLAS_CCC, m, n, k, gA, gB, gC, NULL), NAME, false);

#define KLAS_BODY_GEMM(NAME, L, T, TILE)                                                          \
    KLAS_TILE_GUARDS(TILE)                                                                        \
    klas_compat::finish(klas_b200_gemm(KLAS_CODE_##L, KLAS_RRR, 1, m, n, k, &alpha, &beta, gA, gB, gC, NULL), NAME, false);

#define KLAS_BODY_GEMM_DYNTILE(NAME, L, T, TILE) \
    KPR_ASSERT(tile > 0U);                       \
    KLAS_BODY_GEMM(NAME, L, T, 0)

#define KLAS_BODY_BATCHED_MATMUL(NAME, L, T, TILE) \
    klas_compat::finish(klas_b200_gemm(KLAS_F32, KLAS_RRR, batch, m, n, k, NULL, NULL, a, b, c, NULL), NAME, false);

#define KLAS_BODY_BATCHED_GEMM(NAME, L, T, TILE) \
    klas_compat::finish(klas_b200_gemm(KLAS_F32, KLAS_RRR, batch, m, n, k, &alpha, &beta, a, b, c, NULL), NAME, false);

#define KLAS_BODY_BT2D(NAME, L, T, BM_, BN_, BK_)                                                 \
    KLAS_DIVIDES(BM_##U, m);                                                                      \
    KLAS_DIVIDES(BK_##U, k);                                                                      \
    KLAS_DIVIDES(BN_##U, n);                                                                      \
    klas_compat::finish(klas_b200_gemm(KLAS_CODE_##L, KLAS_RRR, 1, m, n, k, &alpha, &beta, gA, gB, gC, NULL), NAME, false);

#define KLAS_TC_GUARDS(GR, GS, GC) \
    KLAS_DIVIDES(GR##U, rows);     \
    KLAS_DIVIDES(GS##U, shared);   \
    KLAS_DIVIDES(GC##U, cols);

#define KLAS_BODY_TC2D(NAME, IN, OUT, BM_, BN_, BK_)                                              \
    KLAS_TC_GUARDS(BM_, BK_, BN_)                                                                 \
    klas_compat::finish(klas_b200_gemm_tc(IN, OUT, KLAS_B_ROW_MAJOR, 1, rows, shared, cols, gA, gB, NULL, gC, \
                                          1.0f, 0.0f, NULL, NULL), NAME, true);

#define KLAS_BODY_TC2D_TO(NAME, IN, OUT, BM_, BN_, BK_)                                           \
    KLAS_TC_GUARDS(BM_, BK_, BN_)                                                                 \
    klas_compat::finish(klas_b200_gemm_tc(IN, OUT, KLAS_B_ROW_MAJOR, 1, rows, shared, cols, gA, gB, gC, gD, \
                                          alpha, beta, NULL, NULL), NAME, true);

// C += A.B: the accumulator starts from C (dist/Klas_GEMM_TensorCore.cu:28-33).
#define KLAS_BODY_TC1D(NAME, L, TC, GR, GS, GC)                                                   \
    KLAS_TC_GUARDS(GR, GS, GC)                                                                    \
    klas_compat::finish(klas_b200_gemm_tc(KLAS_F16, KLAS_CODE_##L, KLAS_B_ROW_MAJOR, 1, rows, shared, cols, gA, \
                                          gB, gC, gC, 1.0f, 1.0f, NULL, NULL), NAME, true);

#define KLAS_BODY_SPMM(NAME, CODE, T, UNUSED)                                                     \
    klas_compat::finish(klas_b200_spmm(CODE, rows, shared, cols, gA.nnz, gA.elems, gA.col_ind, gA.row_off, \
                                       row_indices, gB, gC, NULL), NAME, false);

// ---- row-wise neighbours ------------------------------------------------------------------------
#define KLAS_IS_LOG_Softmax 0
#define KLAS_IS_LOG_LogSoftmax 1

namespace klas_compat {
// Device-pointer softmax entry points: scratch for the chunked vector path is allocated for the
// call, as the reference allocates its maxs/sums scalars (dist/Klas_Softmax.cu:210-213).
static inline void softmax_device(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a,
                                  const char *entry) {
    void *scratch = NULL;
    const size_t bytes = klas_b200_softmax_scratch_bytes(rows, cols);
    if (bytes) __MUST(cudaMalloc(&scratch, bytes), "cudaMalloc(scratch)", entry, __FILE__, __LINE__);
    finish(klas_b200_softmax(dtype, log_softmax, rows, cols, a, scratch, bytes, NULL), entry, false);
    if (scratch) __MUST(cudaFree(scratch), "cudaFree(scratch)", entry, __FILE__, __LINE__);
}
static inline void check(int status, const char *entry) {
    if (status != KLAS_OK) {
        fprintf(stderr, "*** ABORTING ***\n %s failed: %s\n", entry, klas_b200_last_error());
        exit(1);
    }
}
}  // namespace klas_compat

#define KLAS_BODY_SOFTMAX_DEV(NAME, U, L) \
    klas_compat::softmax_device(KLAS_CODE_##L, KLAS_IS_LOG_##U, 1, lena, a, NAME);
#define KLAS_BODY_SOFTMAX_HOST(NAME, U, L) \
    klas_compat::check(klas_b200_softmax_host(KLAS_CODE_##L, KLAS_IS_LOG_##U, 1, lena, a), NAME);
#define KLAS_BODY_ROWSOFTMAX(NAME, L) klas_compat::softmax_device(KLAS_CODE_##L, 0, m, n, a, NAME);
#define KLAS_BODY_ROWSCALE(NAME, L, COLMAJOR) \
    klas_compat::finish(klas_b200_rowscale(KLAS_CODE_##L, COLMAJOR, m, n, a, b, NULL), NAME, false);

#define KLAS_ENTRY(name, params, KIND, ...) \
    void name params { KLAS_BODY_##KIND(#name, __VA_ARGS__) }

// Reductions return their scalar to the host.
#define KLAS_RENTRY(ret, name, params, L, COUNT)                                                   \
    ret name params {                                                                              \
        ret result;                                                                                \
        klas_compat::check(klas_b200_reduce_sum_host(KLAS_CODE_##L, COUNT, a, &result), #name);    \
        return result;                                                                             \
    }
