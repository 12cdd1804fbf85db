// Internal helpers shared by the translation units of libklas_b200.so.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "klas_b200.h"

namespace klas {

// Stores a printf-style message for klas_b200_last_error() of this thread and
// returns `code`, so that error paths read `return fail(KLAS_ERR_X, "...")`.
int fail(int code, const char *fmt, ...);
void clear_error();

inline int check_cuda(cudaError_t rc, const char *what) {
    if (rc == cudaSuccess) return KLAS_OK;
    return fail(KLAS_ERR_CUDA, "%s: %s", what, cudaGetErrorString(rc));
}

#define KLAS_TRY_CUDA(expr)                                         \
    do {                                                            \
        int _rc = ::klas::check_cuda((expr), #expr);                \
        if (_rc != KLAS_OK) return _rc;                             \
    } while (0)

inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case KLAS_F32: case KLAS_U32: return 4;
        case KLAS_F64: case KLAS_U64: return 8;
        case KLAS_BF16: case KLAS_F16: return 2;
        default: return 0;
    }
}

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int l2_bytes = 0;
    int max_smem_optin = 0;
    int cc_major = 0, cc_minor = 0;
};

// Properties of the current device, cached per device.
int device_info(DeviceInfo *out);

// Current value of a tuning knob (klas_knob of klas_b200.h); set by klas_b200_debug_set.
int debug_knob(int knob);

// Grow-only per-device scratch used by the *_host entry points.
int workspace_reserve(int slot, size_t bytes, void **ptr);
int workspace_release();

// Kernel launchers (one per translation unit).
int launch_gemm_simt(int dtype, int layout, uint32_t batch, uint64_t m, uint64_t n, uint64_t k,
                     const void *alpha, const void *beta, const void *A, const void *B, void *C,
                     cudaStream_t stream);

// C = A.B with a sum that keeps what a compensated (Kahan) sum in the element type keeps: f32 is
// accumulated in f64; the other types take the plain kernel.
int launch_gemm_simt_compensated(int dtype, int layout, uint64_t m, uint64_t n, uint64_t k, const void *A, const void *B,
                                 void *C, cudaStream_t stream);

int launch_gemm_dmma(uint32_t batch, uint64_t m, uint64_t n, uint64_t k, const double *alpha, const double *beta,
                     const void *A, const void *B, void *C, cudaStream_t stream);

int launch_gemm_simt_strided(int dtype, uint32_t batch, uint64_t m, uint64_t n, uint64_t k, const void *alpha,
                             const void *beta, const void *A, uint64_t lda, uint64_t stride_a, const void *B,
                             uint64_t ldb, uint64_t stride_b, void *C, uint64_t ldc, uint64_t stride_c, int map_a,
                             int map_b, int comb, cudaStream_t stream);

int launch_gemm_umma(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                     uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                     void *D, float alpha, float beta, int *status_word, cudaStream_t stream);

int launch_gemm_umma_fused(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                           uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                           void *D, float alpha, float beta, int map_a, int map_b, int comb,
                           int *status_word, cudaStream_t stream);

// Row and page strides (elements) of a tensor-core GEMM; 0 = contiguous.  C shares D's.
struct TcStrides {
    uint64_t lda, stride_a, ldb, stride_b, ldd, stride_d;
};
int launch_gemm_umma_strided(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                             uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                             void *D, const TcStrides &st, float alpha, float beta, int map_a, int map_b, int comb,
                             int *status_word, cudaStream_t stream);

int launch_spmm(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                const uint32_t *row_indices, const void *B, void *C, cudaStream_t stream);

// The gathers of the SpMM kernel alone (no values, products or stores): the rate ceiling it is measured against.
int launch_spmm_gather_probe(uint32_t shared, uint32_t cols, uint32_t nnz, const uint32_t *col_ind, const float *B,
                             cudaStream_t stream);

int launch_sdpa_fused(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e, const void *Q, const void *K,
                      const void *V, void *out, float scale, cudaStream_t stream);

int launch_minplus_u16(uint32_t m, uint32_t n, uint32_t k, const uint16_t *A, const uint16_t *B, uint16_t *C,
                       cudaStream_t stream);

int launch_csr_count(int dtype, uint32_t rows, uint32_t cols, const void *dense, uint32_t *row_off, cudaStream_t stream);
int launch_csr_fill(int dtype, uint32_t rows, uint32_t cols, const void *dense, const uint32_t *row_off, void *elems,
                    uint32_t *col_ind, cudaStream_t stream);
size_t csr_row_order_scratch_bytes(uint32_t rows);
int launch_csr_row_order(uint32_t rows, const uint32_t *row_off, uint32_t *row_indices, void *scratch,
                         size_t scratch_bytes, cudaStream_t stream);

size_t softmax_scratch_bytes(uint64_t rows, uint64_t cols);
size_t reduce_scratch_bytes(uint64_t n);
int launch_softmax(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a, void *scratch,
                   size_t scratch_bytes, cudaStream_t stream);
int launch_softmax_rows(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a, cudaStream_t stream);
int launch_rowscale(int dtype, int col_major, uint64_t m, uint64_t n, const void *scale, void *b,
                    cudaStream_t stream);
int launch_reduce_sum(int dtype, uint64_t n, const void *a, void *out, void *scratch, size_t scratch_bytes,
                      cudaStream_t stream);

}  // namespace klas
