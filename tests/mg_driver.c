/*
 * C consumer of the multi-GPU entry points of include/klas_b200.h (what a C or C++ caller of the
 * reference-style library would write; no Python, no torch).  Usage: mg_driver <devices>
 *
 * On `devices` GPUs (the first ones visible) it runs, sharded, a bf16 -> f32 tensor-core GEMM
 * (gathered on every device), a wrapping u64 GEMM over unequal row blocks (gathered on the first
 * device) and a CSR x dense product over nnz-balanced row ranges (gathered on every device), and
 * compares every assembled result bit for bit with the same product computed on one GPU by the
 * single-GPU entry points.  Prints one line per check and "OK", exit code 0, when all agree.
 */
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime.h>

#include "klas_b200.h"

#define MAXDEV 16

#define CUDA_OK(e)                                                                         \
    do {                                                                                   \
        cudaError_t rc_ = (e);                                                             \
        if (rc_ != cudaSuccess) {                                                          \
            fprintf(stderr, "%s failed: %s\n", #e, cudaGetErrorString(rc_));               \
            exit(2);                                                                       \
        }                                                                                  \
    } while (0)
#define KLAS_OK_(e)                                                                        \
    do {                                                                                   \
        int rc_ = (e);                                                                     \
        if (rc_ != KLAS_OK) {                                                              \
            fprintf(stderr, "%s failed (%d): %s\n", #e, rc_, klas_b200_last_error());      \
            exit(3);                                                                       \
        }                                                                                  \
    } while (0)

static uint64_t rng_state = 0x9e3779b97f4a7c15ull;
static uint64_t rng(void) {   /* splitmix64 */
    uint64_t z = (rng_state += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

static uint16_t bf16_of_small_int(int v) {   /* exact: |v| < 256 */
    float f = (float)v;
    uint32_t bits;
    memcpy(&bits, &f, 4);
    return (uint16_t)(bits >> 16);
}

static void *dev_copy(int device, const void *host, size_t bytes) {
    void *p = NULL;
    CUDA_OK(cudaSetDevice(device));
    CUDA_OK(cudaMalloc(&p, bytes ? bytes : 16));
    if (host && bytes) CUDA_OK(cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice));
    return p;
}

static int same_on_device(int device, const void *dptr, const void *want, size_t bytes, const char *what) {
    void *got = malloc(bytes ? bytes : 1);
    CUDA_OK(cudaSetDevice(device));
    CUDA_OK(cudaMemcpy(got, dptr, bytes, cudaMemcpyDeviceToHost));
    const int same = memcmp(got, want, bytes) == 0;
    printf("%s on device %d: %s\n", what, device, same ? "identical" : "DIFFERENT");
    free(got);
    return same;
}

int main(int argc, char **argv) {
    int n = argc > 1 ? atoi(argv[1]) : 1, visible = 0, ok = 1;
    CUDA_OK(cudaGetDeviceCount(&visible));
    if (n < 1 || n > visible || n > MAXDEV) {
        fprintf(stderr, "asked for %d devices, %d visible\n", n, visible);
        return 4;
    }
    int devices[MAXDEV];
    for (int i = 0; i < n; ++i) devices[i] = i;
    klas_mg_context *ctx = NULL;
    KLAS_OK_(klas_b200_mg_create(devices, n, &ctx));
    if (klas_b200_mg_count(ctx) != n) return 5;

    /* ---- bf16 x bf16 -> f32, column-major B, rows in tile-aligned blocks, gathered everywhere ---- */
    {
        const uint64_t M = 256ull * (uint64_t)(2 * n + 1), N = 384, K = 320;   /* an odd number of tiles: unequal blocks */
        uint16_t *A = malloc(M * K * 2), *Bt = malloc(N * K * 2);
        for (uint64_t i = 0; i < M * K; ++i) A[i] = bf16_of_small_int((int)(rng() % 7) - 3);
        for (uint64_t i = 0; i < N * K; ++i) Bt[i] = bf16_of_small_int((int)(rng() % 7) - 3);
        float *want = malloc(M * N * 4);
        void *dA0 = dev_copy(0, A, M * K * 2), *dB0 = dev_copy(0, Bt, N * K * 2), *dD0 = dev_copy(0, NULL, M * N * 4);
        KLAS_OK_(klas_b200_gemm_tc(KLAS_BF16, KLAS_F32, KLAS_B_COL_MAJOR, 1, M, K, N, dA0, dB0, NULL, dD0, 1.f, 0.f, NULL, NULL));
        CUDA_OK(cudaDeviceSynchronize());
        KLAS_OK_(klas_b200_gemm_tc_status(NULL));
        CUDA_OK(cudaMemcpy(want, dD0, M * N * 4, cudaMemcpyDeviceToHost));

        uint64_t bounds[MAXDEV + 1];
        KLAS_OK_(klas_b200_mg_row_blocks(M, n, 256, bounds));
        const void *As[MAXDEV], *Bs[MAXDEV];
        void *Ds[MAXDEV], *full[MAXDEV], *Bbuf[MAXDEV];
        for (int i = 0; i < n; ++i) {
            As[i] = dev_copy(devices[i], A + bounds[i] * K, (bounds[i + 1] - bounds[i]) * K * 2);
            Bbuf[i] = dev_copy(devices[i], i == 0 ? Bt : NULL, N * K * 2);   /* only the first device has B ... */
            Ds[i] = dev_copy(devices[i], NULL, (bounds[i + 1] - bounds[i]) * N * 4);
            full[i] = dev_copy(devices[i], NULL, M * N * 4);
        }
        KLAS_OK_(klas_b200_mg_broadcast(ctx, Bbuf, N * K * 2, 0));           /* ... until it is replicated */
        for (int i = 0; i < n; ++i) Bs[i] = Bbuf[i];
        KLAS_OK_(klas_b200_mg_gemm_tc(ctx, KLAS_BF16, KLAS_F32, KLAS_B_COL_MAJOR, bounds, K, N, As, Bs, Ds, KLAS_MG_GATHER_ALL, full));
        KLAS_OK_(klas_b200_mg_synchronize(ctx));
        for (int i = 0; i < n; ++i) {
            ok &= same_on_device(devices[i], full[i], want, M * N * 4, "bf16 GEMM, all rows gathered");
            ok &= same_on_device(devices[i], Ds[i], want + bounds[i] * N, (bounds[i + 1] - bounds[i]) * N * 4, "bf16 GEMM, own block");
        }
        free(A); free(Bt); free(want);
    }

    /* ---- wrapping u64 GEMM, deliberately unequal blocks, gathered on the first device ---- */
    {
        const uint64_t M = 100ull * (uint64_t)n + 37, N = 72, K = 90;
        uint64_t *A = malloc(M * K * 8), *B = malloc(K * N * 8), *want = malloc(M * N * 8);
        for (uint64_t i = 0; i < M * K; ++i) A[i] = rng();
        for (uint64_t i = 0; i < K * N; ++i) B[i] = rng();
        void *dA0 = dev_copy(0, A, M * K * 8), *dB0 = dev_copy(0, B, K * N * 8), *dC0 = dev_copy(0, NULL, M * N * 8);
        KLAS_OK_(klas_b200_gemm(KLAS_U64, KLAS_RRR, 1, M, N, K, NULL, NULL, dA0, dB0, dC0, NULL));
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(want, dC0, M * N * 8, cudaMemcpyDeviceToHost));
        uint64_t bounds[MAXDEV + 1];
        KLAS_OK_(klas_b200_mg_row_blocks(M, n, 1, bounds));
        if (n > 1) { bounds[1] = 5; }   /* a very short first block */
        const void *As[MAXDEV], *Bs[MAXDEV];
        void *Cs[MAXDEV], *full[MAXDEV] = {0};
        for (int i = 0; i < n; ++i) {
            As[i] = dev_copy(devices[i], A + bounds[i] * K, (bounds[i + 1] - bounds[i]) * K * 8);
            Bs[i] = dev_copy(devices[i], B, K * N * 8);
            Cs[i] = dev_copy(devices[i], NULL, (bounds[i + 1] - bounds[i]) * N * 8);
        }
        full[0] = dev_copy(devices[0], NULL, M * N * 8);
        KLAS_OK_(klas_b200_mg_gemm(ctx, KLAS_U64, bounds, N, K, As, Bs, Cs, KLAS_MG_GATHER_FIRST, full));
        KLAS_OK_(klas_b200_mg_synchronize(ctx));
        ok &= same_on_device(devices[0], full[0], want, M * N * 8, "u64 GEMM, gathered on the first device");
        free(A); free(B); free(want);
    }

    /* ---- CSR x dense over nnz-balanced row ranges ---- */
    {
        const uint32_t rows = 3000, shared = 2048, cols = 128;
        uint32_t *row_off = malloc((rows + 1) * 4);
        uint32_t cap = rows * 64, nnz = 0;
        uint32_t *col = malloc(cap * 4);
        float *val = malloc(cap * 4);
        row_off[0] = 0;
        for (uint32_t r = 0; r < rows; ++r) {
            const uint32_t len = (uint32_t)(rng() % 40) * (r % 7 == 0 ? 0u : 1u);   /* some empty rows */
            uint32_t c = (uint32_t)(rng() % 8);
            for (uint32_t j = 0; j < len && c < shared; ++j) {
                col[nnz] = c;
                val[nnz] = (float)((int)(rng() % 17) - 8) * 0.125f;
                ++nnz;
                c += 1 + (uint32_t)(rng() % 60);
            }
            row_off[r + 1] = nnz;
        }
        float *B = malloc((size_t)shared * cols * 4), *want = malloc((size_t)rows * cols * 4);
        for (size_t i = 0; i < (size_t)shared * cols; ++i) B[i] = (float)((int)(rng() % 33) - 16) * 0.0625f;
        void *dE = dev_copy(0, val, nnz * 4), *dCi = dev_copy(0, col, nnz * 4), *dRo = dev_copy(0, row_off, (rows + 1) * 4);
        void *dB0 = dev_copy(0, B, (size_t)shared * cols * 4), *dC0 = dev_copy(0, NULL, (size_t)rows * cols * 4);
        KLAS_OK_(klas_b200_spmm(KLAS_F32, rows, shared, cols, nnz, dE, dCi, dRo, NULL, dB0, dC0, NULL));
        CUDA_OK(cudaDeviceSynchronize());
        CUDA_OK(cudaMemcpy(want, dC0, (size_t)rows * cols * 4, cudaMemcpyDeviceToHost));
        uint32_t bounds[MAXDEV + 1], shard_nnz[MAXDEV];
        KLAS_OK_(klas_b200_mg_csr_row_ranges(row_off, rows, n, 1, bounds));
        const void *Es[MAXDEV], *Bs[MAXDEV];
        const uint32_t *Cis[MAXDEV], *Ros[MAXDEV];
        void *Cs[MAXDEV], *full[MAXDEV];
        for (int i = 0; i < n; ++i) {
            const uint32_t r0 = bounds[i], r1 = bounds[i + 1], p0 = row_off[r0], p1 = row_off[r1];
            uint32_t *rebased = malloc((r1 - r0 + 1) * 4);
            for (uint32_t r = r0; r <= r1; ++r) rebased[r - r0] = row_off[r] - p0;
            shard_nnz[i] = p1 - p0;
            Es[i] = dev_copy(devices[i], val + p0, (p1 - p0) * 4);
            Cis[i] = dev_copy(devices[i], col + p0, (p1 - p0) * 4);
            Ros[i] = dev_copy(devices[i], rebased, (r1 - r0 + 1) * 4);
            Bs[i] = dev_copy(devices[i], B, (size_t)shared * cols * 4);
            Cs[i] = dev_copy(devices[i], NULL, (size_t)(r1 - r0) * cols * 4);
            full[i] = dev_copy(devices[i], NULL, (size_t)rows * cols * 4);
            free(rebased);
        }
        KLAS_OK_(klas_b200_mg_spmm(ctx, KLAS_F32, bounds, shared, cols, shard_nnz, Es, Cis, Ros, Bs, Cs, KLAS_MG_GATHER_ALL, full));
        KLAS_OK_(klas_b200_mg_synchronize(ctx));
        for (int i = 0; i < n; ++i) ok &= same_on_device(devices[i], full[i], want, (size_t)rows * cols * 4, "SpMM, all rows gathered");
        free(row_off); free(col); free(val); free(B); free(want);
    }

    KLAS_OK_(klas_b200_mg_destroy(ctx));
    puts(ok ? "OK" : "FAILED");
    return ok ? 0 : 1;
}
