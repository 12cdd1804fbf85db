/*
 * kuiper.h -- runtime shim for code written against the Kuiper C/CUDA runtime header
 * (FStarLang/kuiper include/kuiper.h).  The Klas headers and the reference's test
 * drivers include <kuiper.h>; putting this directory on the include path gives them
 * the same macros and helper names, implemented over the CUDA runtime:
 *
 *   MUST(e), __MUST(...)        CUDA call must succeed, else report and exit(1)   (kuiper.h:21-32,83)
 *   KPR_GUARD(c), KPR_ASSERT(c) precondition checks that abort()                  (kuiper.h:57-81)
 *   KPR_KCALL(...)              kernel launch that is skipped for an empty grid   (kuiper.h:38-46)
 *   KPR_SHMEM(), KPR_SHMEM_AT   dynamic shared memory carving                     (kuiper.h:48-55)
 *   KPR_GPU_ALLOC, KPR_FRESH_STREAM, KPR_SHMEM_FITS, KRML_* host macros           (kuiper.h:85-143)
 *   INFO()                      prints the sizes of the integer types                 (kuiper.h:111-123)
 * and, as the reference's header does (kuiper.h:12-19), pulls in kuiper/atomics.h,
 * kuiper/vectorops.h, kuiper/math.h and -- unless KUIPER_CFG_TENSORCORES is defined as 0 --
 * kuiper/tensorcores.h from the directory beside it.
 */
#ifndef KUIPER_H
#define KUIPER_H 1

#include <assert.h>
#include <float.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "kuiper/atomics.h"
#include "kuiper/vectorops.h"
#include "kuiper/math.h"
#if (!defined(KUIPER_CFG_TENSORCORES) || KUIPER_CFG_TENSORCORES)
#include "kuiper/tensorcores.h"
#endif

/* Prints the standard failure banner and terminates; `how` selects exit(1) or abort(). */
static inline void klas_shim_fail(const char *kind, const char *what, const char *func,
                                  const char *file, int line, const char *detail, int use_abort)
{
    fprintf(stderr, "*** ABORTING ***\n %s: %s\n In function %s\n At %s:%d\n", kind, what, func, file, line);
    if (detail) fprintf(stderr, " CUDA error: %s\n", detail);
    if (use_abort) abort();
    exit(1);
}

static inline void __MUST(cudaError_t rc, const char *str, const char *func, const char *fname, int line)
{
    if (rc != cudaSuccess)
        klas_shim_fail("This call failed", str, func, fname, line, cudaGetErrorString(rc), 0);
}

#define MUST(e) __MUST((e), #e, __func__, __FILE__, __LINE__)

#define KPR_GUARD(b) \
    ((b) ? (void)0 : klas_shim_fail("Guard failed", #b, __func__, __FILE__, __LINE__, NULL, 1))

#ifndef NDEBUG
#define KPR_ASSERT(b) \
    ((b) ? (void)0 : klas_shim_fail("Assertion failed", #b, __func__, __FILE__, __LINE__, NULL, 1))
#else
#define KPR_ASSERT(b) ((void)0)
#endif

/* A launch with an empty grid or block is not an error: it does nothing. */
#define KPR_KCALL(kernel, nblk, nthr, smem_bytes, stream, ...)                                \
    do {                                                                                      \
        const auto klas_shim_blocks = (nblk);                                                 \
        const auto klas_shim_threads = (nthr);                                                \
        if (klas_shim_blocks > 0 && klas_shim_threads > 0) {                                  \
            kernel<<<klas_shim_blocks, klas_shim_threads, (smem_bytes), stream>>>(__VA_ARGS__); \
            __MUST(cudaGetLastError(), "kcall", __func__, __FILE__, __LINE__);                \
        }                                                                                     \
    } while (0)

#define KPR_SHMEM()                                  \
    ({                                               \
        extern __shared__ char klas_shim_dynsmem[];  \
        (char *)klas_shim_dynsmem;                   \
    })
#define KPR_SHMEM_AT(off) ((void *)(KPR_SHMEM() + (off)))
#define KPR_SHMEM_FITS(e) KPR_ASSERT((e) <= 101376) /* 99 KiB */

#define KRML_HOST_MALLOC malloc
#define KRML_HOST_CALLOC calloc
#define KRML_HOST_FREE free
#define KRML_HOST_IGNORE(x) (void)(x)
#define KRML_MAYBE_UNUSED_VAR(x) KRML_HOST_IGNORE(x)
#define KRML_HOST_EPRINTF(s, ...) fprintf(stderr, s, __VA_ARGS__)
#define KRML_HOST_EXIT(rc) exit(rc)
#define KRML_CLITERAL(a) (a)
#define KRML_CHECK_SIZE(size_elt, sz) assert(((size_t)(sz)) <= ((size_t)(SIZE_MAX / (size_elt))))

static inline void *klas_shim_gpu_alloc(size_t elt, size_t len, const char *what, const char *func,
                                        const char *file, int line)
{
    void *p = NULL;
    KRML_CHECK_SIZE(elt, len);
    __MUST(cudaMalloc(&p, elt * len), what, func, file, line);
    return p;
}
#define KPR_GPU_ALLOC(sz, len) \
    klas_shim_gpu_alloc((sz), (len), "KPR_GPU_ALLOC(" #sz ", " #len ")", __func__, __FILE__, __LINE__)

/* A new *blocking* stream: work on it is ordered after earlier legacy-default-stream work
 * such as a cudaMemcpy from the host. */
static inline cudaStream_t KPR_FRESH_STREAM(void)
{
    cudaStream_t s;
    __MUST(cudaStreamCreate(&s), "cudaStreamCreate", __func__, __FILE__, __LINE__);
    return s;
}

/* Sizes of the integer types on this host, one per line. */
static inline void INFO(void)
{
#define KLAS_SHIM_SIZE(T) printf("sizeof(" #T ") = %zu\n", sizeof(T))
    KLAS_SHIM_SIZE(short);
    KLAS_SHIM_SIZE(int);
    KLAS_SHIM_SIZE(long);
    KLAS_SHIM_SIZE(long long);
    KLAS_SHIM_SIZE(unsigned short);
    KLAS_SHIM_SIZE(unsigned int);
    KLAS_SHIM_SIZE(unsigned long);
    KLAS_SHIM_SIZE(unsigned long long);
#undef KLAS_SHIM_SIZE
}

#endif /* KUIPER_H */
