/*
 * klas_oracle.c -- CPU restatement of the Klas matrix-multiply semantics.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the GPU kernels are
 * compared with (tests/, the smoke check and the CPU-baseline leg of the
 * benchmark); nothing in the product library links, loads or calls it.
 *
 * Parity pin: tests/test_oracle.py checks these functions bit-for-bit
 * against the reference's own host loops compiled from where they lie
 * (oracle/_ref, built by oracle/build.py) on the reference drivers'
 * deterministic inputs, and against the golden values committed under
 * tests/golden/ that were produced by those loops.
 *
 * Paths below are relative to the FStarLang/kuiper tree.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ 16-bit floats */

static inline double bf16_bits_to_double(uint16_t b)
{
    uint32_t u = (uint32_t) b << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return (double) f;
}

static inline double f16_bits_to_double(uint16_t h)
{
    const int sign = (h >> 15) & 1;
    const int exp = (h >> 10) & 0x1f;
    const int man = h & 0x3ff;
    double v;
    if (exp == 0)
        v = ldexp((double) man, -24);           /* subnormal or zero */
    else if (exp == 31)
        v = man ? NAN : INFINITY;
    else
        v = ldexp((double) (man | 0x400), exp - 25);
    return sign ? -v : v;
}

/* Round-to-nearest-even conversion of a double to IEEE binary16 bits in ONE
 * rounding step (what `half h = some_double;` does in the reference's gold
 * loop, test/matmul_common.c.inc:49-52).  Values of magnitude >= 65520
 * become infinity. */
static uint16_t double_to_f16_bits(double d)
{
    uint64_t bits;
    memcpy(&bits, &d, sizeof bits);
    const uint16_t sign = (uint16_t) ((bits >> 48) & 0x8000u);
    const double a = fabs(d);
    if (isnan(d)) return (uint16_t) (sign | 0x7e00u);
    if (a >= 65520.0) return (uint16_t) (sign | 0x7c00u);
    if (a < ldexp(1.0, -25)) return sign;                     /* rounds to zero (tie at 2^-25 -> even = 0) */
    int e;
    (void) frexp(a, &e);                                      /* a = f * 2^e, f in [0.5, 1) */
    int exp = e - 1;                                          /* a = 1.xxx * 2^exp */
    if (exp < -14) exp = -14;                                 /* subnormal: fixed quantum 2^-24 */
    const double quantum = ldexp(1.0, exp - 10);
    const double q = nearbyint(a / quantum);                  /* default mode: ties to even; exact division */
    const double r = q * quantum;
    if (r >= 65520.0) return (uint16_t) (sign | 0x7c00u);
    if (r < ldexp(1.0, -14)) return (uint16_t) (sign | (uint16_t) q);   /* subnormal */
    int e2;
    (void) frexp(r, &e2);
    const int ex = e2 - 1;
    const uint32_t man = (uint32_t) (r / ldexp(1.0, ex - 10)) - 1024u;
    return (uint16_t) (sign | (uint16_t) ((ex + 15) << 10) | (uint16_t) man);
}

/* Round-to-nearest-even double -> bfloat16 bits, one rounding step. */
static uint16_t double_to_bf16_bits(double d)
{
    uint64_t bits;
    memcpy(&bits, &d, sizeof bits);
    const uint16_t sign = (uint16_t) ((bits >> 48) & 0x8000u);
    if (isnan(d)) return (uint16_t) (sign | 0x7fc0u);
    const double a = fabs(d);
    if (a == 0.0) return sign;
    if (isinf(a)) return (uint16_t) (sign | 0x7f80u);
    int e;
    (void) frexp(a, &e);
    int exp = e - 1;
    if (exp < -126) exp = -126;
    const double quantum = ldexp(1.0, exp - 7);
    const double r = nearbyint(a / quantum) * quantum;
    if (r >= ldexp(1.0, 128)) return (uint16_t) (sign | 0x7f80u);
    const float f = (float) r;                                /* exact: r has <= 8 significant bits */
    uint32_t u;
    memcpy(&u, &f, sizeof u);
    return (uint16_t) (sign | (uint16_t) (u >> 16));
}

void klas_oracle_f64_to_f16_bits(const double *in, uint16_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = double_to_f16_bits(in[i]);
}

void klas_oracle_f64_to_bf16_bits(const double *in, uint16_t *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = double_to_bf16_bits(in[i]);
}

void klas_oracle_f16_bits_to_f64(const uint16_t *in, double *out, size_t n)
{
    for (size_t i = 0; i < n; i++) out[i] = f16_bits_to_double(in[i]);
}

/* ------------------------------------------------------------------ dense products */

static void set_threads(int threads)
{
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void) threads;
#endif
}

/* Row-major acc[m x n] = A[m x k] . B[k x n] in double, loop order i-k-j with
 * acc starting from 0 -- the reference drivers' gold loop `cpu_mul`
 * (test/matmul_common.c.inc:35-55).  Rows are independent, so they may be
 * spread over `threads` OpenMP threads without changing any result bit. */
#define DEFINE_F64ACC(NAME, ET, TO_DOUBLE)                                              \
    void NAME(size_t m, size_t n, size_t k, const ET *A, const ET *B, double *acc,      \
              int threads)                                                              \
    {                                                                                   \
        set_threads(threads);                                                           \
        _Pragma("omp parallel for schedule(static)")                                    \
        for (long i = 0; i < (long) m; i++) {                                           \
            double *row = acc + (size_t) i * n;                                         \
            for (size_t j = 0; j < n; j++) row[j] = 0.0;                                \
            for (size_t l = 0; l < k; l++) {                                            \
                const double a = TO_DOUBLE(A[(size_t) i * k + l]);                      \
                const ET *brow = B + l * n;                                             \
                for (size_t j = 0; j < n; j++) row[j] += a * TO_DOUBLE(brow[j]);        \
            }                                                                           \
        }                                                                               \
    }

#define ID_TO_DOUBLE(x) ((double) (x))
DEFINE_F64ACC(klas_oracle_acc_f32, float, ID_TO_DOUBLE)
DEFINE_F64ACC(klas_oracle_acc_f64, double, ID_TO_DOUBLE)
DEFINE_F64ACC(klas_oracle_acc_bf16, uint16_t, bf16_bits_to_double)
DEFINE_F64ACC(klas_oracle_acc_f16, uint16_t, f16_bits_to_double)

/* Same product with B stored column-major (as n x k, k contiguous). */
void klas_oracle_acc_bf16_bt(size_t m, size_t n, size_t k, const uint16_t *A, const uint16_t *Bt,
                             double *acc, int threads)
{
    set_threads(threads);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long) m; i++) {
        for (size_t j = 0; j < n; j++) {
            double s = 0.0;
            for (size_t l = 0; l < k; l++)
                s += bf16_bits_to_double(A[(size_t) i * k + l]) * bf16_bits_to_double(Bt[j * k + l]);
            acc[(size_t) i * n + j] = s;
        }
    }
}

/* Component-wise magnitude bound |A|.|B| in double (the scale of a relative-error test). */
void klas_oracle_absacc_f64(size_t m, size_t n, size_t k, const double *A, const double *B,
                            double *acc, int threads)
{
    set_threads(threads);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long) m; i++) {
        double *row = acc + (size_t) i * n;
        for (size_t j = 0; j < n; j++) row[j] = 0.0;
        for (size_t l = 0; l < k; l++) {
            const double a = fabs(A[(size_t) i * k + l]);
            for (size_t j = 0; j < n; j++) row[j] += a * fabs(B[l * n + j]);
        }
    }
}

/* Gold of the f32 / f64 drivers: cet(acc) (test/matmul_common.c.inc:49-52). */
void klas_oracle_gemm_f32(size_t m, size_t n, size_t k, const float *A, const float *B, float *C,
                          int threads)
{
    double *acc = (double *) malloc(sizeof(double) * m * n + 8);
    klas_oracle_acc_f32(m, n, k, A, B, acc, threads);
    for (size_t i = 0; i < m * n; i++) C[i] = (float) acc[i];
    free(acc);
}

void klas_oracle_gemm_f64(size_t m, size_t n, size_t k, const double *A, const double *B,
                          double *C, int threads)
{
    klas_oracle_acc_f64(m, n, k, A, B, C, threads);
}

/* bf16 x bf16 -> f32 and f16 x f16 -> f16 gold (one rounding of the double sum). */
void klas_oracle_gemm_bf16_f32(size_t m, size_t n, size_t k, const uint16_t *A, const uint16_t *B,
                               float *C, int threads)
{
    double *acc = (double *) malloc(sizeof(double) * m * n + 8);
    klas_oracle_acc_bf16(m, n, k, A, B, acc, threads);
    for (size_t i = 0; i < m * n; i++) C[i] = (float) acc[i];
    free(acc);
}

void klas_oracle_gemm_f16_f16(size_t m, size_t n, size_t k, const uint16_t *A, const uint16_t *B,
                              uint16_t *C, int threads)
{
    double *acc = (double *) malloc(sizeof(double) * m * n + 8);
    klas_oracle_acc_f16(m, n, k, A, B, acc, threads);
    klas_oracle_f64_to_f16_bits(acc, C, m * n);
    free(acc);
}

/* `cpu_sgemm` for float: out = alpha * float(acc) + beta * C, evaluated in
 * float with separately rounded operations (test/matmul_common.c.inc:58-68;
 * the spec's lincomb, src/lib/spec/Kuiper.Spec.GEMM.fsti:27-34). */
void klas_oracle_sgemm_f32(size_t m, size_t n, size_t k, float alpha, float beta, const float *A,
                           const float *B, const float *Cin, float *Cout, int threads)
{
    klas_oracle_gemm_f32(m, n, k, A, B, Cout, threads);
    for (size_t i = 0; i < m * n; i++) {
        volatile float p = alpha * Cout[i];
        volatile float q = beta * Cin[i];
        Cout[i] = p + q;
    }
}

/* Wrapping integer products: Z/2^32 and Z/2^64 (src/lib/kuiper/types/Kuiper.Scalars.fst:30-47).
 * The reference drivers' gold accumulates these types in double, which is only
 * exact while every sum stays below 2^53; the drivers' inputs do, and on those
 * inputs this function and that loop agree bit for bit. */
#define DEFINE_WRAP(NAME, ET)                                                           \
    void NAME(size_t m, size_t n, size_t k, ET alpha, ET beta, int scaled, const ET *A, \
              const ET *B, ET *C, int threads)                                          \
    {                                                                                   \
        set_threads(threads);                                                           \
        _Pragma("omp parallel for schedule(static)")                                    \
        for (long i = 0; i < (long) m; i++) {                                           \
            ET *tmp = (ET *) calloc(n ? n : 1, sizeof(ET));                             \
            for (size_t l = 0; l < k; l++) {                                            \
                const ET a = A[(size_t) i * k + l];                                     \
                const ET *brow = B + l * n;                                             \
                for (size_t j = 0; j < n; j++) tmp[j] += a * brow[j];                   \
            }                                                                           \
            ET *crow = C + (size_t) i * n;                                              \
            for (size_t j = 0; j < n; j++)                                              \
                crow[j] = scaled ? (ET) (beta * crow[j] + alpha * tmp[j]) : tmp[j];     \
            free(tmp);                                                                  \
        }                                                                               \
    }

DEFINE_WRAP(klas_oracle_gemm_u32, uint32_t)
DEFINE_WRAP(klas_oracle_gemm_u64, uint64_t)

/* Batched f32 product accumulated in float, order b-i-l-j
 * (test/Test_Klas_GEMM_Naive1__F32_Batched.cu:14-29). */
void klas_oracle_batched_f32(size_t batch, size_t m, size_t n, size_t k, const float *A,
                             const float *B, float *C)
{
    memset(C, 0, sizeof(float) * batch * m * n);
    for (size_t b = 0; b < batch; b++)
        for (size_t i = 0; i < m; i++)
            for (size_t l = 0; l < k; l++)
                for (size_t j = 0; j < n; j++) {
                    volatile float p = A[b * m * k + i * k + l] * B[b * k * n + l * n + j];
                    C[b * m * n + i * n + j] += p;
                }
}

/* ------------------------------------------------------------------ CSR x dense */

/* u32, wrapping, each row's products summed in CSR order from 0: the reference's verified
 * host loop Kuiper_Example_Sparse_MM__mmsd_u32_rr (dist/Kuiper_Example_Sparse_MM.cu:4-24). */
void klas_oracle_spmm_u32(uint32_t rows, uint32_t cols, const uint32_t *elems,
                          const uint32_t *col_ind, const uint32_t *row_off, const uint32_t *B,
                          uint32_t *C, int threads)
{
    set_threads(threads);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long) rows; i++) {
        uint32_t *crow = C + (size_t) i * cols;
        for (uint32_t j = 0; j < cols; j++) crow[j] = 0u;
        for (uint32_t p = row_off[i]; p < row_off[i + 1]; p++) {
            const uint32_t a = elems[p];
            const uint32_t *brow = B + (size_t) col_ind[p] * cols;
            for (uint32_t j = 0; j < cols; j++) crow[j] += a * brow[j];
        }
    }
}

/* f32 values, double accumulation in CSR order (the f32 instance of the same loop;
 * double keeps the checker's own rounding out of the comparison). */
void klas_oracle_spmm_f32(uint32_t rows, uint32_t cols, const float *elems,
                          const uint32_t *col_ind, const uint32_t *row_off, const float *B,
                          double *C, double *Cabs, int threads)
{
    set_threads(threads);
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long) rows; i++) {
        double *crow = C + (size_t) i * cols;
        double *arow = Cabs ? Cabs + (size_t) i * cols : NULL;
        for (uint32_t j = 0; j < cols; j++) crow[j] = 0.0;
        if (arow)
            for (uint32_t j = 0; j < cols; j++) arow[j] = 0.0;
        for (uint32_t p = row_off[i]; p < row_off[i + 1]; p++) {
            const double a = elems[p];
            const float *brow = B + (size_t) col_ind[p] * cols;
            for (uint32_t j = 0; j < cols; j++) crow[j] += a * (double) brow[j];
            if (arow)
                for (uint32_t j = 0; j < cols; j++) arow[j] += fabs(a * (double) brow[j]);
        }
    }
}

/* Dense float product with a float running sum, order i-j-k: the SpMM drivers' gold
 * `cpu_matmul` (test/Test_Klas_SPMM__F32.cu:11-20). */
void klas_oracle_dense_matmul_f32(size_t rows, size_t shared, size_t cols, const float *A,
                                  const float *B, float *C)
{
    for (size_t i = 0; i < rows; i++)
        for (size_t j = 0; j < cols; j++) {
            float sum = 0;
            for (size_t l = 0; l < shared; l++) {
                volatile float p = A[i * shared + l] * B[l * cols + j];
                sum += p;
            }
            C[i * cols + j] = sum;
        }
}

/* ------------------------------------------------------------------ row-wise neighbours */

/* Softmax / log-softmax of n doubles: maximum, then sum of exp(x - max), then the quotient (or
 * x - (max + log sum)) -- the gold of the softmax drivers, cpu_softmax / cpu_logsoftmax
 * (test/softmax_test_common.c.inc:37-63). */
void klas_oracle_softmax_f64(const double *in, double *out, size_t n, int log_softmax)
{
    if (n == 0) return;
    double mx = in[0];
    for (size_t i = 1; i < n; i++)
        if (in[i] > mx) mx = in[i];
    double sum = 0.0;
    for (size_t i = 0; i < n; i++) {
        out[i] = exp(in[i] - mx);
        sum += out[i];
    }
    if (log_softmax) {
        const double lse = mx + log(sum);
        for (size_t i = 0; i < n; i++) out[i] = in[i] - lse;
    } else {
        for (size_t i = 0; i < n; i++) out[i] /= sum;
    }
}

/* b[r][c] = a[r] * b[r][c] in double, b row-major (dist/Klas_RowScale.cu:9-15). */
void klas_oracle_rowscale_f64(size_t m, size_t n, const double *a, double *b)
{
    for (size_t r = 0; r < m; r++)
        for (size_t c = 0; c < n; c++) b[r * n + c] = a[r] * b[r * n + c];
}

/* Element-wise operand maps of the fused tensor-core GEMM: evaluated in float on the 16-bit
 * value and rounded once (nearest even) back to the 16-bit type -- what the reference's
 * KPR_LOAD_MAP does to the registers of a loaded wmma fragment (include/kuiper/tensorcores.h:30-38),
 * e.g. sqrt in the demo dist/Kuiper_Example_Fused_GEMM.cu:8-27.
 * map: 0 id, 1 sqrt, 2 abs, 3 square, 4 relu, 5 neg. */
void klas_oracle_map16(const uint16_t *in, uint16_t *out, size_t n, int bf16, int map)
{
    for (size_t i = 0; i < n; ++i) {
        const float x = (float)(bf16 ? bf16_bits_to_double(in[i]) : f16_bits_to_double(in[i]));
        float y;
        switch (map) {
            case 1: y = sqrtf(x); break;
            case 2: y = fabsf(x); break;
            case 3: y = x * x; break;
            case 4: y = x > 0.0f ? x : 0.0f; break;
            case 5: y = -x; break;
            default: y = x; break;
        }
        out[i] = bf16 ? double_to_bf16_bits((double)y) : double_to_f16_bits((double)y);
    }
}

/* The (min,+) ring on 16-bit path lengths, 0 = no path, and the squaring step built on it:
 * dist/Kuiper_GraphDist.cu:9-24 (add_, mult) and :26-45 (b[i][j] = add_(b[i][j], sum_k ...)),
 * generalised to C = add(C, A (x) B) with A m x k, B k x n. */
static uint16_t dist_add(uint16_t x, uint16_t y) { return (x == 0 || (y != 0 && y < x)) ? y : x; }
static uint16_t dist_mult(uint16_t x, uint16_t y) { return (x == 0 || y == 0) ? 0 : (uint16_t)((uint32_t)x + (uint32_t)y); }

void klas_oracle_minplus_u16(size_t m, size_t n, size_t k, const uint16_t *A, const uint16_t *B, uint16_t *C)
{
#pragma omp parallel for
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j) {
            uint16_t sum = 0;
            for (size_t kk = 0; kk < k; ++kk) sum = dist_add(sum, dist_mult(A[i * k + kk], B[kk * n + j]));
            C[i * n + j] = dist_add(C[i * n + j], sum);
        }
}

/* Dense -> CSR as the drivers build it on the host (test/spmm_common.c.inc:107-137): entries != 0
 * in row-major scan order.  `as_float` selects the float comparison (-0.0 == 0, NaN != 0) on the
 * same 32-bit words.  elems / col_ind may be NULL to count only; returns nnz. */
uint32_t klas_oracle_sparsify32(const uint32_t *M, size_t rows, size_t cols, int as_float, uint32_t *row_off,
                                uint32_t *elems, uint32_t *col_ind)
{
    uint32_t idx = 0;
    row_off[0] = 0;
    for (size_t i = 0; i < rows; ++i) {
        for (size_t j = 0; j < cols; ++j) {
            const uint32_t w = M[i * cols + j];
            int nz;
            if (as_float) {
                float f;
                memcpy(&f, &w, 4);
                nz = f != 0.0f;
            } else {
                nz = w != 0;
            }
            if (nz) {
                if (elems) {
                    elems[idx] = w;
                    col_ind[idx] = (uint32_t)j;
                }
                idx++;
            }
        }
        row_off[i + 1] = idx;
    }
    return idx;
}

int klas_oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
