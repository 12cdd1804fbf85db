// Row-wise neighbours of the matrix products: softmax / log-softmax of a vector or of the
// rows of a matrix, row scaling, and sum reduction.  All are bandwidth-bound; each is written
// as the minimum number of passes over the data.
//
//   softmax, one long vector   two launches: (1) every CTA folds one chunk (>= 16384 elements, at
//                              most 2048 chunks) into a running (max, sum of exp(x - max)) pair
//                              and writes it to scratch; (2) every CTA folds the per-chunk pairs
//                              (<= 32 KiB, L2 resident), then rewrites its chunk.  2 reads + 1
//                              write of the vector.
//   softmax, rows of a matrix  one CTA per row, the same two passes inside the CTA, no scratch.
//   reduce                     per-CTA partial sums to scratch, one CTA folds them in a fixed order
//                              (deterministic for floating point).
//
// Takes over the work of the reference's multi-launch kernels: dist/Klas_Softmax.cu:128-260
// (block max -> subtract -> block sum of exp -> divide, one CTA for the reductions),
// dist/Klas_LogSoftmax.cu, dist/Klas_RowSoftmax.cu:3-45, dist/Klas_RowScale.cu:3-30,
// dist/Klas_HReduce.cu and dist/Klas_AtomicReduce.cu (one atomic per element).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <type_traits>

#include "klas_internal.h"

namespace klas {
namespace rowops {

constexpr int THREADS = 256;
constexpr uint64_t MIN_CHUNK = 16384;   // fewest elements of a long vector one CTA owns
constexpr uint32_t MAX_PARTS = 2048;    // most CTAs (and per-chunk statistics) of one vector

template <typename T>
struct Num {
    using Acc = float;
    static __device__ __forceinline__ float up(T v) { return float(v); }
    static __device__ __forceinline__ T down(float v) { return T(v); }
};
template <>
struct Num<__half> {
    using Acc = float;
    static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <>
struct Num<__nv_bfloat16> {
    using Acc = float;
    static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct Num<double> {
    using Acc = double;
    static __device__ __forceinline__ double up(double v) { return v; }
    static __device__ __forceinline__ double down(double v) { return v; }
};
template <>
struct Num<uint32_t> {
    using Acc = uint32_t;
    static __device__ __forceinline__ uint32_t up(uint32_t v) { return v; }
    static __device__ __forceinline__ uint32_t down(uint32_t v) { return v; }
};
template <>
struct Num<uint64_t> {
    using Acc = uint64_t;
    static __device__ __forceinline__ uint64_t up(uint64_t v) { return v; }
    static __device__ __forceinline__ uint64_t down(uint64_t v) { return v; }
};

// f32 exponential as 2^(x log2 e) on the special-function unit: 2 ulp plus the rounding of the
// product, i.e. a relative error below 1e-6 wherever exp(x) is not negligible (the arguments
// here are x - max <= 0).  expf's extra range reduction would triple the instruction count of
// kernels that are otherwise bandwidth-bound on 16-bit data.
__device__ __forceinline__ float fexp(float x) { return exp2f(x * 1.4426950408889634f); }
__device__ __forceinline__ double fexp(double x) { return exp(x); }
__device__ __forceinline__ float flog(float x) { return logf(x); }
__device__ __forceinline__ double flog(double x) { return log(x); }

// Running softmax statistics of a set of values: their maximum and sum of exp(x - maximum).
template <typename A>
struct MaxSum {
    A m, s;
};
template <typename A>
__device__ __forceinline__ MaxSum<A> ms_empty() {
    return {A(-INFINITY), A(0)};
}
template <typename A>
__device__ __forceinline__ MaxSum<A> ms_merge(MaxSum<A> x, MaxSum<A> y) {
    if (y.s == A(0)) return x;
    if (x.s == A(0)) return y;
    const A m = x.m > y.m ? x.m : y.m;
    return {m, x.s * fexp(x.m - m) + y.s * fexp(y.m - m)};
}
template <typename A>
__device__ __forceinline__ MaxSum<A> ms_block_reduce(MaxSum<A> v, MaxSum<A> *smem) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        MaxSum<A> o;
        o.m = __shfl_xor_sync(0xffffffffu, v.m, off);
        o.s = __shfl_xor_sync(0xffffffffu, v.s, off);
        v = ms_merge(v, o);
    }
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    MaxSum<A> r = ms_empty<A>();
    for (int w = 0; w < THREADS / 32; ++w) r = ms_merge(r, smem[w]);   // same order in every thread
    __syncthreads();
    return r;
}

template <typename T, bool LOG>
__device__ __forceinline__ T finish(T x, typename Num<T>::Acc m, typename Num<T>::Acc inv_or_logs) {
    using A = typename Num<T>::Acc;
    const A v = Num<T>::up(x);
    if (LOG) return Num<T>::down((v - m) - inv_or_logs);   // inv_or_logs = log(sum)
    return Num<T>::down(fexp(v - m) * inv_or_logs);          // inv_or_logs = 1 / sum
}

// 16 bytes of T, moved with one access where the address allows it.
template <typename T>
struct alignas(16) Pack {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
};

// Folds k values into the running statistics: one exp per value plus one per new maximum.
// A state whose maximum is still -inf (nothing finite seen yet) accumulates nothing, so -inf
// entries (masked positions) contribute exactly zero wherever they stand.
template <typename A, int K>
__device__ __forceinline__ void ms_fold(MaxSum<A> &st, const A (&v)[K]) {
    A bm = v[0];
#pragma unroll
    for (int j = 1; j < K; ++j) bm = v[j] > bm ? v[j] : bm;
    if (bm > st.m) {
        st.s *= fexp(st.m - bm);   // exp(-inf) = 0 on the first finite value; s is 0 then anyway
        st.m = bm;
    }
    if (st.m > A(-INFINITY)) {
#pragma unroll
        for (int j = 0; j < K; ++j) st.s += fexp(v[j] - st.m);
    }
}

// Elements of a[lo, hi) in front of the first 16-byte boundary (all of them if none is reached).
template <typename T>
__device__ __forceinline__ uint64_t head_elems(const T *a, uint64_t lo, uint64_t hi) {
    const uint64_t h = ((16u - (reinterpret_cast<uintptr_t>(a + lo) & 15u)) & 15u) / sizeof(T);
    return h < hi - lo ? h : hi - lo;
}

// Statistics of a[lo, hi) gathered by the whole CTA; every thread returns the CTA's result.
// Scalar accesses up to the first 16-byte boundary and after the last, 16-byte packs between,
// four in flight per thread.
template <typename T>
__device__ __forceinline__ MaxSum<typename Num<T>::Acc> cta_stats(const T *a, uint64_t lo, uint64_t hi,
                                                                   MaxSum<typename Num<T>::Acc> *smem) {
    using A = typename Num<T>::Acc;
    constexpr int N = Pack<T>::N;
    constexpr int UNROLL = 4;
    MaxSum<A> st = ms_empty<A>();
    const uint64_t head = head_elems(a, lo, hi);
    if (threadIdx.x < head) {
        const A one[1] = {A(Num<T>::up(a[lo + threadIdx.x]))};
        ms_fold(st, one);
    }
    lo += head;
    uint64_t done = lo;
    {
        const uint64_t packs = (hi - lo) / N;
        const Pack<T> *p = reinterpret_cast<const Pack<T> *>(a + lo);
        uint64_t i = threadIdx.x;
        for (; i + uint64_t(UNROLL - 1) * THREADS < packs; i += uint64_t(UNROLL) * THREADS) {
            Pack<T> buf[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) buf[u] = p[i + uint64_t(u) * THREADS];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                A vals[N];
#pragma unroll
                for (int j = 0; j < N; ++j) vals[j] = A(Num<T>::up(buf[u].v[j]));
                ms_fold(st, vals);
            }
        }
        for (; i < packs; i += THREADS) {
            const Pack<T> one = p[i];
            A vals[N];
#pragma unroll
            for (int j = 0; j < N; ++j) vals[j] = A(Num<T>::up(one.v[j]));
            ms_fold(st, vals);
        }
        done = lo + packs * N;
    }
    for (uint64_t i = done + threadIdx.x; i < hi; i += THREADS) {
        const A one[1] = {A(Num<T>::up(a[i]))};
        ms_fold(st, one);
    }
    return ms_block_reduce(st, smem);
}

// Rewrites a[lo, hi) as the (log-)softmax given the statistics of the whole row or vector.
template <typename T, bool LOG>
__device__ __forceinline__ void cta_apply(T *a, uint64_t lo, uint64_t hi, typename Num<T>::Acc m,
                                          typename Num<T>::Acc scale_or_logs) {
    constexpr int N = Pack<T>::N;
    const uint64_t head = head_elems(a, lo, hi);
    if (threadIdx.x < head) a[lo + threadIdx.x] = finish<T, LOG>(a[lo + threadIdx.x], m, scale_or_logs);
    lo += head;
    uint64_t done = lo;
    {
        const uint64_t packs = (hi - lo) / N;
        Pack<T> *p = reinterpret_cast<Pack<T> *>(a + lo);
        for (uint64_t i = threadIdx.x; i < packs; i += THREADS) {
            Pack<T> one = p[i];
#pragma unroll
            for (int j = 0; j < N; ++j) one.v[j] = finish<T, LOG>(one.v[j], m, scale_or_logs);
            p[i] = one;
        }
        done = lo + packs * N;
    }
    for (uint64_t i = done + threadIdx.x; i < hi; i += THREADS) a[i] = finish<T, LOG>(a[i], m, scale_or_logs);
}

// ---- long vector ------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) softmax_partials_kernel(const T *__restrict__ a, uint64_t n,
                                                                  uint64_t chunk,
                                                                  MaxSum<typename Num<T>::Acc> *partials) {
    using A = typename Num<T>::Acc;
    __shared__ MaxSum<A> smem[THREADS / 32];
    const uint64_t lo = uint64_t(blockIdx.x) * chunk;
    const uint64_t hi = lo + chunk < n ? lo + chunk : n;
    const MaxSum<A> st = cta_stats<T>(a, lo, hi, smem);
    if (threadIdx.x == 0) partials[blockIdx.x] = st;
}

template <typename T, bool LOG>
__global__ void __launch_bounds__(THREADS) softmax_apply_kernel(T *a, uint64_t n, uint64_t chunk,
                                                               const MaxSum<typename Num<T>::Acc> *partials,
                                                               uint32_t nparts) {
    using A = typename Num<T>::Acc;
    __shared__ MaxSum<A> smem[THREADS / 32];
    MaxSum<A> st = ms_empty<A>();
    for (uint32_t i = threadIdx.x; i < nparts; i += THREADS) st = ms_merge(st, partials[i]);
    st = ms_block_reduce(st, smem);
    const A denom = LOG ? flog(st.s) : A(1) / st.s;
    // Last chunk first: the end of the vector is what the first launch left in L2.
    const uint64_t lo = uint64_t(nparts - 1 - blockIdx.x) * chunk;
    const uint64_t hi = lo + chunk < n ? lo + chunk : n;
    cta_apply<T, LOG>(a, lo, hi, st.m, denom);
}

// ---- rows of a matrix -------------------------------------------------------------------------
template <typename T, bool LOG>
__global__ void __launch_bounds__(THREADS) row_softmax_kernel(T *a, uint64_t cols) {
    using A = typename Num<T>::Acc;
    __shared__ MaxSum<A> smem[THREADS / 32];
    T *row = a + uint64_t(blockIdx.x) * cols;
    const MaxSum<A> st = cta_stats<T>(row, 0, cols, smem);
    const A denom = LOG ? flog(st.s) : A(1) / st.s;
    cta_apply<T, LOG>(row, 0, cols, st.m, denom);   // second read of the row comes from L2
}

// Rows that fit in registers (one warp or one CTA per row, PACKS 16-byte packs per thread) are
// read once and written once, and need ONE exponential per element: the maximum first (a
// compare per element), then e = exp(x - max) kept in registers while it is summed, then e / sum.
// For f32 arithmetic exp(x - max) is ex2(x * log2 e - max * log2 e), one fused multiply-add and
// one special-function instruction; the rounding of max * log2 e scales every e of the row by
// the same factor, which cancels in e / sum.  `reduce_max` / `reduce_sum` combine the partial
// results of the threads that share the row.
template <typename T, bool LOG, int PACKS, typename RMax, typename RSum>
__device__ __forceinline__ void row_in_registers(Pack<T> *row, uint32_t packs, uint32_t first, uint32_t step,
                                                 RMax reduce_max, RSum reduce_sum) {
    using A = typename Num<T>::Acc;
    constexpr int N = Pack<T>::N;
    A e[PACKS][N];
    A m = A(-INFINITY);
#pragma unroll
    for (int u = 0; u < PACKS; ++u) {
        const uint32_t i = first + step * u;
        if (i < packs) {
            const Pack<T> in = row[i];
#pragma unroll
            for (int j = 0; j < N; ++j) {
                e[u][j] = A(Num<T>::up(in.v[j]));
                m = e[u][j] > m ? e[u][j] : m;
            }
        }
    }
    m = reduce_max(m);
    A sum = A(0);
    if constexpr (std::is_same<A, float>::value) {
        constexpr float L = 1.4426950408889634f;
        const float nml = -m * L;
#pragma unroll
        for (int u = 0; u < PACKS; ++u) {
            if (first + step * u < packs) {
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    float p;
                    // LOG keeps the common factor (it does not cancel in log(sum)): subtract first
                    const float arg = LOG ? (e[u][j] - m) * L : fmaf(e[u][j], L, nml);
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(p) : "f"(arg));
                    sum += p;
                    if (!LOG) e[u][j] = p;
                }
            }
        }
    } else {
#pragma unroll
        for (int u = 0; u < PACKS; ++u) {
            if (first + step * u < packs) {
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    const A p = fexp(e[u][j] - m);
                    sum += p;
                    if (!LOG) e[u][j] = p;
                }
            }
        }
    }
    sum = reduce_sum(sum);
    const A k = LOG ? m + flog(sum) : A(1) / sum;
#pragma unroll
    for (int u = 0; u < PACKS; ++u) {
        const uint32_t i = first + step * u;
        if (i < packs) {
            Pack<T> out;
#pragma unroll
            for (int j = 0; j < N; ++j) out.v[j] = Num<T>::down(LOG ? e[u][j] - k : e[u][j] * k);
            row[i] = out;
        }
    }
}

// Short rows: one warp per row; the reductions are shuffles.  Needs 16-byte aligned rows (cols a
// multiple of the pack size, aligned base).
template <typename T, bool LOG, int PACKS>
__global__ void __launch_bounds__(THREADS) row_softmax_warp_kernel(T *a, uint64_t rows, uint32_t cols) {
    using A = typename Num<T>::Acc;
    const uint64_t row_id = uint64_t(blockIdx.x) * (THREADS / 32) + (threadIdx.x >> 5);
    if (row_id >= rows) return;
    auto warp_max = [](A v) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const A o = __shfl_xor_sync(0xffffffffu, v, off);
            v = o > v ? o : v;
        }
        return v;
    };
    auto warp_sum = [](A v) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        return v;
    };
    row_in_registers<T, LOG, PACKS>(reinterpret_cast<Pack<T> *>(a + row_id * cols), cols / Pack<T>::N,
                                    threadIdx.x & 31u, 32u, warp_max, warp_sum);
}

// Medium rows: one CTA per row; the partial results meet in shared memory.
template <typename T, bool LOG, int PACKS>
__global__ void __launch_bounds__(THREADS) row_softmax_cta_kernel(T *a, uint64_t rows, uint32_t cols) {
    using A = typename Num<T>::Acc;
    __shared__ A part[2][THREADS / 32];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    auto cta_max = [&](A v) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const A o = __shfl_xor_sync(0xffffffffu, v, off);
            v = o > v ? o : v;
        }
        if (lane == 0) part[0][warp] = v;
        __syncthreads();
        A r = part[0][0];
#pragma unroll
        for (int w = 1; w < THREADS / 32; ++w) r = part[0][w] > r ? part[0][w] : r;
        return r;
    };
    auto cta_sum = [&](A v) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        if (lane == 0) part[1][warp] = v;
        __syncthreads();
        A r = A(0);
#pragma unroll
        for (int w = 0; w < THREADS / 32; ++w) r += part[1][w];   // same order in every thread
        return r;
    };
    if (blockIdx.x < rows)
        row_in_registers<T, LOG, PACKS>(reinterpret_cast<Pack<T> *>(a + uint64_t(blockIdx.x) * cols), cols / Pack<T>::N,
                                        threadIdx.x, uint32_t(THREADS), cta_max, cta_sum);
}

// ---- row scaling: b[r][c] = scale[r] * b[r][c], b row- or column-major -------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) rowscale_kernel(const T *__restrict__ scale, T *b, uint64_t m,
                                                          uint64_t n, int col_major) {
    // i walks memory order in both layouts; the row index follows it incrementally (one division
    // per thread instead of one per element).
    const uint64_t total = m * n, stride = uint64_t(gridDim.x) * THREADS;
    uint64_t i = uint64_t(blockIdx.x) * THREADS + threadIdx.x;
    if (col_major) {
        uint64_t r = i % m;
        const uint64_t dr = stride % m;
        for (; i < total; i += stride) {
            b[i] = scale[r] * b[i];
            r += dr;
            if (r >= m) r -= m;
        }
    } else {
        uint64_t r = i / n, c = i % n;
        const uint64_t dr = stride / n, dc = stride % n;
        for (; i < total; i += stride) {
            b[i] = scale[r] * b[i];
            r += dr;
            c += dc;
            if (c >= n) {
                c -= n;
                ++r;
            }
        }
    }
}

// ---- sum reduction ----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(THREADS) reduce_partials_kernel(const T *__restrict__ a, uint64_t n,
                                                                 typename Num<T>::Acc *partials) {
    using A = typename Num<T>::Acc;
    __shared__ A smem[THREADS / 32];
    constexpr int N = Pack<T>::N;
    A acc = A(0);
    const uint64_t packs = (reinterpret_cast<uintptr_t>(a) & 15u) == 0 ? n / N : 0;
    const Pack<T> *p = reinterpret_cast<const Pack<T> *>(a);
    for (uint64_t i = uint64_t(blockIdx.x) * THREADS + threadIdx.x; i < packs; i += uint64_t(gridDim.x) * THREADS) {
        const Pack<T> one = p[i];
#pragma unroll
        for (int j = 0; j < N; ++j) acc += A(Num<T>::up(one.v[j]));
    }
    for (uint64_t i = packs * N + uint64_t(blockIdx.x) * THREADS + threadIdx.x; i < n;
         i += uint64_t(gridDim.x) * THREADS)
        acc += A(Num<T>::up(a[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        A r = A(0);
        for (int w = 0; w < THREADS / 32; ++w) r += smem[w];
        partials[blockIdx.x] = r;
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) reduce_final_kernel(const typename Num<T>::Acc *partials, uint32_t nparts,
                                                              T *out) {
    using A = typename Num<T>::Acc;
    __shared__ A smem[THREADS];
    A acc = A(0);
    for (uint32_t i = threadIdx.x; i < nparts; i += THREADS) acc += partials[i];
    smem[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        A r = A(0);
        for (int i = 0; i < THREADS; ++i) r += smem[i];
        *out = Num<T>::down(r);
    }
}

// Elements per CTA of an n-element vector: a multiple of 1024, at least MIN_CHUNK, and large
// enough that no more than MAX_PARTS CTAs are needed.
static uint64_t vector_chunk(uint64_t n) {
    uint64_t c = (n + MAX_PARTS - 1) / MAX_PARTS;
    c = (c + 1023) / 1024 * 1024;
    return c < MIN_CHUNK ? MIN_CHUNK : c;
}
static uint32_t vector_chunks(uint64_t n) {
    const uint64_t c = vector_chunk(n);
    return uint32_t((n + c - 1) / c);
}
static uint32_t reduce_blocks(uint64_t n) {
    const uint64_t want = (n + uint64_t(THREADS) * 16 - 1) / (uint64_t(THREADS) * 16);
    return uint32_t(want < 1 ? 1 : (want > 1024 ? 1024 : want));
}

template <typename T>
static int softmax_t(int log_softmax, uint64_t rows, uint64_t cols, void *a, void *scratch, cudaStream_t s,
                     bool as_rows = false) {
    T *p = static_cast<T *>(a);
    if (rows > 1 || as_rows) {   // as_rows: a single row takes the row kernels too (no scratch)
        if (rows > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "softmax: too many rows");
        constexpr uint64_t N = Pack<T>::N;
        if (cols % N == 0 && cols / N <= 32 * 4 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0) {
            // warp per row, row held in registers: 2 or 4 packs per lane (more costs occupancy: measured slower)
            const uint64_t per_lane = (cols / N + 31) / 32;
            const uint64_t ctas = (rows + THREADS / 32 - 1) / (THREADS / 32);
            const unsigned grid = unsigned(ctas);
#define KLAS_ROW_WARP(P)                                                                                   \
    do {                                                                                                   \
        if (log_softmax)                                                                                   \
            row_softmax_warp_kernel<T, true, P><<<grid, THREADS, 0, s>>>(p, rows, uint32_t(cols));         \
        else                                                                                               \
            row_softmax_warp_kernel<T, false, P><<<grid, THREADS, 0, s>>>(p, rows, uint32_t(cols));        \
    } while (0)
            if (per_lane <= 2) KLAS_ROW_WARP(2);
            else KLAS_ROW_WARP(4);
#undef KLAS_ROW_WARP
            return check_cuda(cudaGetLastError(), "row_softmax_warp_kernel launch");
        }
        if (cols % N == 0 && cols / N <= uint64_t(THREADS) * 8 && (reinterpret_cast<uintptr_t>(a) & 15u) == 0) {
            // CTA per row, row held in registers: 2, 4 or 8 packs per thread
            const uint64_t per_thread = (cols / N + THREADS - 1) / THREADS;
            const unsigned grid = unsigned(rows);
#define KLAS_ROW_CTA(P)                                                                                    \
    do {                                                                                                   \
        if (log_softmax)                                                                                   \
            row_softmax_cta_kernel<T, true, P><<<grid, THREADS, 0, s>>>(p, rows, uint32_t(cols));          \
        else                                                                                               \
            row_softmax_cta_kernel<T, false, P><<<grid, THREADS, 0, s>>>(p, rows, uint32_t(cols));         \
    } while (0)
            if (per_thread <= 2) KLAS_ROW_CTA(2);
            else if (per_thread <= 4) KLAS_ROW_CTA(4);
            else KLAS_ROW_CTA(8);
#undef KLAS_ROW_CTA
            return check_cuda(cudaGetLastError(), "row_softmax_cta_kernel launch");
        }
        if (log_softmax)
            row_softmax_kernel<T, true><<<unsigned(rows), THREADS, 0, s>>>(p, cols);
        else
            row_softmax_kernel<T, false><<<unsigned(rows), THREADS, 0, s>>>(p, cols);
        return check_cuda(cudaGetLastError(), "row_softmax_kernel launch");
    }
    using A = typename Num<T>::Acc;
    const uint64_t chunk = vector_chunk(cols);
    const uint32_t parts = vector_chunks(cols);
    auto *partials = static_cast<MaxSum<A> *>(scratch);
    softmax_partials_kernel<T><<<parts, THREADS, 0, s>>>(p, cols, chunk, partials);
    if (int rc = check_cuda(cudaGetLastError(), "softmax_partials_kernel launch")) return rc;
    if (log_softmax)
        softmax_apply_kernel<T, true><<<parts, THREADS, 0, s>>>(p, cols, chunk, partials, parts);
    else
        softmax_apply_kernel<T, false><<<parts, THREADS, 0, s>>>(p, cols, chunk, partials, parts);
    return check_cuda(cudaGetLastError(), "softmax_apply_kernel launch");
}

template <typename T>
static int reduce_t(uint64_t n, const void *a, void *out, void *scratch, cudaStream_t s) {
    using A = typename Num<T>::Acc;
    const uint32_t blocks = reduce_blocks(n);
    reduce_partials_kernel<T><<<blocks, THREADS, 0, s>>>(static_cast<const T *>(a), n, static_cast<A *>(scratch));
    if (int rc = check_cuda(cudaGetLastError(), "reduce_partials_kernel launch")) return rc;
    reduce_final_kernel<T><<<1, THREADS, 0, s>>>(static_cast<const A *>(scratch), blocks, static_cast<T *>(out));
    return check_cuda(cudaGetLastError(), "reduce_final_kernel launch");
}

}  // namespace rowops

size_t softmax_scratch_bytes(uint64_t rows, uint64_t cols) {
    if (rows != 1) return 0;
    return size_t(rowops::vector_chunks(cols)) * 16;
}

size_t reduce_scratch_bytes(uint64_t n) { return size_t(rowops::reduce_blocks(n)) * 8; }

int launch_softmax(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a, void *scratch,
                   size_t scratch_bytes, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return KLAS_OK;
    if (!a) return fail(KLAS_ERR_INVALID, "softmax: null data pointer");
    const size_t need = softmax_scratch_bytes(rows, cols);
    if (need > 0 && (!scratch || scratch_bytes < need))
        return fail(KLAS_ERR_INVALID, "softmax: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
    if (need > 0 && (reinterpret_cast<uintptr_t>(scratch) & 15u))
        return fail(KLAS_ERR_INVALID, "softmax: scratch must be 16-byte aligned");
    switch (dtype) {
        case KLAS_F16: return rowops::softmax_t<__half>(log_softmax, rows, cols, a, scratch, stream);
        case KLAS_BF16: return rowops::softmax_t<__nv_bfloat16>(log_softmax, rows, cols, a, scratch, stream);
        case KLAS_F32: return rowops::softmax_t<float>(log_softmax, rows, cols, a, scratch, stream);
        case KLAS_F64: return rowops::softmax_t<double>(log_softmax, rows, cols, a, scratch, stream);
        default: return fail(KLAS_ERR_INVALID, "softmax: dtype must be F16, BF16, F32 or F64");
    }
}

// Softmax of every row with the row kernels whatever `rows` is: a one-row matrix (one query of one
// head in attention) must not fall into the chunked vector path, which needs scratch.
int launch_softmax_rows(int dtype, int log_softmax, uint64_t rows, uint64_t cols, void *a, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return KLAS_OK;
    if (!a) return fail(KLAS_ERR_INVALID, "softmax: null data pointer");
    switch (dtype) {
        case KLAS_F16: return rowops::softmax_t<__half>(log_softmax, rows, cols, a, nullptr, stream, true);
        case KLAS_BF16: return rowops::softmax_t<__nv_bfloat16>(log_softmax, rows, cols, a, nullptr, stream, true);
        case KLAS_F32: return rowops::softmax_t<float>(log_softmax, rows, cols, a, nullptr, stream, true);
        case KLAS_F64: return rowops::softmax_t<double>(log_softmax, rows, cols, a, nullptr, stream, true);
        default: return fail(KLAS_ERR_INVALID, "softmax: dtype must be F16, BF16, F32 or F64");
    }
}

int launch_rowscale(int dtype, int col_major, uint64_t m, uint64_t n, const void *scale, void *b,
                    cudaStream_t stream) {
    if (m == 0 || n == 0) return KLAS_OK;
    if (!scale || !b) return fail(KLAS_ERR_INVALID, "rowscale: null pointer");
    const uint64_t total = m * n;
    uint64_t blocks = (total + rowops::THREADS - 1) / rowops::THREADS;
    if (blocks > 148 * 32) blocks = 148 * 32;
    switch (dtype) {
        case KLAS_F16:
            rowops::rowscale_kernel<__half><<<unsigned(blocks), rowops::THREADS, 0, stream>>>(
                static_cast<const __half *>(scale), static_cast<__half *>(b), m, n, col_major);
            break;
        case KLAS_F32:
            rowops::rowscale_kernel<float><<<unsigned(blocks), rowops::THREADS, 0, stream>>>(
                static_cast<const float *>(scale), static_cast<float *>(b), m, n, col_major);
            break;
        case KLAS_F64:
            rowops::rowscale_kernel<double><<<unsigned(blocks), rowops::THREADS, 0, stream>>>(
                static_cast<const double *>(scale), static_cast<double *>(b), m, n, col_major);
            break;
        default: return fail(KLAS_ERR_INVALID, "rowscale: dtype must be F16, F32 or F64");
    }
    return check_cuda(cudaGetLastError(), "rowscale_kernel launch");
}

int launch_reduce_sum(int dtype, uint64_t n, const void *a, void *out, void *scratch, size_t scratch_bytes,
                      cudaStream_t stream) {
    if (!out) return fail(KLAS_ERR_INVALID, "reduce: null result pointer");
    if (n > 0 && !a) return fail(KLAS_ERR_INVALID, "reduce: null data pointer");
    const size_t need = reduce_scratch_bytes(n);
    if (!scratch || scratch_bytes < need)
        return fail(KLAS_ERR_INVALID, "reduce: scratch of %zu bytes needed, %zu given", need, scratch_bytes);
    switch (dtype) {
        case KLAS_F16: return rowops::reduce_t<__half>(n, a, out, scratch, stream);
        case KLAS_F32: return rowops::reduce_t<float>(n, a, out, scratch, stream);
        case KLAS_F64: return rowops::reduce_t<double>(n, a, out, scratch, stream);
        case KLAS_U32: return rowops::reduce_t<uint32_t>(n, a, out, scratch, stream);
        case KLAS_U64: return rowops::reduce_t<uint64_t>(n, a, out, scratch, stream);
        default: return fail(KLAS_ERR_INVALID, "reduce: bad dtype");
    }
}

}  // namespace klas

// ---- vector softmax that allocates nothing ------------------------------------------------------
// Some callers have nowhere to get the per-chunk scratch of the vector softmax from: a process
// that handed all device memory to its own arena at start-up (a later cudaMalloc fails or
// fragments it), or a latency-critical loop that must not call cudaMalloc / cudaFree because
// both synchronise the whole device and stall every other stream.  For them the statistics live
// in the fixed array below, which is part of the loaded module, so no allocator is involved.
//
// The array holds one (max, sum) pair per chunk and so bounds the vector length:
// KLAS_B200_SOFTMAX_STATIC_MAX_COLS elements.  Every call on a device uses the same array, and it
// keeps what the last call left there.  Nothing in it has to start at zero -- the first launch
// writes every pair the second launch reads -- but two calls that overlap in time on one device
// (different streams or threads) would overwrite each other's pairs: serialise them.
namespace klas {
namespace rowops {

constexpr uint32_t STATIC_PARTS = 1024;
static_assert(uint64_t(STATIC_PARTS) * MIN_CHUNK == KLAS_B200_SOFTMAX_STATIC_MAX_COLS,
              "the documented limit is what the static array can hold");
static __device__ __align__(256) unsigned char g_static_softmax_scratch[STATIC_PARTS * 16];

constexpr int STATIC_MAX_DEVICES = 64;
static void *g_static_scratch_addr[STATIC_MAX_DEVICES];   // device address of the array, per device
static std::mutex g_static_scratch_mutex;

// Device address of the array on the current device.  Looked up once per device, with that
// device current, on the first call there (a symbol has one address per device).
static int static_scratch(void **out) {
    int dev = -1;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES)
        return fail(KLAS_ERR_UNSUPPORTED, "softmax_static: device ordinal %d beyond %d", dev, STATIC_MAX_DEVICES - 1);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_addr[dev]) {
        void *ptr = nullptr;
        const cudaError_t rc = cudaGetSymbolAddress(&ptr, g_static_softmax_scratch);
        if (rc != cudaSuccess)
            return fail(KLAS_ERR_CUDA, "softmax_static: cudaGetSymbolAddress: %s", cudaGetErrorString(rc));
        if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255u))
            return fail(KLAS_ERR_CUDA, "softmax_static: the scratch symbol resolved to %p", ptr);
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return KLAS_OK;
}

}  // namespace rowops
}  // namespace klas

extern "C" int klas_b200_softmax_static(int dtype, int log_softmax, uint64_t cols, void *a, void *stream) {
    using namespace klas;
    clear_error();
    if (cols == 0) return KLAS_OK;
    if (cols > KLAS_B200_SOFTMAX_STATIC_MAX_COLS)
        return fail(KLAS_ERR_TOO_LARGE,
                    "softmax_static: %llu elements, the built-in scratch holds the statistics of at most %llu; "
                    "use klas_b200_softmax with caller scratch",
                    (unsigned long long)cols, (unsigned long long)KLAS_B200_SOFTMAX_STATIC_MAX_COLS);
    const size_t need = softmax_scratch_bytes(1, cols);
    if (need > sizeof(rowops::g_static_softmax_scratch))   // cannot happen below the limit; kept as a guard
        return fail(KLAS_ERR_TOO_LARGE, "softmax_static: %zu bytes of statistics exceed the built-in %zu", need,
                    sizeof(rowops::g_static_softmax_scratch));
    void *scratch = nullptr;
    if (int rc = rowops::static_scratch(&scratch)) return rc;
    return launch_softmax(dtype, log_softmax, 1, cols, a, scratch, need, static_cast<cudaStream_t>(stream));
}
