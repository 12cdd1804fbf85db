// CUDA-core GEMM for f32 / f64 / u32 / u64 (and bf16 storage with f32 math):
//   C = A.B            or            C = beta*C + alpha*(A.B)
// B200 has no tensor-core path for fp64 or for wrapping 32/64-bit integers, so
// these run as a register-blocked, shared-memory-staged kernel:
//   * a CTA of 256 threads owns a BM x BN tile of C and walks K in BK steps;
//   * global -> register -> shared staging is double buffered (the loads of
//     step i+1 are in flight while step i is multiplied);
//   * A is stored transposed in shared memory, and each thread's TM x TN
//     register tile is split into 16-byte groups that are BM/ (TM/VEC) apart,
//     so every shared read is a conflict-free 128-bit access;
//   * each output element is accumulated strictly in ascending k, starting
//     from 0 (the order of the reference's exact spec,
//     src/lib/kernel/gemm/Kuiper.Kernel.GEMM.BlockTiling2D.fsti:18-28);
//   * integer types wrap mod 2^32 / 2^64 (src/lib/kuiper/types/Kuiper.Scalars.fst:30-47).
// A "fast" instantiation (sizes multiples of the tile, 16-byte aligned rows)
// uses unpredicated vector loads; every other shape takes the predicated one.
//
// The strided entry point adds row strides, page strides (0 = one matrix shared by every page)
// and the element-wise hooks of the reference's general batched interface (mapA / mapB / comb of
// src/lib/kernel/gemm/Kuiper.Kernel.GEMM.SHMem.fsti:40-64 and ...BlockTiling2D.fsti:34-60) in
// separate instantiations, so the plain kernels keep their code.
//
// Takes over the work of dist/Klas_GEMM_SHMem.cu:9-72, dist/Klas_GEMM_Tiled.cu:8-54,
// dist/Klas_GEMM_BlockTiling1D.cu:8-69, dist/Klas_GEMM_BlockTiling2D.cu:9-214 and
// dist/Klas_GEMM_Naive{1,2,3}.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "klas_internal.h"

namespace klas {
namespace simt {

#ifndef KLAS_SIMT_BK8
#define KLAS_SIMT_BK8 8   // K depth of the large tile of the 8-byte types
#endif
constexpr int THREADS = 256;
constexpr int TX = 16;  // threads along N
constexpr int TY = 16;  // threads along M

template <typename S, typename T>
struct Conv {
    static __device__ __forceinline__ T load(S v) { return static_cast<T>(v); }
    static __device__ __forceinline__ S store(T v) { return static_cast<S>(v); }
};
template <>
struct Conv<__nv_bfloat16, float> {
    static __device__ __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 store(float v) {
        return __float2bfloat16_rn(v);
    }
};

// Blackwell issues fp32 multiply-adds two per instruction (fma.rn.f32x2 on a packed pair);
// a kernel made of scalar FFMAs is bound by instruction issue at ~60 % of the fp32 rate.  The
// f32 kernels therefore keep accumulators as packed pairs of neighbouring columns.  Each half
// is an ordinary IEEE fused multiply-add, so results equal the scalar formulation bit for bit.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    unsigned int a, b;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a);
    hi = __uint_as_float(b);
}
__device__ __forceinline__ void ffma2(unsigned long long &acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

template <typename T>
struct IsF32 {
    static constexpr bool value = false;
};
template <>
struct IsF32<float> {
    static constexpr bool value = true;
};

template <typename T>
struct Args {
    const void *A;
    const void *B;
    void *C;
    uint64_t M, N, K;
    uint64_t lda, ldb, ldc;   // row strides in elements
    uint64_t sa, sb, sc;      // page strides in elements
    uint64_t tiles_m, tiles_n;
    uint64_t k_chunk;         // K range of one CTA: K, or half of it when two CTAs share a tile
    uint32_t ksplits;         // CTAs per output tile along K: 1, or 2 (partial sums added atomically to a zeroed C)
    T alpha, beta;
    int scaled;  // 0: C = A.B   1: C = beta*C + alpha*A.B
    int map_a, map_b, comb;   // klas_map / klas_comb, read by the HOOKS instantiations only
};

// What one call asks for, as the launch helpers pass it down.
struct Problem {
    uint32_t batch;
    uint64_t m, n, k;
    uint64_t lda, ldb, ldc, sa, sb, sc;
    int map_a, map_b, comb;
    bool hooks;   // any map or a combine rule other than overwrite / axpby
    bool wide_acc = false;   // f32 storage, f64 arithmetic: the compensated-sum entry points
    bool split_k = false;    // the tile was chosen so that two CTAs per tile along K fill the machine
};

template <typename T>
__device__ __forceinline__ T map_val(T x, int op) {
    if constexpr (std::is_floating_point<T>::value) {
        switch (op) {
            case KLAS_MAP_SQRT: return sqrt(x);
            case KLAS_MAP_ABS: return fabs(x);
            case KLAS_MAP_SQUARE: return x * x;
            case KLAS_MAP_RELU: return x > T(0) ? x : T(0);
            case KLAS_MAP_NEG: return -x;
            default: return x;
        }
    } else {
        switch (op) {   // unsigned, wrapping: abs and relu are the identity, sqrt is refused by the host
            case KLAS_MAP_SQUARE: return x * x;
            case KLAS_MAP_NEG: return T(0) - x;
            default: return x;
        }
    }
}

template <typename T>
__device__ __forceinline__ T comb_val(T old, T acc, T alpha, T beta, int comb) {
    switch (comb) {
        case KLAS_COMB_NEW: return acc;
        case KLAS_COMB_MAX: return old > acc ? old : acc;
        case KLAS_COMB_MIN: return old < acc ? old : acc;
        case KLAS_COMB_MUL: return old * acc;
        case KLAS_COMB_RELU: return acc > T(0) ? acc : T(0);
        case KLAS_COMB_SCALED: return alpha * acc;
        default: return beta * old + alpha * acc;
    }
}

__device__ __forceinline__ void atomic_add(float *p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(double *p, double v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(uint32_t *p, uint32_t v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(uint64_t *p, uint64_t v) {
    atomicAdd(reinterpret_cast<unsigned long long *>(p), static_cast<unsigned long long>(v));
}

template <typename T, int N>
struct alignas(16) Vec {
    T v[N];
};

// S = storage type in global memory, T = arithmetic type.
// FAST: whole tiles, vector accesses without predicates.  EDGE (with FAST): the same vector accesses
// for shapes that are not multiples of the tile -- rows of A beyond M are read from the last row
// (their results are never stored), vectors of B beyond N or of either operand beyond K are zeros,
// stores are predicated per vector; needs N and K (and the strides) to be multiples of the vector.
template <typename S, typename T, int BM, int BN, int BK, bool FAST, bool HOOKS = false, bool EDGE = false>
__global__ void __launch_bounds__(THREADS, (BM * BN * sizeof(T) <= 64 * 64 * 4) ? 3 : 2) gemm_simt_kernel(const Args<T> a) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int TM = BM / TY;
    constexpr int TN = BN / TX;
    static_assert(TM % VEC == 0 && TN % VEC == 0, "thread tile must be whole 16-byte groups");
    constexpr int GM = TM / VEC;  // 16-byte groups per thread along M
    constexpr int GN = TN / VEC;
    constexpr int PAD = VEC;      // keeps rows 16-byte aligned
    constexpr int A_VECS = BM * BK / VEC;
    constexpr int B_VECS = BK * BN / VEC;
    constexpr int A_PER_THREAD = (A_VECS + THREADS - 1) / THREADS;
    constexpr int B_PER_THREAD = (B_VECS + THREADS - 1) / THREADS;
    static_assert(BK % VEC == 0 && BN % VEC == 0, "tile not vectorisable");

    // Dynamic shared memory: the deepest tiles need a little more than the 48 KiB static limit.
    extern __shared__ __align__(16) unsigned char simt_smem[];
    T(*As)[BK][BM + PAD] = reinterpret_cast<T(*)[BK][BM + PAD]>(simt_smem);  // transposed: [k][m]
    T(*Bs)[BK][BN + PAD] = reinterpret_cast<T(*)[BK][BN + PAD]>(simt_smem + sizeof(T) * 2 * BK * (BM + PAD));

    constexpr bool PACKED = IsF32<T>::value;   // f32: accumulate column pairs with fma.rn.f32x2
    const int tid = threadIdx.x;
    // Integer and fp64 tiles: a warp covers 4 x 8 thread tiles and each half-warp 2 x 8, so a
    // half-warp's 16-byte reads of a k-row touch 32 bytes of A and 128 bytes of B, one
    // shared-memory wavefront each (16 threads in a row touch 256 bytes of B: two wavefronts per
    // half-warp; measured 3 % slower for u32).  The packed f32 loop measured 1-2 % faster on
    // the plain 2 x 16 arrangement, which it keeps.
    static_assert(TX == 16 && TY == 16 && THREADS == 256, "warp layout assumes a 16 x 16 thread grid");
    const int tx = PACKED ? tid % TX : ((tid >> 5) & 1) * 8 + (tid & 7);
    const int ty = PACKED ? tid / TX : (tid >> 6) * 4 + ((tid >> 3) & 3);

    const uint64_t per_batch = a.tiles_m * a.tiles_n * a.ksplits;
    const uint64_t bidx = blockIdx.x / per_batch;
    const uint64_t rem = (blockIdx.x - bidx * per_batch) / a.ksplits;
    const uint64_t k_base = ((blockIdx.x - bidx * per_batch) % a.ksplits) * a.k_chunk;   // 0 unless K is split
    const uint64_t k_len = a.K - k_base < a.k_chunk ? a.K - k_base : a.k_chunk;
    const uint64_t m0 = (rem / a.tiles_n) * BM;
    const uint64_t n0 = (rem % a.tiles_n) * BN;

    const S *__restrict__ A = static_cast<const S *>(a.A) + bidx * a.sa;
    const S *__restrict__ B = static_cast<const S *>(a.B) + bidx * a.sb;
    S *C = static_cast<S *>(a.C) + bidx * a.sc;

    T acc[PACKED ? 1 : TM][PACKED ? 1 : TN];
    unsigned long long acc2[PACKED ? TM : 1][PACKED ? TN / 2 : 1];
#pragma unroll
    for (int i = 0; i < (PACKED ? 1 : TM); ++i)
#pragma unroll
        for (int j = 0; j < (PACKED ? 1 : TN); ++j) acc[i][j] = T(0);
#pragma unroll
    for (int i = 0; i < (PACKED ? TM : 1); ++i)
#pragma unroll
        for (int j = 0; j < (PACKED ? TN / 2 : 1); ++j) acc2[i][j] = 0ull;

    Vec<T, VEC> ra[A_PER_THREAD], rb[B_PER_THREAD];

    auto load_global = [&](uint64_t k0) {
#pragma unroll
        for (int i = 0; i < A_PER_THREAD; ++i) {
            const int idx = tid + i * THREADS;
            if (A_VECS % THREADS == 0 || idx < A_VECS) {
                const int r = idx / (BK / VEC);
                const int kv = (idx % (BK / VEC)) * VEC;
                if constexpr (FAST && EDGE) {
                    // every load is unconditional, from a clamped address, so the loads of a step still go
                    // out together; what lies beyond K is zeroed in registers
                    const uint64_t gr = m0 + r < a.M ? m0 + r : a.M - 1;
                    const bool inside = k0 + kv < a.K;
                    const uint64_t gk = inside ? k0 + kv : a.K - VEC;
                    ra[i] = *reinterpret_cast<const Vec<T, VEC> *>(reinterpret_cast<const T *>(A) + gr * a.lda + gk);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) ra[i].v[e] = inside ? ra[i].v[e] : T(0);
                } else if constexpr (FAST) {
                    ra[i] = *reinterpret_cast<const Vec<T, VEC> *>(
                        reinterpret_cast<const T *>(A) + (m0 + r) * a.lda + k_base + k0 + kv);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const uint64_t gr = m0 + r, gk = k0 + kv + e;
                        ra[i].v[e] = (gr < a.M && gk < a.K) ? Conv<S, T>::load(A[gr * a.lda + gk]) : T(0);
                    }
                }
                if constexpr (HOOKS) {
                    if (a.map_a != KLAS_MAP_ID) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) ra[i].v[e] = map_val<T>(ra[i].v[e], a.map_a);   // map(0) = 0 keeps the padding neutral
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < B_PER_THREAD; ++i) {
            const int idx = tid + i * THREADS;
            if (B_VECS % THREADS == 0 || idx < B_VECS) {
                const int kr = idx / (BN / VEC);
                const int nv = (idx % (BN / VEC)) * VEC;
                if constexpr (FAST && EDGE) {
                    const bool inside = k0 + kr < a.K && n0 + nv < a.N;
                    const uint64_t gk = k0 + kr < a.K ? k0 + kr : a.K - 1;
                    const uint64_t gc = n0 + nv < a.N ? n0 + nv : a.N - VEC;
                    rb[i] = *reinterpret_cast<const Vec<T, VEC> *>(reinterpret_cast<const T *>(B) + gk * a.ldb + gc);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) rb[i].v[e] = inside ? rb[i].v[e] : T(0);
                } else if constexpr (FAST) {
                    rb[i] = *reinterpret_cast<const Vec<T, VEC> *>(
                        reinterpret_cast<const T *>(B) + (k_base + k0 + kr) * a.ldb + n0 + nv);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        const uint64_t gk = k0 + kr, gc = n0 + nv + e;
                        rb[i].v[e] = (gk < a.K && gc < a.N) ? Conv<S, T>::load(B[gk * a.ldb + gc]) : T(0);
                    }
                }
                if constexpr (HOOKS) {
                    if (a.map_b != KLAS_MAP_ID) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) rb[i].v[e] = map_val<T>(rb[i].v[e], a.map_b);
                    }
                }
            }
        }
    };

    auto store_shared = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER_THREAD; ++i) {
            const int idx = tid + i * THREADS;
            if (A_VECS % THREADS == 0 || idx < A_VECS) {
                const int r = idx / (BK / VEC);
                const int kv = (idx % (BK / VEC)) * VEC;
#pragma unroll
                for (int e = 0; e < VEC; ++e) As[buf][kv + e][r] = ra[i].v[e];
            }
        }
#pragma unroll
        for (int i = 0; i < B_PER_THREAD; ++i) {
            const int idx = tid + i * THREADS;
            if (B_VECS % THREADS == 0 || idx < B_VECS) {
                const int kr = idx / (BN / VEC);
                const int nv = (idx % (BN / VEC)) * VEC;
                *reinterpret_cast<Vec<T, VEC> *>(&Bs[buf][kr][nv]) = rb[i];
            }
        }
    };

    const uint64_t num_kb = (k_len + BK - 1) / BK;   // k_len == K unless K is split (fast instantiations only)
    // Tile kb + 1 travels global -> registers -> shared memory while tile kb is multiplied.  EARLY:
    // its global reads are issued just before the barrier that ends step kb - 1 (they cannot be
    // scheduled past it) and its shared-memory stores come at the end of step kb, a whole step
    // between issue and use wherever the compiler puts the rest.  That is what the tiles that run
    // with few warps per SM need (f32 1024^3: 32.7 -> 36.1 TFLOP/s; fp64 4096^3 20.8 -> 23.1;
    // u64 +3 %).  The 128 x 128 tiles of the 4-byte types, two CTAs per SM, measured 4 % faster
    // with the reads at the top of step kb instead, and keep that.
    constexpr bool EARLY = sizeof(T) == 8 || BM * BN < 128 * 128;
    if (num_kb > 0) {
        load_global(0);
        store_shared(0);
        if (EARLY && num_kb > 1) load_global(BK);
    }
    __syncthreads();

    for (uint64_t kb = 0; kb < num_kb; ++kb) {
        const int buf = int(kb & 1);
        const bool more = kb + 1 < num_kb;
        if (!EARLY && more) load_global((kb + 1) * BK);
        // The packed f32 loop reads the operands of step k + 1 before the multiply-adds of step k
        // (in program order: it is fully unrolled); without that hint the compiler's schedule left
        // the FP32 pipe idle 30 % of the time (50.7 -> 58 TFLOP/s at 4096^3).  The other types
        // measured no better with it.
        Vec<T, VEC> avq[2][GM], bvq[2][GN];
        auto load_frag = [&](int slot, int k) {
#pragma unroll
            for (int g = 0; g < GM; ++g)
                avq[slot][g] = *reinterpret_cast<const Vec<T, VEC> *>(&As[buf][k][g * (BM / GM) + ty * VEC]);
#pragma unroll
            for (int g = 0; g < GN; ++g)
                bvq[slot][g] = *reinterpret_cast<const Vec<T, VEC> *>(&Bs[buf][k][g * (BN / GN) + tx * VEC]);
        };
        if constexpr (PACKED) load_frag(0, 0);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            Vec<T, VEC> avk[GM], bvk[GN];
            if constexpr (PACKED) {
                if (k + 1 < BK) load_frag((k + 1) & 1, k + 1);
            } else {
#pragma unroll
                for (int g = 0; g < GM; ++g)
                    avk[g] = *reinterpret_cast<const Vec<T, VEC> *>(&As[buf][k][g * (BM / GM) + ty * VEC]);
#pragma unroll
                for (int g = 0; g < GN; ++g)
                    bvk[g] = *reinterpret_cast<const Vec<T, VEC> *>(&Bs[buf][k][g * (BN / GN) + tx * VEC]);
            }
            Vec<T, VEC>(&av)[GM] = PACKED ? avq[k & 1] : avk;
            Vec<T, VEC>(&bv)[GN] = PACKED ? bvq[k & 1] : bvk;
            if constexpr (PACKED) {
                unsigned long long bp[TN / 2];
#pragma unroll
                for (int j = 0; j < TN / 2; ++j)
                    bp[j] = pack2(float(bv[(2 * j) / VEC].v[(2 * j) % VEC]), float(bv[(2 * j + 1) / VEC].v[(2 * j + 1) % VEC]));
#pragma unroll
                for (int i = 0; i < TM; ++i) {
                    const float ai = float(av[i / VEC].v[i % VEC]);
                    const unsigned long long a2 = pack2(ai, ai);
#pragma unroll
                    for (int j = 0; j < TN / 2; ++j) ffma2(acc2[i][j], a2, bp[j]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        acc[i][j] += av[i / VEC].v[i % VEC] * bv[j / VEC].v[j % VEC];
            }
        }
        if (more) store_shared(buf ^ 1);
        if (EARLY && kb + 2 < num_kb) load_global((kb + 2) * BK);
        __syncthreads();
    }

    // Accumulator (i, j) whichever way it is held.
    auto acc_at = [&](int i, int j) -> T {
        if constexpr (PACKED) {
            float lo, hi;
            unpack2(acc2[i][j / 2], lo, hi);
            return T((j & 1) ? hi : lo);
        } else {
            return acc[i][j];
        }
    };

    // Epilogue: thread-tile row i lives at m0 + (i/VEC)*(BM/GM) + ty*VEC + i%VEC.
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const uint64_t r = m0 + (i / VEC) * (BM / GM) + ty * VEC + (i % VEC);
#pragma unroll
        for (int g = 0; g < GN; ++g) {
            const uint64_t c = n0 + g * (BN / GN) + tx * VEC;
            if constexpr (FAST) {
                if constexpr (EDGE) {
                    if (r >= a.M || c >= a.N) continue;
                }
                Vec<T, VEC> out;
                T *cp = reinterpret_cast<T *>(C) + r * a.ldc + c;
                if (HOOKS && a.comb != KLAS_COMB_AXPBY) {
                    Vec<T, VEC> old{};
                    if (a.comb != KLAS_COMB_NEW && a.comb != KLAS_COMB_RELU && a.comb != KLAS_COMB_SCALED) old = *reinterpret_cast<const Vec<T, VEC> *>(cp);
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        out.v[e] = comb_val<T>(old.v[e], acc_at(i, g * VEC + e), a.alpha, a.beta, a.comb);
                } else if (a.scaled) {
                    const Vec<T, VEC> old = *reinterpret_cast<const Vec<T, VEC> *>(cp);
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        out.v[e] = a.beta * old.v[e] + a.alpha * acc_at(i, g * VEC + e);
                } else {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) out.v[e] = acc_at(i, g * VEC + e);
                    if (a.ksplits > 1) {
                        // two CTAs hold the two halves of this tile's sum: both add onto a zeroed C
                        // (two addends: the result does not depend on which arrives first)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) atomic_add(cp + e, out.v[e]);
                        continue;
                    }
                }
                *reinterpret_cast<Vec<T, VEC> *>(cp) = out;
            } else {
                if (r < a.M) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        if (c + e < a.N) {
                            S *cp = C + r * a.ldc + c + e;
                            T val = acc_at(i, g * VEC + e);
                            if (HOOKS && a.comb != KLAS_COMB_AXPBY) {
                                const T old = (a.comb != KLAS_COMB_NEW && a.comb != KLAS_COMB_RELU && a.comb != KLAS_COMB_SCALED) ? Conv<S, T>::load(*cp) : T(0);
                                val = comb_val<T>(old, val, a.alpha, a.beta, a.comb);
                            } else if (a.scaled) {
                                val = a.beta * Conv<S, T>::load(*cp) + a.alpha * val;
                            }
                            *cp = Conv<S, T>::store(val);
                        }
                    }
                }
            }
        }
    }
}

template <typename S, typename T, int BM, int BN, int BK, bool FAST, bool HOOKS, bool EDGE = false>
static int launch_kernel(const Args<T> &a, unsigned blocks, cudaStream_t stream) {
    constexpr int PAD = 16 / sizeof(T);
    constexpr size_t SMEM = sizeof(T) * 2 * BK * (BM + PAD + BN + PAD);
    if constexpr (SMEM > 48 * 1024) {
        static std::atomic<bool> configured[64] = {};
        int dev = 0;
        KLAS_TRY_CUDA(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            KLAS_TRY_CUDA(cudaFuncSetAttribute(gemm_simt_kernel<S, T, BM, BN, BK, FAST, HOOKS, EDGE>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
    }
    gemm_simt_kernel<S, T, BM, BN, BK, FAST, HOOKS, EDGE><<<blocks, THREADS, SMEM, stream>>>(a);
    return check_cuda(cudaGetLastError(), "gemm_simt_kernel launch");
}

template <typename S, typename T, int BM, int BN, int BK>
static int launch_cfg(const Problem &q, T alpha, T beta, int scaled, const void *A, const void *B, void *C,
                      cudaStream_t stream) {
    Args<T> a;
    a.A = A;
    a.B = B;
    a.C = C;
    a.M = q.m;
    a.N = q.n;
    a.K = q.k;
    a.lda = q.lda;
    a.ldb = q.ldb;
    a.ldc = q.ldc;
    a.sa = q.sa;
    a.sb = q.sb;
    a.sc = q.sc;
    a.tiles_m = (q.m + BM - 1) / BM;
    a.tiles_n = (q.n + BN - 1) / BN;
    a.alpha = alpha;
    a.beta = beta;
    a.scaled = scaled;
    a.map_a = q.map_a;
    a.map_b = q.map_b;
    a.comb = q.comb;
    const uint64_t blocks = a.tiles_m * a.tiles_n * q.batch;
    if (blocks > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "gemm: too many tiles for one grid");
    constexpr int VEC = 16 / sizeof(T);
    const bool same_storage = sizeof(S) == sizeof(T);
    const bool fast = same_storage && q.m % BM == 0 && q.n % BN == 0 && q.k % BK == 0 && q.k > 0 &&
                      (q.lda | q.ldb | q.ldc | q.sa | q.sb | q.sc) % VEC == 0 &&
                      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                        reinterpret_cast<uintptr_t>(C)) & 15u) == 0;
    a.ksplits = 1;
    a.k_chunk = q.k;
    if constexpr (sizeof(S) == sizeof(T)) {
        if (fast) {
            if (q.hooks) return launch_kernel<S, T, BM, BN, BK, true, true>(a, unsigned(blocks), stream);
            // Fewer tiles than half the SMs (the caller picked the tile for this): two CTAs per tile,
            // each summing half of K.  The halves are added atomically onto a zeroed C -- two addends,
            // so the result does not depend on their order; it differs from the unsplit sum by one
            // rounding (integers: not at all).
            DeviceInfo info;
            if (int rc = device_info(&info)) return rc;
            const int knob = debug_knob(KLAS_KNOB_SIMT_SPLIT_K);
            const bool can_split = !scaled && q.comb == KLAS_COMB_NEW && q.batch == 1 && q.k % (2 * BK) == 0 && q.k >= 8 * BK;
            const bool want_split = knob == 2 || (knob == 0 && q.split_k && 2 * blocks <= uint64_t(info.sm_count));
            if (can_split && want_split) {
                a.ksplits = 2;
                a.k_chunk = q.k / 2;
                KLAS_TRY_CUDA(cudaMemset2DAsync(C, q.ldc * sizeof(T), 0, q.n * sizeof(T), q.m, stream));
                return launch_kernel<S, T, BM, BN, BK, true, false>(a, unsigned(blocks * 2), stream);
            }
            return launch_kernel<S, T, BM, BN, BK, true, false>(a, unsigned(blocks), stream);
        }
        // Shapes that are not whole tiles but whose rows are whole vectors (1000^3, 4000^3, ...):
        // the vector path with guarded edges (f32 4000^3: 41 TFLOP/s element by element).
        const bool vector_rows = q.k > 0 && q.m > 0 && q.n % VEC == 0 && q.k % VEC == 0 &&
                                 (q.lda | q.ldb | q.ldc | q.sa | q.sb | q.sc) % VEC == 0 &&
                                 ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
                                   reinterpret_cast<uintptr_t>(C)) & 15u) == 0;
        if (vector_rows && !q.hooks) return launch_kernel<S, T, BM, BN, BK, true, false, true>(a, unsigned(blocks), stream);
    }
    if (q.hooks) return launch_kernel<S, T, BM, BN, BK, false, true>(a, unsigned(blocks), stream);
    return launch_kernel<S, T, BM, BN, BK, false, false>(a, unsigned(blocks), stream);
}

template <typename S, typename T>
static int launch_type(const Problem &q, T alpha, T beta, int scaled, const void *A, const void *B, void *C,
                       int sm_count, cudaStream_t stream) {
    const uint64_t m = q.m, n = q.n, batch = q.batch;
    if constexpr (sizeof(T) == 4) {
        // 128 x 128 tiles from 0.6 tiles per SM on (a part-filled single wave of large tiles beat
        // two waves of smaller ones: 51 against 41 TFLOP/s at 1536^3, 35 against 31 at 1280^3; at
        // 1024^3, 64 tiles, the 128 x 64 tile wins 33 to 22), 128 x 64 from 0.8 per SM, else 64 x 64.
        // The two smaller tiles walk K in steps of 32: they run one wave with few warps per SM,
        // where a barrier per step costs more (+6 % at 1024^3).
        const uint64_t big_tiles = ((m + 127) / 128) * ((n + 127) / 128) * batch;
        const uint64_t mid_tiles = ((m + 127) / 128) * ((n + 63) / 64) * batch;
        int pick = big_tiles * 10 >= uint64_t(sm_count) * 6 ? 2 : (mid_tiles * 10 >= uint64_t(sm_count) * 8 ? 1 : 0);
        // A small output with a long K is better served by the larger tiles (8 x 8 per thread:
        // fewer shared-memory bytes per multiply-add) run as two CTAs per tile along K than by
        // small tiles: the smallest of the two larger tiles that still leaves room for the second
        // CTA of every tile.  Measured, f32: 1024^3 59.6 -> 57.5 us, 1024 x 1024 x 4096 227 -> 195,
        // 768 x 768 x 2048 77.8 -> 66.5.
        Problem qs = q;
        // (Only whole tiles are split: a shape that would run the larger tile unsplit keeps the pick above.)
        auto whole = [&](uint64_t bm, uint64_t bn, uint64_t bk) { return m % bm == 0 && n % bn == 0 && q.k % (2 * bk) == 0; };
        if (q.k >= 512 && q.batch == 1 && !q.hooks && !scaled && debug_knob(KLAS_KNOB_SIMT_SPLIT_K) != 1) {
            if (2 * mid_tiles <= uint64_t(sm_count) && whole(128, 64, 32)) {
                pick = 1;
                qs.split_k = true;
            } else if (2 * big_tiles <= uint64_t(sm_count) && whole(128, 128, 16)) {
                pick = 2;
                qs.split_k = true;
            }
        }
        if (const int t = debug_knob(KLAS_KNOB_SIMT_TILE); t >= 0) pick = t;
        if (pick == 2) return launch_cfg<S, T, 128, 128, 16>(qs, alpha, beta, scaled, A, B, C, stream);
        if (pick == 1) return launch_cfg<S, T, 128, 64, 32>(qs, alpha, beta, scaled, A, B, C, stream);
        return launch_cfg<S, T, 64, 64, 32>(qs, alpha, beta, scaled, A, B, C, stream);
    } else {
        const uint64_t big_tiles = ((m + 127) / 128) * ((n + 63) / 64) * batch;
        if (big_tiles >= uint64_t(sm_count)) return launch_cfg<S, T, 128, 64, KLAS_SIMT_BK8>(q, alpha, beta, scaled, A, B, C, stream);
        return launch_cfg<S, T, 64, 32, 8>(q, alpha, beta, scaled, A, B, C, stream);
    }
}

static int dispatch(int dtype, const Problem &q, const void *alpha, const void *beta, const void *A, const void *B,
                    void *C, cudaStream_t stream) {
    DeviceInfo info;
    if (int rc = device_info(&info)) return rc;
    const int scaled = alpha != nullptr;
    switch (dtype) {
        case KLAS_F32:
            if (q.wide_acc)   // exact products and an f64 sum, rounded once: at least what a compensated f32 sum keeps
                return launch_type<float, double>(q, scaled ? double(*static_cast<const float *>(alpha)) : 1.0,
                                                  scaled ? double(*static_cast<const float *>(beta)) : 0.0, scaled, A, B, C,
                                                  info.sm_count, stream);
            return launch_type<float, float>(q, scaled ? *static_cast<const float *>(alpha) : 1.0f,
                                             scaled ? *static_cast<const float *>(beta) : 0.0f, scaled, A, B, C,
                                             info.sm_count, stream);
        case KLAS_F64: {
            // Plain contiguous products go to the FP64 tensor-core kernel (the KLAS_KNOB_F64_MODE knob
            // keeps them here); strided pages and the element-wise hooks stay on this kernel.
            const bool keep_simt = debug_knob(KLAS_KNOB_F64_MODE) == 1;
            const bool contiguous = q.lda == q.k && q.ldb == q.n && q.ldc == q.n && q.sa == q.m * q.k &&
                                    q.sb == q.k * q.n && q.sc == q.m * q.n;
            if (!q.hooks && contiguous && !keep_simt)
                return launch_gemm_dmma(q.batch, q.m, q.n, q.k, static_cast<const double *>(alpha),
                                        static_cast<const double *>(beta), A, B, C, stream);
            return launch_type<double, double>(q, scaled ? *static_cast<const double *>(alpha) : 1.0,
                                               scaled ? *static_cast<const double *>(beta) : 0.0, scaled, A, B, C,
                                               info.sm_count, stream);
        }
        case KLAS_U32:
            return launch_type<uint32_t, uint32_t>(q, scaled ? *static_cast<const uint32_t *>(alpha) : 1u,
                                                   scaled ? *static_cast<const uint32_t *>(beta) : 0u, scaled, A, B, C,
                                                   info.sm_count, stream);
        case KLAS_U64:
            return launch_type<uint64_t, uint64_t>(q, scaled ? *static_cast<const uint64_t *>(alpha) : 1ull,
                                                   scaled ? *static_cast<const uint64_t *>(beta) : 0ull, scaled, A, B, C,
                                                   info.sm_count, stream);
        case KLAS_BF16: {
            float fa = 1.0f, fb = 0.0f;
            if (scaled) {
                fa = __bfloat162float(*static_cast<const __nv_bfloat16 *>(alpha));
                fb = __bfloat162float(*static_cast<const __nv_bfloat16 *>(beta));
            }
            return launch_type<__nv_bfloat16, float>(q, fa, fb, scaled, A, B, C, info.sm_count, stream);
        }
        default:
            return fail(KLAS_ERR_INVALID, "gemm: dtype must be F32, F64, U32, U64 or BF16");
    }
}

}  // namespace simt

int launch_gemm_simt(int dtype, int layout, uint32_t batch, uint64_t m, uint64_t n, uint64_t k,
                     const void *alpha, const void *beta, const void *A, const void *B, void *C,
                     cudaStream_t stream) {
    if (layout != KLAS_RRR && layout != KLAS_CCC) return fail(KLAS_ERR_INVALID, "gemm: bad layout");
    if ((alpha == nullptr) != (beta == nullptr))
        return fail(KLAS_ERR_INVALID, "gemm: alpha and beta must both be NULL or both be set");
    if (m == 0 || n == 0 || batch == 0) return KLAS_OK;
    if (!C || (k > 0 && (!A || !B))) return fail(KLAS_ERR_INVALID, "gemm: null matrix pointer");
    if (layout == KLAS_CCC) {
        // Column-major C = A.B is the row-major product C^T = B^T.A^T on the same buffers.
        const void *t = A;
        A = B;
        B = t;
        const uint64_t tm = m;
        m = n;
        n = tm;
    }
    simt::Problem q{};
    q.batch = batch;
    q.m = m;
    q.n = n;
    q.k = k;
    q.lda = k;
    q.ldb = n;
    q.ldc = n;
    q.sa = m * k;
    q.sb = k * n;
    q.sc = m * n;
    q.map_a = q.map_b = KLAS_MAP_ID;
    q.comb = alpha ? KLAS_COMB_AXPBY : KLAS_COMB_NEW;
    q.hooks = false;
    return simt::dispatch(dtype, q, alpha, beta, A, B, C, stream);
}

int launch_gemm_simt_compensated(int dtype, int layout, uint64_t m, uint64_t n, uint64_t k, const void *A, const void *B,
                                 void *C, cudaStream_t stream) {
    if (dtype != KLAS_F32) return launch_gemm_simt(dtype, layout, 1, m, n, k, nullptr, nullptr, A, B, C, stream);
    if (layout != KLAS_RRR && layout != KLAS_CCC) return fail(KLAS_ERR_INVALID, "gemm: bad layout");
    if (m == 0 || n == 0) return KLAS_OK;
    if (!C || (k > 0 && (!A || !B))) return fail(KLAS_ERR_INVALID, "gemm: null matrix pointer");
    if (layout == KLAS_CCC) {
        const void *t = A;
        A = B;
        B = t;
        const uint64_t tm = m;
        m = n;
        n = tm;
    }
    simt::Problem q{};
    q.batch = 1;
    q.m = m;
    q.n = n;
    q.k = k;
    q.lda = k;
    q.ldb = n;
    q.ldc = n;
    q.sa = m * k;
    q.sb = k * n;
    q.sc = m * n;
    q.map_a = q.map_b = KLAS_MAP_ID;
    q.comb = KLAS_COMB_NEW;
    q.hooks = false;
    q.wide_acc = true;
    return simt::dispatch(dtype, q, nullptr, nullptr, A, B, C, stream);
}

int launch_gemm_simt_strided(int dtype, uint32_t batch, uint64_t m, uint64_t n, uint64_t k, const void *alpha,
                             const void *beta, const void *A, uint64_t lda, uint64_t stride_a, const void *B,
                             uint64_t ldb, uint64_t stride_b, void *C, uint64_t ldc, uint64_t stride_c, int map_a,
                             int map_b, int comb, cudaStream_t stream) {
    if (map_a < KLAS_MAP_ID || map_a > KLAS_MAP_NEG || map_b < KLAS_MAP_ID || map_b > KLAS_MAP_NEG)
        return fail(KLAS_ERR_INVALID, "gemm_strided: unknown operand map (%d, %d)", map_a, map_b);
    if (comb < KLAS_COMB_NEW || comb > KLAS_COMB_SCALED) return fail(KLAS_ERR_INVALID, "gemm_strided: unknown combine rule %d", comb);
    if (comb == KLAS_COMB_AXPBY && (!alpha || !beta))
        return fail(KLAS_ERR_INVALID, "gemm_strided: the axpby rule needs alpha and beta");
    if (comb == KLAS_COMB_SCALED && !alpha) return fail(KLAS_ERR_INVALID, "gemm_strided: the scaled rule needs alpha");
    if ((dtype == KLAS_U32 || dtype == KLAS_U64) && (map_a == KLAS_MAP_SQRT || map_b == KLAS_MAP_SQRT))
        return fail(KLAS_ERR_UNSUPPORTED, "gemm_strided: sqrt is not defined on the wrapping integer types");
    if (m == 0 || n == 0 || batch == 0) return KLAS_OK;
    if (!C || (k > 0 && (!A || !B))) return fail(KLAS_ERR_INVALID, "gemm_strided: null matrix pointer");
    if (lda < k || ldb < n || ldc < n) return fail(KLAS_ERR_INVALID, "gemm_strided: a row stride is shorter than the row");
    if (batch > 1 && stride_c < (m - 1) * ldc + n)
        return fail(KLAS_ERR_INVALID, "gemm_strided: pages of C overlap (stride_c too small)");
    simt::Problem q{};
    q.batch = batch;
    q.m = m;
    q.n = n;
    q.k = k;
    q.lda = lda;
    q.ldb = ldb;
    q.ldc = ldc;
    q.sa = stride_a;
    q.sb = stride_b;
    q.sc = stride_c;
    q.map_a = map_a;
    q.map_b = map_b;
    q.comb = comb;
    q.hooks = map_a != KLAS_MAP_ID || map_b != KLAS_MAP_ID || (comb != KLAS_COMB_AXPBY && comb != KLAS_COMB_NEW);
    // alpha / beta reach the kernel through the "scaled" arguments; SCALED needs alpha only
    static const double zero_words[1] = {0.0};   // 8 zero bytes: beta = 0 in every dtype
    const bool scaled = comb == KLAS_COMB_AXPBY || comb == KLAS_COMB_SCALED;
    const void *beta_arg = comb == KLAS_COMB_SCALED ? static_cast<const void *>(zero_words) : beta;
    return simt::dispatch(dtype, q, scaled ? alpha : nullptr, scaled ? beta_arg : nullptr, A, B, C, stream);
}

}  // namespace klas
