// (min, +) matrix product on 16-bit path lengths, 0 standing for "no path":
//
//   C[i][j] = add( C[i][j], add_k mult(A[i][k], B[k][j]) )
//   mult(x, y) = 0 if x == 0 or y == 0, else (x + y) mod 2^16
//   add(x, y)  = the smaller non-zero one of x, y (0 if both are 0)
//
// the ring of dist/Kuiper_GraphDist.cu:9-24, whose kernel (one thread per output, operands
// read from global memory every step; dist/Kuiper_GraphDist.cu:26-45) squares a distance
// matrix: A = B, C updated in place.
//
// Same skeleton as the CUDA-core GEMM: 256 threads own a 128 x 128 (small problems: 64 x 64) tile
// of C, walk K in steps of 16 through double-buffered shared memory (A transposed), 8 x 8 (4 x 4)
// outputs per thread.  The
// ring is evaluated on 32-bit lanes with "no path" encoded as a huge value, so that one fused
// add-then-min instruction (__viaddmin_u32) is a whole ring step.  That encoding ignores the
// reference's wrap-around of x + y at 2^16, which cannot occur while every length is below
// 2^15.  A CTA that meets a larger operand while loading recomputes its tile with the ring
// written out literally, wrap-around included, so results equal the reference's bit for bit on
// any input.  C must not overlap A or B (other CTAs still read them).
#include <cuda_runtime.h>

#include "klas_internal.h"

namespace klas {
namespace minplus {

constexpr int THREADS = 256;
constexpr int BK = 16;
constexpr int PAD = 4;
constexpr uint32_t INF = 0x3fffffffu;   // INF + INF still fits 32 bits

struct Args {
    const uint16_t *A, *B;
    uint16_t *C;
    uint32_t M, N, K;
    uint32_t tiles_n;
};

// FAST: operands encoded (0 -> INF), accumulator = smallest sum so far.
// !FAST: operands raw, accumulator holds (length - 1) mod 2^16, so "no path" (0) is the largest
// value 0xffff and `min` is the ring's add.
template <bool FAST>
__device__ __forceinline__ uint32_t encode(uint16_t x) {
    if constexpr (FAST) return x ? uint32_t(x) : INF;
    return uint32_t(x);
}

template <bool FAST>
__device__ __forceinline__ void step(uint32_t &acc, uint32_t a, uint32_t b) {
    if constexpr (FAST) {
        acc = __viaddmin_u32(a, b, acc);
    } else {
        const uint32_t prod = (a == 0u || b == 0u) ? 0u : ((a + b) & 0xffffu);
        acc = min(acc, (prod - 1u) & 0xffffu);
    }
}

template <bool FAST>
__device__ __forceinline__ uint16_t finish(uint32_t acc, uint16_t old) {
    uint32_t sum;   // the ring sum over k, as a plain length (0 = no path)
    if constexpr (FAST) sum = acc >= 0x10000u ? 0u : acc;
    else sum = (acc + 1u) & 0xffffu;
    if (old == 0 || (sum != 0u && sum < old)) return uint16_t(sum);
    return old;
}

// One pass over K for this CTA's tile.  Returns (to every thread) whether an operand >= 2^15 was
// loaded, i.e. whether a FAST pass may have missed a wrap-around.
template <bool FAST, int BM, int BN>
__device__ __forceinline__ bool tile_pass(const Args &a, uint32_t m0, uint32_t n0, uint32_t (&acc)[BM / 16][BN / 16],
                                          uint32_t (&As)[2][BK][BM + PAD], uint32_t (&Bs)[2][BK][BN + PAD]) {
    constexpr int TM = BM / 16, TN = BN / 16;
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = FAST ? 0xffffffffu : 0xffffu;

    // A thread stages 8 consecutive k of one A row (the first 2 BM threads) and 8 consecutive
    // columns of one B row (the first 2 BN threads).
    const int ar = tid / 2, ak = (tid % 2) * 8;                    // A: BM rows x 16 k
    const int bk = tid / (BN / 8), bn = (tid % (BN / 8)) * 8;      // B: 16 k x BN columns
    const bool has_a = tid < 2 * BM, has_b = tid < 2 * BN;
    alignas(16) uint16_t ra[8];
    alignas(16) uint16_t rb[8];
    uint32_t big = 0;

    auto load_global = [&](uint32_t k0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) ra[e] = rb[e] = 0;
        const uint32_t gr = has_a ? m0 + ar : a.M;
        const uint16_t *ap = a.A + size_t(gr) * a.K + k0 + ak;
        if (gr < a.M && k0 + ak + 8 <= a.K && (reinterpret_cast<uintptr_t>(ap) & 15u) == 0) {
            const uint4 v = *reinterpret_cast<const uint4 *>(ap);
            *reinterpret_cast<uint4 *>(ra) = v;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) ra[e] = (gr < a.M && k0 + ak + e < a.K) ? ap[e] : uint16_t(0);
        }
        const uint32_t gk = has_b ? k0 + bk : a.K;
        const uint16_t *bp = a.B + size_t(gk) * a.N + n0 + bn;
        if (gk < a.K && n0 + bn + 8 <= a.N && (reinterpret_cast<uintptr_t>(bp) & 15u) == 0) {
            const uint4 v = *reinterpret_cast<const uint4 *>(bp);
            *reinterpret_cast<uint4 *>(rb) = v;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) rb[e] = (gk < a.K && n0 + bn + e < a.N) ? bp[e] : uint16_t(0);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) big |= uint32_t(ra[e] | rb[e]);
    };
    auto store_shared = [&](int buf) {
        if (has_a) {
#pragma unroll
            for (int e = 0; e < 8; ++e) As[buf][ak + e][ar] = encode<FAST>(ra[e]);
        }
        if (has_b) {
#pragma unroll
            for (int e = 0; e < 8; ++e) Bs[buf][bk][bn + e] = encode<FAST>(rb[e]);
        }
    };

    const uint32_t num_kb = (a.K + BK - 1) / BK;
    if (num_kb > 0) {
        load_global(0);
        store_shared(0);
    }
    __syncthreads();
    for (uint32_t kb = 0; kb < num_kb; ++kb) {
        const int buf = int(kb & 1u);
        const bool more = kb + 1 < num_kb;
        if (more) load_global((kb + 1) * BK);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            uint32_t av[TM], bv[TN];
#pragma unroll
            for (int g = 0; g < TM / 4; ++g)
                *reinterpret_cast<uint4 *>(&av[g * 4]) = *reinterpret_cast<const uint4 *>(&As[buf][k][g * (BM / 2) + ty * 4]);
#pragma unroll
            for (int g = 0; g < TN / 4; ++g)
                *reinterpret_cast<uint4 *>(&bv[g * 4]) = *reinterpret_cast<const uint4 *>(&Bs[buf][k][g * (BN / 2) + tx * 4]);
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) step<FAST>(acc[i][j], av[i], bv[j]);
        }
        if (more) store_shared(buf ^ 1);
        __syncthreads();
    }
    return __syncthreads_or(int(big >= 0x8000u)) != 0;
}

template <int BM, int BN>
__global__ void __launch_bounds__(THREADS, BM * BN <= 64 * 64 ? 4 : 2) minplus_kernel(const Args a) {
    constexpr int TM = BM / 16, TN = BN / 16;
    __shared__ __align__(16) uint32_t As[2][BK][BM + PAD];
    __shared__ __align__(16) uint32_t Bs[2][BK][BN + PAD];
    const uint32_t m0 = (blockIdx.x / a.tiles_n) * BM;
    const uint32_t n0 = (blockIdx.x % a.tiles_n) * BN;
    static_assert(BM % 64 == 0 && BN % 64 == 0 && 2 * BM <= THREADS && 2 * BN <= THREADS, "tile shape");
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    uint32_t acc[TM][TN];

    const bool may_wrap = tile_pass<true, BM, BN>(a, m0, n0, acc, As, Bs);
    if (may_wrap) tile_pass<false, BM, BN>(a, m0, n0, acc, As, Bs);

#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const uint32_t r = m0 + (i / 4) * (BM / 2) + ty * 4 + (i % 4);
        if (r >= a.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const uint32_t c = n0 + (j / 4) * (BN / 2) + tx * 4 + (j % 4);
            if (c >= a.N) continue;
            uint16_t *cp = a.C + size_t(r) * a.N + c;
            *cp = may_wrap ? finish<false>(acc[i][j], *cp) : finish<true>(acc[i][j], *cp);
        }
    }
}

}  // namespace minplus

int launch_minplus_u16(uint32_t m, uint32_t n, uint32_t k, const uint16_t *A, const uint16_t *B, uint16_t *C,
                       cudaStream_t stream) {
    using namespace minplus;
    if (m == 0 || n == 0) return KLAS_OK;
    if (!C || (k > 0 && (!A || !B))) return fail(KLAS_ERR_INVALID, "minplus: null matrix pointer");
    DeviceInfo info;
    if (int rc = device_info(&info)) return rc;
    Args a;
    a.A = A;
    a.B = B;
    a.C = C;
    a.M = m;
    a.N = n;
    a.K = k;
    // 128 x 128 tiles once they fill the machine twice over, 64 x 64 ones below that.
    const uint64_t big = uint64_t((m + 127) / 128) * ((n + 127) / 128);
    const bool use_big = big >= 2ull * uint64_t(info.sm_count);
    const uint32_t bm = use_big ? 128 : 64;
    a.tiles_n = (n + bm - 1) / bm;
    const uint64_t blocks = uint64_t((m + bm - 1) / bm) * a.tiles_n;
    if (blocks > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "minplus: too many tiles for one grid");
    if (use_big)
        minplus_kernel<128, 128><<<unsigned(blocks), THREADS, 0, stream>>>(a);
    else
        minplus_kernel<64, 64><<<unsigned(blocks), THREADS, 0, stream>>>(a);
    return check_cuda(cudaGetLastError(), "minplus_kernel launch");
}

}  // namespace klas
