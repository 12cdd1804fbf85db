// fp64 GEMM on the FP64 tensor cores:  C = A.B   or   C = beta*C + alpha*(A.B), row-major.
//
// sm_100a has one FP64 matrix instruction, the warp-level mma.sync m8n8k4 (tcgen05 has no FP64
// kind).  It runs at the same 64 FMA per clock per SM as scalar DFMA, but takes its operands as
// fragments spread over the warp, so a warp tile of 32 x 32 needs 8 doubles per lane per 4 steps
// of k for 4096 multiply-adds -- 0.5 bytes of shared-memory delivery per multiply-add, where the
// register-blocked scalar kernel (8 x 4 outputs per thread) needs 3 and is held to two thirds of
// the FP64 rate by the 128 bytes per clock a shared-memory pipe delivers.
//
// 256 threads (8 warps, 4 x 2) own a 128 x 64 tile of C; K advances in blocks of 16 through
// double-buffered shared memory (global -> registers -> shared, the next block's loads in
// flight during the multiply); rows of the A tile are padded to 20 doubles and rows of the B
// tile to 68 so that the fragment reads (8 rows x 4 k, 4 k x 8 columns per half-warp) touch
// every bank once.  Ragged edges are zero-filled on the way in and predicated on the way out.
// Each product is an IEEE fp64 fused multiply-add.
//
// Takes over the fp64 instances of dist/Klas_GEMM_SHMem.cu, dist/Klas_GEMM_Tiled.cu,
// dist/Klas_GEMM_BlockTiling1D.cu and dist/Klas_GEMM_Naive{1,2,3}.cu.
#include <cuda_runtime.h>

#include <atomic>

#include "klas_internal.h"

namespace klas {
namespace dmma {

constexpr int THREADS = 256;
constexpr int BM = 128, BN = 64, BK = 16;
constexpr int LDA_S = BK + 4;    // doubles per row of the A tile in shared memory
constexpr int LDB_S = BN + 4;    // doubles per row of the B tile
constexpr int WM = 32, WN = 32;  // warp tile
constexpr int MI = WM / 8, NJ = WN / 8;
constexpr size_t SMEM = sizeof(double) * 2 * (BM * LDA_S + BK * LDB_S);

struct Args {
    const double *A, *B;
    double *C;
    uint64_t M, N, K;
    uint64_t tiles_m, tiles_n;
    double alpha, beta;
    int scaled;
};

__device__ __forceinline__ void mma_m8n8k4(double (&c)[2], double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0, %1}, {%2}, {%3}, {%0, %1};"
                 : "+d"(c[0]), "+d"(c[1])
                 : "d"(a), "d"(b));
}

template <bool FAST>
__global__ void __launch_bounds__(THREADS, 2) gemm_dmma_kernel(const Args a) {
    extern __shared__ __align__(16) unsigned char dmma_smem[];
    double(*As)[BM][LDA_S] = reinterpret_cast<double(*)[BM][LDA_S]>(dmma_smem);
    double(*Bs)[BK][LDB_S] = reinterpret_cast<double(*)[BK][LDB_S]>(dmma_smem + sizeof(double) * 2 * BM * LDA_S);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = (warp >> 1) * WM, wn = (warp & 1) * WN;
    const int grp = lane >> 2, tig = lane & 3;

    const uint64_t per_batch = a.tiles_m * a.tiles_n;
    const uint64_t bidx = blockIdx.x / per_batch;
    const uint64_t rem = blockIdx.x - bidx * per_batch;
    const uint64_t m0 = (rem / a.tiles_n) * BM, n0 = (rem % a.tiles_n) * BN;
    const double *__restrict__ A = a.A + bidx * a.M * a.K;
    const double *__restrict__ B = a.B + bidx * a.K * a.N;
    double *C = a.C + bidx * a.M * a.N;

    double acc[MI][NJ][2];
#pragma unroll
    for (int i = 0; i < MI; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j) acc[i][j][0] = acc[i][j][1] = 0.0;

    // staging: A tile 128 x 16 = 1024 pairs of doubles (4 per thread), B tile 16 x 64 = 512 pairs (2 per thread)
    double2 ra[4], rb[2];
    auto load_global = [&](uint64_t k0) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * THREADS;
            const uint64_t r = m0 + idx / (BK / 2), kk = k0 + (idx % (BK / 2)) * 2;
            if (FAST) {
                ra[i] = *reinterpret_cast<const double2 *>(A + r * a.K + kk);
            } else {
                ra[i].x = (r < a.M && kk < a.K) ? A[r * a.K + kk] : 0.0;
                ra[i].y = (r < a.M && kk + 1 < a.K) ? A[r * a.K + kk + 1] : 0.0;
            }
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * THREADS;
            const uint64_t kr = k0 + idx / (BN / 2), c = n0 + (idx % (BN / 2)) * 2;
            if (FAST) {
                rb[i] = *reinterpret_cast<const double2 *>(B + kr * a.N + c);
            } else {
                rb[i].x = (kr < a.K && c < a.N) ? B[kr * a.N + c] : 0.0;
                rb[i].y = (kr < a.K && c + 1 < a.N) ? B[kr * a.N + c + 1] : 0.0;
            }
        }
    };
    auto store_shared = [&](int buf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * THREADS;
            *reinterpret_cast<double2 *>(&As[buf][idx / (BK / 2)][(idx % (BK / 2)) * 2]) = ra[i];
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = tid + i * THREADS;
            *reinterpret_cast<double2 *>(&Bs[buf][idx / (BN / 2)][(idx % (BN / 2)) * 2]) = rb[i];
        }
    };

    const uint64_t num_kb = (a.K + BK - 1) / BK;
    if (num_kb > 0) {
        load_global(0);
        store_shared(0);
    }
    __syncthreads();
    for (uint64_t kb = 0; kb < num_kb; ++kb) {
        const int buf = int(kb & 1);
        const bool more = kb + 1 < num_kb;
        if (more) load_global((kb + 1) * BK);
#pragma unroll
        for (int kk = 0; kk < BK; kk += 4) {
            double af[MI], bf[NJ];
#pragma unroll
            for (int i = 0; i < MI; ++i) af[i] = As[buf][wm + i * 8 + grp][kk + tig];
#pragma unroll
            for (int j = 0; j < NJ; ++j) bf[j] = Bs[buf][kk + tig][wn + j * 8 + grp];
#pragma unroll
            for (int i = 0; i < MI; ++i)
#pragma unroll
                for (int j = 0; j < NJ; ++j) mma_m8n8k4(acc[i][j], af[i], bf[j]);
        }
        if (more) store_shared(buf ^ 1);
        __syncthreads();
    }

    // fragment (i, j): row m0 + wm + 8 i + grp, columns n0 + wn + 8 j + 2 tig + {0, 1}
#pragma unroll
    for (int i = 0; i < MI; ++i) {
        const uint64_t r = m0 + wm + i * 8 + grp;
        if (!FAST && r >= a.M) continue;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const uint64_t c = n0 + wn + j * 8 + tig * 2;
            double *cp = C + r * a.N + c;
            if (FAST) {
                double2 out = make_double2(acc[i][j][0], acc[i][j][1]);
                if (a.scaled) {
                    const double2 old = *reinterpret_cast<const double2 *>(cp);
                    out.x = a.beta * old.x + a.alpha * out.x;
                    out.y = a.beta * old.y + a.alpha * out.y;
                }
                *reinterpret_cast<double2 *>(cp) = out;
            } else {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (c + e < a.N) {
                        double v = acc[i][j][e];
                        if (a.scaled) v = a.beta * cp[e] + a.alpha * v;
                        cp[e] = v;
                    }
                }
            }
        }
    }
}

}  // namespace dmma

int launch_gemm_dmma(uint32_t batch, uint64_t m, uint64_t n, uint64_t k, const double *alpha, const double *beta,
                     const void *A, const void *B, void *C, cudaStream_t stream) {
    using namespace dmma;
    Args a;
    a.A = static_cast<const double *>(A);
    a.B = static_cast<const double *>(B);
    a.C = static_cast<double *>(C);
    a.M = m;
    a.N = n;
    a.K = k;
    a.tiles_m = (m + BM - 1) / BM;
    a.tiles_n = (n + BN - 1) / BN;
    a.scaled = alpha != nullptr;
    a.alpha = alpha ? *alpha : 1.0;
    a.beta = beta ? *beta : 0.0;
    const uint64_t blocks = a.tiles_m * a.tiles_n * batch;
    if (blocks > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "gemm: too many tiles for one grid");
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        KLAS_TRY_CUDA(cudaFuncSetAttribute(gemm_dmma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
        KLAS_TRY_CUDA(cudaFuncSetAttribute(gemm_dmma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    const bool fast = m % BM == 0 && n % BN == 0 && k % BK == 0 && k > 0 &&
                      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u) == 0;
    if (fast)
        gemm_dmma_kernel<true><<<unsigned(blocks), THREADS, SMEM, stream>>>(a);
    else
        gemm_dmma_kernel<false><<<unsigned(blocks), THREADS, SMEM, stream>>>(a);
    return check_cuda(cudaGetLastError(), "gemm_dmma_kernel launch");
}

}  // namespace klas
