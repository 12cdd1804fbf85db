// CSR x dense SpMM:  C[rows x cols] = CSR(A) . B,  B and C row-major.
//
// The work list is (column slab, row) pairs, slab-major: all rows of the first
// slab of 32*VEC columns come before any row of the second, so that the part
// of B one slab touches (shared x 32*VEC elements) can stay resident in L2
// while the rows stream through.  Inside a slab rows are taken in the
// caller's `row_indices` order (longest first in the reference's drivers,
// test/spmm_common.c.inc:140-157), which keeps the tail of the grid short.
//
// One warp owns one pair.  Its lanes load 32 (value, column) pairs of the row
// with coalesced 4-byte loads, broadcast them with shuffles, and every lane
// gathers VEC consecutive elements of B's row `column` with one 16-byte load
// (the warp reads 512 contiguous bytes per nonzero), UNROLL nonzeros in flight.
// Products are added in CSR order starting from zero, exactly one FMA (or
// wrapping multiply-add) per nonzero per output element, and each C row
// segment is written once -- zeros for empty rows, as the reference does
// (dist/Klas_SPMM.cu:78-82,183-186).
//
// Takes over the work of dist/Klas_SPMM.cu:9-105 (u32), :112-209 (f32) and the
// 91 g_spmm_f32_* instances.
#include <cuda_runtime.h>

#include "klas_internal.h"

namespace klas {
namespace spmm {

constexpr int WARPS_PER_BLOCK = 8;
constexpr int UNROLL = 8;

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Pack {
    T v[VEC];
};

template <typename T>
__device__ __forceinline__ T mul_add(T a, T b, T c);
template <>
__device__ __forceinline__ float mul_add<float>(float a, float b, float c) {
    return fmaf(a, b, c);
}
template <>
__device__ __forceinline__ uint32_t mul_add<uint32_t>(uint32_t a, uint32_t b, uint32_t c) {
    return a * b + c;
}

struct Args {
    const void *elems;
    const uint32_t *col_ind;
    const uint32_t *row_off;
    const uint32_t *row_indices;
    const void *B;
    void *C;
    uint32_t rows, shared, cols;
    uint32_t slabs;
    uint64_t items;  // rows * slabs
};

template <typename T, int VEC>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32) spmm_kernel(const Args a) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t item = uint64_t(blockIdx.x) * WARPS_PER_BLOCK + (threadIdx.x >> 5);
    if (item >= a.items) return;
    const uint32_t slab = uint32_t(item / a.rows);
    const uint32_t ridx = uint32_t(item - uint64_t(slab) * a.rows);
    const uint32_t row = a.row_indices ? a.row_indices[ridx] : ridx;

    const T *__restrict__ elems = static_cast<const T *>(a.elems);
    const uint32_t *__restrict__ col_ind = a.col_ind;
    const T *__restrict__ B = static_cast<const T *>(a.B);
    T *__restrict__ C = static_cast<T *>(a.C);

    const uint32_t col = slab * (32 * VEC) + lane * VEC;
    const bool active = col < a.cols;  // cols is a multiple of VEC on this path
    const uint32_t begin = a.row_off[row];
    const uint32_t end = a.row_off[row + 1];

    Pack<T, VEC> acc;
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc.v[e] = T(0);

    for (uint32_t base = begin; base < end; base += 32) {
        const uint32_t idx = base + lane;
        uint32_t my_col = 0;
        T my_val = T(0);
        if (idx < end) {
            my_col = col_ind[idx];
            my_val = elems[idx];
        }
        const uint32_t cnt = min(32u, end - base);
        uint32_t j = 0;
        for (; j + UNROLL <= cnt; j += UNROLL) {
            Pack<T, VEC> bv[UNROLL];
            T av[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const uint32_t c = __shfl_sync(0xffffffffu, my_col, j + u);
                av[u] = __shfl_sync(0xffffffffu, my_val, j + u);
                if (active)
                    bv[u] = *reinterpret_cast<const Pack<T, VEC> *>(B + size_t(c) * a.cols + col);
            }
            if (active) {
#pragma unroll
                for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc.v[e] = mul_add<T>(av[u], bv[u].v[e], acc.v[e]);
            }
        }
        for (; j < cnt; ++j) {
            const uint32_t c = __shfl_sync(0xffffffffu, my_col, j);
            const T v = __shfl_sync(0xffffffffu, my_val, j);
            if (active) {
                const Pack<T, VEC> bv =
                    *reinterpret_cast<const Pack<T, VEC> *>(B + size_t(c) * a.cols + col);
#pragma unroll
                for (int e = 0; e < VEC; ++e) acc.v[e] = mul_add<T>(v, bv.v[e], acc.v[e]);
            }
        }
    }
    if (active) *reinterpret_cast<Pack<T, VEC> *>(C + size_t(row) * a.cols + col) = acc;
}

template <typename T>
static int launch_t(const Args &base, cudaStream_t stream) {
    Args a = base;
    const bool vec4 = a.cols % 4 == 0 &&
                      ((reinterpret_cast<uintptr_t>(a.B) | reinterpret_cast<uintptr_t>(a.C)) & 15u) == 0;
    const uint32_t slab_cols = vec4 ? 128u : 32u;
    a.slabs = (a.cols + slab_cols - 1) / slab_cols;
    a.items = uint64_t(a.rows) * a.slabs;
    const uint64_t blocks = (a.items + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK;
    if (blocks > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "spmm: too many work items");
    if (vec4)
        spmm_kernel<T, 4><<<unsigned(blocks), WARPS_PER_BLOCK * 32, 0, stream>>>(a);
    else
        spmm_kernel<T, 1><<<unsigned(blocks), WARPS_PER_BLOCK * 32, 0, stream>>>(a);
    return check_cuda(cudaGetLastError(), "spmm_kernel launch");
}

}  // namespace spmm

int launch_spmm(int dtype, uint32_t rows, uint32_t shared, uint32_t cols, uint32_t nnz,
                const void *elems, const uint32_t *col_ind, const uint32_t *row_off,
                const uint32_t *row_indices, const void *B, void *C, cudaStream_t stream) {
    if (dtype != KLAS_F32 && dtype != KLAS_U32)
        return fail(KLAS_ERR_INVALID, "spmm: dtype must be KLAS_F32 or KLAS_U32");
    if (rows == 0 || cols == 0) return KLAS_OK;
    if (!row_off || !C) return fail(KLAS_ERR_INVALID, "spmm: null row_off or C");
    if (nnz > 0 && (!elems || !col_ind || !B))
        return fail(KLAS_ERR_INVALID, "spmm: null elems, col_ind or B with nnz > 0");
    (void)shared;
    spmm::Args a{};
    a.elems = elems;
    a.col_ind = col_ind;
    a.row_off = row_off;
    a.row_indices = row_indices;
    a.B = B;
    a.C = C;
    a.rows = rows;
    a.shared = shared;
    a.cols = cols;
    return dtype == KLAS_F32 ? spmm::launch_t<float>(a, stream) : spmm::launch_t<uint32_t>(a, stream);
}

}  // namespace klas
