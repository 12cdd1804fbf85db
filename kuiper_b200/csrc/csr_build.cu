// Building a CSR matrix on the device: what the reference does on the host before every
// sparse product (test/spmm_common.c.inc:107-137 `sparsify_*`: scan the dense matrix row by row,
// keep the entries != 0 in column order; :139-157 `mk_row_indices`: rows sorted by decreasing
// length, the order the SpMM kernels schedule them in).
//
//   count   one warp per row counts its non-zeros (coalesced 128-byte reads), then one CTA
//           turns the counts into offsets in place; row_off[rows] is nnz.
//   fill    one warp per row again: ballot + prefix popcount place values and columns, in
//           ascending column order.
//   order   bitonic sort of 64-bit keys (~length << 32 | row): longest rows first, equal
//           lengths by ascending row -- a deterministic refinement of the reference's
//           (unstable) std::sort.  Runs of 2048 keys are sorted in shared memory; wider
//           compare-exchange steps go through global memory.
#include <cuda_runtime.h>

#include "klas_internal.h"

namespace klas {
namespace csr {

constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;

template <typename T>
__global__ void __launch_bounds__(THREADS) count_kernel(const T *__restrict__ dense, uint32_t rows, uint32_t cols,
                                                        uint32_t *row_off) {
    const uint32_t lane = threadIdx.x & 31u;
    for (uint64_t r = uint64_t(blockIdx.x) * WARPS + (threadIdx.x >> 5); r < rows; r += uint64_t(gridDim.x) * WARPS) {
        const T *row = dense + r * cols;
        uint32_t n = 0;
        for (uint32_t c = lane; c < cols; c += 32) n += row[c] != T(0) ? 1u : 0u;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) n += __shfl_xor_sync(0xffffffffu, n, off);
        if (lane == 0) row_off[r + 1] = n;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) row_off[0] = 0;
}

// In-place inclusive scan of v[1..n] by one CTA of 1024 threads: thread t owns a contiguous
// chunk, sums it, the CTA scans the 1024 sums, the thread rewrites its chunk.
__global__ void __launch_bounds__(1024) scan_kernel(uint32_t *v, uint32_t n) {
    __shared__ uint32_t sums[1024];
    const uint32_t per = (n + 1023u) / 1024u;
    const uint64_t lo = uint64_t(threadIdx.x) * per;
    const uint64_t hi = lo + per < n ? lo + per : n;
    uint32_t s = 0;
    for (uint64_t i = lo; i < hi; ++i) s += v[1 + i];
    sums[threadIdx.x] = s;
    __syncthreads();
    for (uint32_t d = 1; d < 1024; d <<= 1) {
        const uint32_t add = threadIdx.x >= d ? sums[threadIdx.x - d] : 0u;
        __syncthreads();
        sums[threadIdx.x] += add;
        __syncthreads();
    }
    uint32_t run = threadIdx.x ? sums[threadIdx.x - 1] : 0u;
    for (uint64_t i = lo; i < hi; ++i) {
        run += v[1 + i];
        v[1 + i] = run;
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS) fill_kernel(const T *__restrict__ dense, uint32_t rows, uint32_t cols,
                                                       const uint32_t *__restrict__ row_off, T *elems,
                                                       uint32_t *col_ind) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t below = (1u << lane) - 1u;
    for (uint64_t r = uint64_t(blockIdx.x) * WARPS + (threadIdx.x >> 5); r < rows; r += uint64_t(gridDim.x) * WARPS) {
        const T *row = dense + r * cols;
        uint32_t base = row_off[r];
        for (uint32_t c0 = 0; c0 < cols; c0 += 32) {
            const uint32_t c = c0 + lane;
            const T v = c < cols ? row[c] : T(0);
            const bool nz = v != T(0);
            const uint32_t mask = __ballot_sync(0xffffffffu, nz);
            if (nz) {
                const uint32_t pos = base + __popc(mask & below);
                elems[pos] = v;
                col_ind[pos] = c;
            }
            base += __popc(mask);
        }
    }
}

// ---- longest-first row order ---------------------------------------------------------------------
constexpr uint32_t RUN = 2048;   // keys sorted per CTA in shared memory (16 KiB)

__global__ void __launch_bounds__(THREADS) keys_kernel(const uint32_t *__restrict__ row_off, uint32_t rows, uint32_t padded,
                                                       unsigned long long *keys) {
    for (uint64_t i = uint64_t(blockIdx.x) * THREADS + threadIdx.x; i < padded; i += uint64_t(gridDim.x) * THREADS) {
        unsigned long long key = ~0ull;   // padding sorts last
        if (i < rows) key = (static_cast<unsigned long long>(~(row_off[i + 1] - row_off[i])) << 32) | i;
        keys[i] = key;
    }
}

__device__ __forceinline__ void compare_exchange(unsigned long long &a, unsigned long long &b, bool ascending) {
    if ((a > b) == ascending) {
        const unsigned long long t = a;
        a = b;
        b = t;
    }
}

// All steps (k, j) with j < RUN of the phases k_first .. k_last (powers of two), on this CTA's
// run of RUN keys.  For k <= RUN that is the whole phase.
__global__ void __launch_bounds__(1024) bitonic_local_kernel(unsigned long long *keys, uint32_t k_first, uint32_t k_last) {
    __shared__ unsigned long long s[RUN];
    const uint32_t base = blockIdx.x * RUN;
    for (uint32_t i = threadIdx.x; i < RUN; i += 1024) s[i] = keys[base + i];
    __syncthreads();
    for (uint32_t k = k_first; k <= k_last; k <<= 1) {
        for (uint32_t j = (k >> 1) < RUN ? (k >> 1) : (RUN >> 1); j > 0; j >>= 1) {
            for (uint32_t t = threadIdx.x; t < RUN / 2; t += 1024) {
                const uint32_t lo = ((t & ~(j - 1)) << 1) | (t & (j - 1));   // index with bit j clear
                const bool ascending = ((base + lo) & k) == 0;
                compare_exchange(s[lo], s[lo | j], ascending);
            }
            __syncthreads();
        }
    }
    for (uint32_t i = threadIdx.x; i < RUN; i += 1024) keys[base + i] = s[i];
}

// One step (k, j) with j >= RUN over the whole array.
__global__ void __launch_bounds__(THREADS) bitonic_global_kernel(unsigned long long *keys, uint32_t padded, uint32_t k, uint32_t j) {
    for (uint64_t t = uint64_t(blockIdx.x) * THREADS + threadIdx.x; t < padded / 2; t += uint64_t(gridDim.x) * THREADS) {
        const uint64_t lo = ((t & ~uint64_t(j - 1)) << 1) | (t & (j - 1));
        unsigned long long a = keys[lo], b = keys[lo | j];
        const bool ascending = (lo & k) == 0;
        if ((a > b) == ascending) {
            keys[lo] = b;
            keys[lo | j] = a;
        }
    }
}

__global__ void __launch_bounds__(THREADS) unpack_kernel(const unsigned long long *__restrict__ keys, uint32_t rows,
                                                         uint32_t *row_indices) {
    for (uint64_t i = uint64_t(blockIdx.x) * THREADS + threadIdx.x; i < rows; i += uint64_t(gridDim.x) * THREADS)
        row_indices[i] = uint32_t(keys[i]);
}

static uint32_t padded_rows(uint32_t rows) {
    uint64_t p = RUN;
    while (p < rows) p <<= 1;
    return uint32_t(p);
}

static unsigned grid_for(uint64_t items, uint64_t per_block) {
    const uint64_t want = (items + per_block - 1) / per_block;
    return unsigned(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
}

template <typename T>
static int count_t(uint32_t rows, uint32_t cols, const void *dense, uint32_t *row_off, cudaStream_t s) {
    count_kernel<T><<<grid_for(rows, WARPS), THREADS, 0, s>>>(static_cast<const T *>(dense), rows, cols, row_off);
    if (int rc = check_cuda(cudaGetLastError(), "csr count_kernel launch")) return rc;
    scan_kernel<<<1, 1024, 0, s>>>(row_off, rows);
    return check_cuda(cudaGetLastError(), "csr scan_kernel launch");
}

template <typename T>
static int fill_t(uint32_t rows, uint32_t cols, const void *dense, const uint32_t *row_off, void *elems,
                  uint32_t *col_ind, cudaStream_t s) {
    fill_kernel<T><<<grid_for(rows, WARPS), THREADS, 0, s>>>(static_cast<const T *>(dense), rows, cols, row_off,
                                                             static_cast<T *>(elems), col_ind);
    return check_cuda(cudaGetLastError(), "csr fill_kernel launch");
}

}  // namespace csr

int launch_csr_count(int dtype, uint32_t rows, uint32_t cols, const void *dense, uint32_t *row_off, cudaStream_t stream) {
    if (!row_off) return fail(KLAS_ERR_INVALID, "csr_count: null row_off");
    if (rows && cols && !dense) return fail(KLAS_ERR_INVALID, "csr_count: null matrix pointer");
    if (rows == 0xffffffffu) return fail(KLAS_ERR_TOO_LARGE, "csr_count: too many rows");
    switch (dtype) {
        case KLAS_F32: return csr::count_t<float>(rows, cols, dense, row_off, stream);
        case KLAS_U32: return csr::count_t<uint32_t>(rows, cols, dense, row_off, stream);
        default: return fail(KLAS_ERR_INVALID, "csr_count: dtype must be F32 or U32");
    }
}

int launch_csr_fill(int dtype, uint32_t rows, uint32_t cols, const void *dense, const uint32_t *row_off, void *elems,
                    uint32_t *col_ind, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return KLAS_OK;
    if (!dense || !row_off) return fail(KLAS_ERR_INVALID, "csr_fill: null pointer");
    // elems / col_ind may be NULL only for an all-zero matrix, which the kernel then never writes
    switch (dtype) {
        case KLAS_F32: return csr::fill_t<float>(rows, cols, dense, row_off, elems, col_ind, stream);
        case KLAS_U32: return csr::fill_t<uint32_t>(rows, cols, dense, row_off, elems, col_ind, stream);
        default: return fail(KLAS_ERR_INVALID, "csr_fill: dtype must be F32 or U32");
    }
}

size_t csr_row_order_scratch_bytes(uint32_t rows) { return rows ? size_t(csr::padded_rows(rows)) * 8 : 0; }

int launch_csr_row_order(uint32_t rows, const uint32_t *row_off, uint32_t *row_indices, void *scratch,
                         size_t scratch_bytes, cudaStream_t stream) {
    using namespace csr;
    if (rows == 0) return KLAS_OK;
    if (!row_off || !row_indices) return fail(KLAS_ERR_INVALID, "csr_row_order: null pointer");
    if (rows > 0x80000000u) return fail(KLAS_ERR_TOO_LARGE, "csr_row_order: more than 2^31 rows");
    const size_t need = csr_row_order_scratch_bytes(rows);
    if (!scratch || scratch_bytes < need || (reinterpret_cast<uintptr_t>(scratch) & 7u))
        return fail(KLAS_ERR_INVALID, "csr_row_order: %zu bytes of 8-byte aligned scratch needed, %zu given", need, scratch_bytes);
    const uint32_t padded = padded_rows(rows);
    auto *keys = static_cast<unsigned long long *>(scratch);
    keys_kernel<<<grid_for(padded, THREADS), THREADS, 0, stream>>>(row_off, rows, padded, keys);
    if (int rc = check_cuda(cudaGetLastError(), "csr keys_kernel launch")) return rc;
    const unsigned runs = padded / RUN;
    bitonic_local_kernel<<<runs, 1024, 0, stream>>>(keys, 2, RUN);
    if (int rc = check_cuda(cudaGetLastError(), "csr bitonic_local_kernel launch")) return rc;
    for (uint64_t k = 2ull * RUN; k <= padded; k <<= 1) {
        for (uint32_t j = uint32_t(k >> 1); j >= RUN; j >>= 1) {
            bitonic_global_kernel<<<grid_for(padded / 2, THREADS), THREADS, 0, stream>>>(keys, padded, uint32_t(k), j);
            if (int rc = check_cuda(cudaGetLastError(), "csr bitonic_global_kernel launch")) return rc;
        }
        bitonic_local_kernel<<<runs, 1024, 0, stream>>>(keys, uint32_t(k), uint32_t(k));
        if (int rc = check_cuda(cudaGetLastError(), "csr bitonic_local_kernel launch")) return rc;
    }
    unpack_kernel<<<grid_for(rows, THREADS), THREADS, 0, stream>>>(keys, rows, row_indices);
    return check_cuda(cudaGetLastError(), "csr unpack_kernel launch");
}

}  // namespace klas
