// CSR x dense SpMM:  C[rows x cols] = CSR(A) . B,  B and C row-major.
//
// What bounds it.  Every nonzero (r, c) needs the piece of B's row c that the
// lane group owns: with columns drawn at random no two nonzeros handled by one
// SM share a row of B, so nnz * 4 * cols bytes cross from L2 to the SMs whatever
// the schedule (8.6 GB at 131072^2, 64 nonzeros per row, 256 columns -- 25 times
// the bytes DRAM has to move).  The kernel is therefore built to keep as many
// 512-byte gathers in flight as the load/store path takes, and nothing else on
// the critical path:
//
//  * Work is cut by merge path: the sequence "row 0, its nonzeros, row 1, its
//    nonzeros, ..." (rows + nnz keys) is split into ranges of equal length, and
//    a row belongs to the range its row key falls in.  A warp walks a range, so
//    the (column, value) pairs it needs are ONE contiguous piece of the CSR
//    arrays: 32 pairs per coalesced load, fetched one step ahead, no
//    row_indices -> row_off -> col_ind chain per row.  Empty rows cost one key,
//    so long runs of them are spread over warps as well.
//  * Gathers go out in batches of eight per lane (16 bytes each, 512 contiguous
//    bytes per warp per nonzero).  A rotating register ring would keep more in
//    flight on paper, but a wait on a load's scoreboard is a wait for every load
//    that shares it; measured, rings of 8-16 ran at half the rate of batches.
//  * Column slabs of 128 are the outer loop (ranges are numbered slab-major), so
//    the part of B in use (shared x 512 bytes) stays L2-resident while the rows
//    stream by.
//  * A row longer than `long_row` keys is not kept on one warp: each range adds
//    the piece of the row that falls inside it to C with atomic adds (C's row
//    is zeroed by a small kernel launched first).  Every other row -- all of them
//    in the benchmark's matrix -- is summed by one warp in CSR order from zero
//    with one FMA (or wrapping multiply-add) per nonzero and stored once, which
//    is the reference's order (dist/Klas_SPMM.cu:78-82,183-186): results are bit
//    for bit those of the reference's kernel.
//
// `row_indices` (the reference's longest-row-first schedule,
// test/spmm_common.c.inc:140-157) only orders work there; ranges of equal work
// make it unnecessary and it is not read.  Every row is written, empty ones
// with zeros.
//
// Tried and measured on this GPU at the benchmark size, not kept: TMA copies of
// the row pieces into a shared-memory ring (cp.async.bulk, tiled 2-D boxes of
// one row, tile::gather4 boxes of four rows: all three 2.5 TB/s of gathers at
// 512 bytes per row and 4.3 TB/s at 1 KiB -- the copy engine spends about 60
// cycles per row whatever form the request takes); cp.async into shared memory
// (8.4 TB/s); register rings (7 TB/s).  Plain batches reach 19 TB/s in the
// gather-only probe below.
//
// Takes over the work of dist/Klas_SPMM.cu:9-105 (u32), :112-209 (f32) and the
// 91 g_spmm_f32_* instances.
#include <cstring>
#include <type_traits>
#include <cuda_runtime.h>

#include "klas_internal.h"

namespace klas {
namespace spmm {

constexpr int WARPS_PER_BLOCK = 8;
#ifndef KLAS_SPMM_UNROLL
#define KLAS_SPMM_UNROLL 8
#endif
constexpr int UNROLL = KLAS_SPMM_UNROLL;   // gathers in flight per lane (16-byte pieces; twice as many 8-byte ones)
// gathers in flight per lane by piece size: 8 pieces of 16 bytes (slabs of 128 columns) or 16 of
// 8 bytes (slabs of 64 columns: the same bytes in flight, a slab of B half as large)
template <int VEC>
constexpr int UNR = VEC == 2 ? 2 * UNROLL : UNROLL;
#ifndef KLAS_SPMM_MIN_BLOCKS
#define KLAS_SPMM_MIN_BLOCKS 4
#endif
constexpr int MIN_BLOCKS = KLAS_SPMM_MIN_BLOCKS;   // 32 warps per SM: the occupancy the gather-only probe is fastest at
constexpr uint32_t MIN_RANGE = 256;     // keys per range, at least
constexpr uint32_t MIN_LONG_ROW = 1024; // rows up to this length always stay on one warp
#ifndef KLAS_SPMM_RPW
#define KLAS_SPMM_RPW 2
#endif
constexpr int RANGES_PER_WARP = KLAS_SPMM_RPW;

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

template <typename T>
__device__ __forceinline__ T bits_as(uint32_t w);
template <>
__device__ __forceinline__ float bits_as<float>(uint32_t w) {
    return __uint_as_float(w);
}
template <>
__device__ __forceinline__ uint32_t bits_as<uint32_t>(uint32_t w) {
    return w;
}

struct Args {
    const void *elems;
    const uint32_t *col_ind;
    const uint32_t *row_off;
    const void *B;
    void *C;
    uint32_t rows, cols, nnz;
    uint32_t slabs;        // column slabs of 32 * VEC columns
    uint32_t nranges;      // merge-path ranges per slab
    uint64_t range_len;    // keys per range
    uint32_t long_row;     // rows with more nonzeros are cut at range boundaries
};

// First row r in [0, rows] with row_off[r] + r >= key (row_off[rows] + rows = the number of keys
// bounds every key asked for).  The 32 lanes probe 32 positions per step.
__device__ __forceinline__ uint32_t first_row_at_or_after(const uint32_t *__restrict__ row_off, uint32_t rows,
                                                          uint64_t key, uint32_t lane) {
    uint32_t lo = 0, hi = rows;
    while (lo < hi) {
        const uint32_t step = (hi - lo + 31) / 32;
        const uint64_t q = uint64_t(lo) + uint64_t(lane) * step;
        const bool below = q < hi && uint64_t(row_off[q]) + q < key;
        const uint32_t c = __popc(__ballot_sync(0xffffffffu, below));
        if (c == 0) {
            hi = lo;
        } else {
            const uint64_t next = uint64_t(lo) + uint64_t(c) * step;
            lo = lo + (c - 1) * step + 1;
            if (next < hi) hi = uint32_t(next);
        }
    }
    return lo;
}

// One row piece of C: stored (streaming: C is not read again) or, for a row assembled from pieces, added.
template <typename T, int VEC>
__device__ __forceinline__ void put_row(T *dst, const Pack<T, VEC> &acc, bool add) {
    if (add) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) atomicAdd(dst + e, acc.v[e]);
    } else if constexpr (VEC == 4) {
        uint4 w;
        memcpy(&w, &acc, 16);
        __stcs(reinterpret_cast<uint4 *>(dst), w);
    } else if constexpr (VEC == 2) {
        uint2 w;
        memcpy(&w, &acc, 8);
        __stcs(reinterpret_cast<uint2 *>(dst), w);
    } else {
        __stcs(dst, acc.v[0]);
    }
}

// One 16-byte (VEC = 4), 8-byte (VEC = 2) or 4-byte piece of row c of B: `Bbytes` points at this lane's columns of
// row 0, rows are `row_bytes` apart (one multiply-add with a 64-bit addend forms the address).
template <typename T, int VEC>
__device__ __forceinline__ Pack<T, VEC> gather(const char *Bbytes, uint32_t c, uint32_t row_bytes) {
    const char *p = Bbytes + uint64_t(c) * row_bytes;
    Pack<T, VEC> r;
    if constexpr (VEC == 4) {
        const uint4 w = __ldg(reinterpret_cast<const uint4 *>(p));
        memcpy(&r, &w, 16);
    } else if constexpr (VEC == 2) {
        const uint2 w = __ldg(reinterpret_cast<const uint2 *>(p));
        memcpy(&r, &w, 8);
    } else {
        r.v[0] = __ldg(reinterpret_cast<const T *>(p));
    }
    return r;
}

// What a warp carries along the nonzero stream of its range.
template <typename T, int VEC>
struct Stream {
    uint32_t p;        // next nonzero
    uint32_t r;        // row p belongs to
    uint32_t rend;     // end of row r
    uint32_t r_stop;   // rows [r, r_stop) are written by this range
    uint32_t rbase;    // ends[i] = row_off[rbase + i + 1]
    bool partial;      // row r's other nonzeros belong to other ranges: add instead of store
    Pack<T, VEC> acc;
};

// Writes every row that ends at the current nonzero (the row just completed and empty rows after it).
template <typename T, int VEC>
__device__ __forceinline__ void flush_finished_rows(Stream<T, VEC> &st, const uint32_t *__restrict__ row_off,
                                                    uint32_t rows, uint32_t cols, uint32_t *ends, T *Cc, bool active,
                                                    uint32_t lane) {
    while (st.r < st.r_stop && st.p == st.rend) {
        if (active) put_row<T, VEC>(Cc + size_t(st.r) * cols, st.acc, st.partial);
#pragma unroll
        for (int e = 0; e < VEC; ++e) st.acc.v[e] = T(0);
        ++st.r;
        st.partial = false;
        if (st.r - st.rbase == 32) {
            st.rbase = st.r;
            __syncwarp();
            ends[lane] = row_off[min(st.rbase + lane + 1, rows)];
            __syncwarp();
        }
        st.rend = ends[st.r - st.rbase];
    }
}

// One batch: UNROLL gathers go out, then their products are added in CSR order.  FULL: all UNROLL
// slots hold nonzeros; otherwise the first nb do.  The products are added in passes that end
// where a row ends -- one pass, without predicates, for the seven batches in eight in which no row
// does -- so the bulky row-end sequence exists once.  (Written out after each of the eight
// products it took the kernel from under 70 to over 110 registers; moved out of line it put the
// gathered pieces in local memory.)
__device__ __forceinline__ uint32_t word_of(const uint4 &q, int i) { return i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w; }

template <typename T, int VEC, bool FULL>
__device__ __forceinline__ void batch(Stream<T, VEC> &st, uint32_t nb, const uint32_t *cols_n, const T *vals_n,
                                      const char *Bbytes, uint32_t row_bytes, const uint32_t *__restrict__ row_off,
                                      uint32_t rows, uint32_t cols, uint32_t *ends, T *Cc, bool active, uint32_t lane) {
    constexpr int N = UNR<VEC>;
    static_assert(N % 4 == 0, "columns and values are read back four at a time");
    Pack<T, VEC> bv[N];
#pragma unroll
    for (int g = 0; g < N / 4; ++g) {
        const uint4 c = *reinterpret_cast<const uint4 *>(cols_n + 4 * g);
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (FULL || uint32_t(4 * g + q) < nb) bv[4 * g + q] = gather<T, VEC>(Bbytes, word_of(c, q), row_bytes);
    }
    if (FULL && st.rend - st.p > uint32_t(N)) {   // no row ends inside this batch
#pragma unroll
        for (int g = 0; g < N / 4; ++g) {
            const uint4 v = *reinterpret_cast<const uint4 *>(vals_n + 4 * g);
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int e = 0; e < VEC; ++e)
                    st.acc.v[e] = mul_add<T>(bits_as<T>(word_of(v, q)), bv[4 * g + q].v[e], st.acc.v[e]);
        }
        st.p += N;
        return;
    }
    uint32_t done = 0;
    do {
        const uint32_t left = nb - done, in_row = st.rend - st.p;
        const uint32_t seg = left < in_row ? left : in_row;   // nonzeros [done, done + seg) finish or stay inside the row
#pragma unroll
        for (int g = 0; g < N / 4; ++g) {
            const uint4 v = *reinterpret_cast<const uint4 *>(vals_n + 4 * g);
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (uint32_t(4 * g + q) - done < seg) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e)
                        st.acc.v[e] = mul_add<T>(bits_as<T>(word_of(v, q)), bv[4 * g + q].v[e], st.acc.v[e]);
                }
        }
        done += seg;
        st.p += seg;
        if (st.p == st.rend) flush_finished_rows<T, VEC>(st, row_off, rows, cols, ends, Cc, active, lane);
    } while (done < nb);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32, MIN_BLOCKS) spmm_kernel(const Args a) {
    // per warp: the 32 (column, value) pairs being worked on and the ends of 32 rows.  Lanes read
    // them back as broadcasts, four at a time, which takes a quarter of an instruction per
    // nonzero where shuffles took two.
    __shared__ __align__(16) uint32_t s_col[WARPS_PER_BLOCK][32];
    __shared__ __align__(16) T s_val[WARPS_PER_BLOCK][32];
    __shared__ uint32_t s_end[WARPS_PER_BLOCK][32];
    const uint32_t lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
    const uint32_t warp = blockIdx.x * WARPS_PER_BLOCK + wib;
    const uint32_t nwarps = gridDim.x * WARPS_PER_BLOCK;
    const T *__restrict__ elems = static_cast<const T *>(a.elems);
    const uint32_t *__restrict__ col_ind = a.col_ind;
    const uint32_t *__restrict__ row_off = a.row_off;
    const uint64_t total = uint64_t(a.nnz) + a.rows;
    const uint32_t all_ranges = a.slabs * a.nranges;   // the host keeps this below 2^32
    const uint32_t row_bytes = a.cols * uint32_t(sizeof(T));   // the host keeps this below 2^32
    uint32_t *my_cols = s_col[wib];
    T *my_vals = s_val[wib];
    uint32_t *my_ends = s_end[wib];

    for (uint32_t item = warp; item < all_ranges; item += nwarps) {
        const uint32_t slab = item / a.nranges;
        const uint32_t range = item - slab * a.nranges;
        const uint64_t ka = uint64_t(range) * a.range_len;
        const uint64_t kb = ka + a.range_len < total ? ka + a.range_len : total;
        if (ka >= kb) continue;
        const uint32_t col = slab * (32 * VEC) + lane * VEC;
        const bool active = col < a.cols;   // cols is a multiple of VEC on this path
        // inactive lanes (a ragged last slab) read column 0 and write nothing
        const char *Bbytes = static_cast<const char *>(a.B) + size_t(active ? col : 0) * sizeof(T);
        T *Cc = static_cast<T *>(a.C) + (active ? col : 0);

        // rows whose key lies in [ka, kb): [ra, rb)
        const uint32_t ra = first_row_at_or_after(row_off, a.rows, ka, lane);
        const uint32_t rb = first_row_at_or_after(row_off, a.rows, kb, lane);

        // The piece [ps, pe) of the nonzero stream this range sums and the rows [r, r_stop) it
        // writes.  The nonzero at position q of row x has key q + x + 1, so a row x that spans
        // key k is cut at position k - x - 1.
        Stream<T, VEC> st;
        st.r = ra;
        st.r_stop = rb;
        st.partial = false;
        uint32_t ps, pe;
        const uint32_t he = row_off[ra];   // end of row ra - 1 = start of row ra
        if (ra > 0 && uint64_t(he) + ra > ka && he - row_off[ra - 1] > a.long_row) {
            // row ra - 1 reaches into this range and is long: its nonzeros from key ka on are ours
            st.r = ra - 1;
            ps = uint32_t(ka - ra);
            st.partial = true;
        } else {
            ps = he;
        }
        if (rb > ra) {
            const uint32_t ls = row_off[rb - 1], le = row_off[rb];
            pe = le;   // the last row is summed to its end, unless it is long and leaves the range
            if (uint64_t(le) + rb > kb && le - ls > a.long_row) pe = uint32_t(kb - rb);
        } else if (st.partial) {
            st.r_stop = ra;
            const uint64_t cut = kb - ra;
            pe = cut < he ? uint32_t(cut) : he;
        } else {
            continue;   // the range lies inside a row that another range sums
        }

        st.rbase = st.r;
        __syncwarp();
        my_ends[lane] = row_off[min(st.rbase + lane + 1, a.rows)];
        __syncwarp();
        st.rend = my_ends[0];
#pragma unroll
        for (int e = 0; e < VEC; ++e) st.acc.v[e] = T(0);
        st.p = ps;
        flush_finished_rows<T, VEC>(st, row_off, a.rows, a.cols, my_ends, Cc, active, lane);   // leading empty rows

        // 32 (column, value) pairs per step, fetched one step ahead: the gathers depend on the columns
        uint32_t nxt_col = 0;
        T nxt_val = T(0);
        if (ps + lane < pe) {
            nxt_col = col_ind[ps + lane];
            nxt_val = elems[ps + lane];
        }
        for (uint32_t base = ps; base < pe; base += 32) {
            __syncwarp();   // the previous step's pairs have been read by every lane
            my_cols[lane] = nxt_col;
            my_vals[lane] = nxt_val;
            if (base + 32 + lane < pe) {
                nxt_col = col_ind[base + 32 + lane];
                nxt_val = elems[base + 32 + lane];
            }
            __syncwarp();
            const uint32_t cnt = min(32u, pe - base);
            uint32_t j0 = 0;
#pragma unroll 1
            for (; j0 + UNR<VEC> <= cnt; j0 += UNR<VEC>)
                batch<T, VEC, true>(st, UNR<VEC>, my_cols + j0, my_vals + j0, Bbytes, row_bytes, row_off, a.rows, a.cols,
                                    my_ends, Cc, active, lane);
            if (j0 < cnt)
                batch<T, VEC, false>(st, cnt - j0, my_cols + j0, my_vals + j0, Bbytes, row_bytes, row_off, a.rows, a.cols,
                                     my_ends, Cc, active, lane);
        }
        // a long row that goes on past the range: add what was summed, the next range continues
        if (st.r < st.r_stop && active) put_row<T, VEC>(Cc + size_t(st.r) * a.cols, st.acc, true);
    }
}

// Zeroes the rows of C whose sums are assembled with atomic adds (more than long_row nonzeros).
template <typename T>
__global__ void __launch_bounds__(256) zero_long_rows_kernel(const uint32_t *__restrict__ row_off, uint32_t rows, uint32_t cols,
                                                             uint32_t long_row, T *__restrict__ C) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp * 32 >= rows) return;
    const uint32_t r = warp * 32 + lane;
    const bool is_long = r < rows && row_off[r + 1] - row_off[r] > long_row;
    uint32_t m = __ballot_sync(0xffffffffu, is_long);
    while (m) {
        const uint32_t l = __ffs(m) - 1;
        m &= m - 1;
        T *dst = C + size_t(warp * 32 + l) * cols;
        for (uint32_t c = lane; c < cols; c += 32) dst[c] = T(0);
    }
}

// The gathers of spmm_kernel<float, 4> and nothing else: every warp walks a contiguous piece of
// the column-index stream once per slab of 128 columns and reads the 512-byte pieces of B's rows
// in batches of eight.  No values, no products, no C.  What this reaches is the rate the memory
// system delivers such gathers at, i.e. the ceiling the SpMM kernel is measured against.
template <int VEC>
__global__ void __launch_bounds__(WARPS_PER_BLOCK * 32, MIN_BLOCKS)
gather_probe_kernel(const uint32_t *__restrict__ col_ind, uint32_t nnz, const float *__restrict__ B, uint32_t cols,
                    uint32_t slabs, uint32_t per_warp, uint32_t *sink) {
    constexpr int N = UNR<VEC>;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * WARPS_PER_BLOCK + (threadIdx.x >> 5);
    const uint32_t row_bytes = cols * 4u;
    uint32_t x = 0;
    for (uint32_t slab = 0; slab < slabs; ++slab) {
        const uint64_t b64 = uint64_t(warp) * per_warp;
        const uint32_t begin = b64 < nnz ? uint32_t(b64) : nnz;
        const uint32_t end = nnz - begin < per_warp ? nnz : begin + per_warp;
        const uint32_t col = slab * (32 * VEC) + lane * VEC;
        const char *Bbytes = reinterpret_cast<const char *>(B + (col < cols ? col : 0));
        uint32_t nxt = begin + lane < end ? col_ind[begin + lane] : 0u;
        for (uint32_t base = begin; base < end; base += 32) {
            const uint32_t my_col = nxt;
            if (base + 32 + lane < end) nxt = col_ind[base + 32 + lane];
            const uint32_t cnt = min(32u, end - base);
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += N) {
                if (uint32_t(j0) < cnt) {
                    Pack<float, VEC> bv[N];
#pragma unroll
                    for (int u = 0; u < N; ++u) {
                        const uint32_t c = __shfl_sync(0xffffffffu, my_col, j0 + u);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) bv[u].v[e] = 0.f;
                        if (uint32_t(j0 + u) < cnt) bv[u] = gather<float, VEC>(Bbytes, c, row_bytes);
                    }
#pragma unroll
                    for (int u = 0; u < N; ++u)
#pragma unroll
                        for (int e = 0; e < VEC; ++e) x ^= __float_as_uint(bv[u].v[e]) + uint32_t(e);
                }
            }
        }
    }
    // keeps the loads alive; the comparison is not expected to hold
    if (x == 0x12345678u && sink) *sink = warp;
}

static int persistent_grid(const void *kernel, int *blocks) {
    DeviceInfo info;
    if (int rc = device_info(&info)) return rc;
    int per_sm = 0;
    KLAS_TRY_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, WARPS_PER_BLOCK * 32, 0));
    if (per_sm < 1) per_sm = 1;
    *blocks = per_sm * info.sm_count;
    return KLAS_OK;
}

// Elements per gathered piece: 4 (slabs of 128 columns), 2 (slabs of 64) or 1 (slabs of 32; any
// cols and alignment).  Slabs of 128 move the fewest instructions per byte and win whenever B has
// more than 64 columns -- also when a slab of B (shared x 512 bytes) outgrows L2: at 131072 rows
// of B the 64-column form, whose slab does fit, measured 0.66 ms against 0.50 (it streams the CSR
// arrays twice as often and issues twice the loads).  With 64 columns or fewer the narrower
// piece keeps every lane busy (131072^2 x 64: 0.17 against 0.22 ms).
static int piece_elems(uint32_t shared, uint32_t cols, const void *B, const void *C) {
    const uintptr_t both = reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C);
    const bool can4 = cols % 4 == 0 && (both & 15u) == 0, can2 = cols % 2 == 0 && (both & 7u) == 0;
    const int knob = debug_knob(KLAS_KNOB_SPMM_SLAB);
    if (knob == 128 && can4) return 4;
    if (knob == 64 && can2) return 2;
    if (knob == 32) return 1;
    (void)shared;
    if (cols <= 32) return 1;
    if (cols <= 64 || !can4) return can2 ? 2 : 1;
    return 4;
}

template <typename T>
static int launch_t(const Args &base, uint32_t shared, cudaStream_t stream) {
    Args a = base;
    const int vec = piece_elems(shared, a.cols, a.B, a.C);
    const uint32_t slab_cols = 32u * uint32_t(vec);
    a.slabs = (a.cols + slab_cols - 1) / slab_cols;
    int blocks = 0;
    if (int rc = persistent_grid(vec == 4   ? reinterpret_cast<const void *>(spmm_kernel<T, 4>)
                                 : vec == 2 ? reinterpret_cast<const void *>(spmm_kernel<T, 2>)
                                            : reinterpret_cast<const void *>(spmm_kernel<T, 1>), &blocks))
        return rc;
    const uint64_t total = uint64_t(a.nnz) + a.rows;
    // about RANGES_PER_WARP ranges per resident warp and slab, but no range shorter than MIN_RANGE keys
    uint64_t nranges = uint64_t(blocks) * WARPS_PER_BLOCK * RANGES_PER_WARP / a.slabs;
    const uint64_t most = (total + MIN_RANGE - 1) / MIN_RANGE;
    if (nranges > most) nranges = most;
    if (nranges < 1) nranges = 1;
    a.range_len = (total + nranges - 1) / nranges;
    a.nranges = uint32_t((total + a.range_len - 1) / a.range_len);
    const uint64_t half = a.range_len / 2;
    a.long_row = half > MIN_LONG_ROW ? (half > 0xffffffffull ? 0xffffffffu : uint32_t(half)) : MIN_LONG_ROW;
    const uint64_t items = uint64_t(a.slabs) * a.nranges;
    if (items > 0xffffffffull) return fail(KLAS_ERR_TOO_LARGE, "spmm: too many work items");
    if (uint64_t(a.cols) * sizeof(T) > 0xffffffffull) return fail(KLAS_ERR_TOO_LARGE, "spmm: rows of B of 4 GiB or more");
    const uint64_t want = (items + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK;
    const unsigned grid = unsigned(want < uint64_t(blocks) ? want : uint64_t(blocks));
    if (a.long_row < a.nnz) {   // a row longer than long_row can exist
        const unsigned zb = unsigned((uint64_t(a.rows) + 255) / 256);
        zero_long_rows_kernel<T><<<zb, 256, 0, stream>>>(a.row_off, a.rows, a.cols, a.long_row, static_cast<T *>(a.C));
        KLAS_TRY_CUDA(cudaGetLastError());
    }
    if (vec == 4)
        spmm_kernel<T, 4><<<grid, WARPS_PER_BLOCK * 32, 0, stream>>>(a);
    else if (vec == 2)
        spmm_kernel<T, 2><<<grid, WARPS_PER_BLOCK * 32, 0, stream>>>(a);
    else
        spmm_kernel<T, 1><<<grid, WARPS_PER_BLOCK * 32, 0, stream>>>(a);
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
    (void)row_indices;   // a scheduling hint in the reference; ranges of equal work replace it
    spmm::Args a{};
    a.elems = elems;
    a.col_ind = col_ind;
    a.row_off = row_off;
    a.B = B;
    a.C = C;
    a.rows = rows;
    a.cols = cols;
    a.nnz = nnz;
    return dtype == KLAS_F32 ? spmm::launch_t<float>(a, shared, stream) : spmm::launch_t<uint32_t>(a, shared, stream);
}

int launch_spmm_gather_probe(uint32_t shared, uint32_t cols, uint32_t nnz, const uint32_t *col_ind, const float *B,
                             cudaStream_t stream) {
    if (nnz == 0 || cols == 0) return KLAS_OK;
    if (!col_ind || !B) return fail(KLAS_ERR_INVALID, "gather_probe: null col_ind or B");
    const int vec = spmm::piece_elems(shared, cols, B, B);   // the piece size klas_b200_spmm would use
    if (vec == 1) return fail(KLAS_ERR_UNSUPPORTED, "gather_probe: cols must be even and B 8-byte aligned");
    int blocks = 0;
    if (int rc = spmm::persistent_grid(vec == 4 ? reinterpret_cast<const void *>(spmm::gather_probe_kernel<4>)
                                                : reinterpret_cast<const void *>(spmm::gather_probe_kernel<2>), &blocks))
        return rc;
    const uint32_t warps = uint32_t(blocks) * spmm::WARPS_PER_BLOCK;
    const uint32_t per_warp = (nnz + warps - 1) / warps;
    const uint32_t slabs = (cols + 32u * vec - 1) / (32u * vec);
    if (vec == 4)
        spmm::gather_probe_kernel<4><<<blocks, spmm::WARPS_PER_BLOCK * 32, 0, stream>>>(col_ind, nnz, B, cols, slabs, per_warp, nullptr);
    else
        spmm::gather_probe_kernel<2><<<blocks, spmm::WARPS_PER_BLOCK * 32, 0, stream>>>(col_ind, nnz, B, cols, slabs, per_warp, nullptr);
    return check_cuda(cudaGetLastError(), "gather_probe_kernel launch");
}

}  // namespace klas
