// Tensor-core GEMM for sm_100a: D = out( alpha * A.B + beta * C ).
//
// Persistent, warp-specialised CTAs walk a rasterised list of output tiles:
//   warp 0      TMA producer: streams 128x64 A tiles and 64-deep B tiles (bf16/f16,
//               128-byte swizzle) through a shared-memory ring;
//   warp 1      owns tensor memory and issues tcgen05.mma (K=16 per instruction) from
//               one thread; the fp32 accumulator lives in TMEM, double-buffered
//               (2 x 256 columns) so tile i+1's main loop overlaps tile i's epilogue;
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, the output rule (alpha /
//               beta / the old C / relu / the output type) and coalesced stores through a
//               swizzled 32-row x 128-byte staging block per warp; with an old C the block of C
//               comes in the same way, one block ahead (instantiations of their own, OLD_C).
// Three kernels:
//   single   one CTA per 128 x 256 (or 128 x 128, 128 x 64) tile over a 192 KiB ring cut into
//            4 x 48 (6 x 32, 8 x 24) KiB stages: small problems;
//   pair     two CTAs of a cluster share a 256 x 256 tile (cta_group::2): each stages
//            its own 128 rows of A and its own 128 columns of B (32 KiB per stage,
//            6 stages), the even CTA issues M=256 MMAs that read both CTAs' shared
//            memory, and each CTA drains its own 128 accumulator rows.  Per SM this
//            halves the B bytes staged and read per flop.  Every load is an ordinary
//            per-CTA TMA load; completion of the odd CTA's loads is counted on the even
//            CTA's barrier;
//   wide     two CTAs share a 512 x 256 tile (see gemm_umma_wide_kernel): problems that fill the
//            machine.
// The single and pair kernels can cut a tile's K range into parts (few tiles with a long K, or the
// tiles of a part-filled last round): the parts go to a workspace as f32 and splitk_reduce_kernel
// adds them in a fixed order.  The host picks kernel, tile width and split from the shape
// (launch_gemm_umma_strided).
// All hand-offs are mbarriers; every wait is bounded in time and a wait that
// gives up raises a status word and makes all roles drain and return.
//
// Takes over the work of the reference's wmma kernels, e.g.
// dist/Klas_GEMM_TensorCore2D.cu:16797-16936 (bf16 -> f32, 128x128x32 tiles),
// dist/Klas_GEMM_TensorCore2D_To.cu:9-176 (alpha/beta, bf16 out) and
// dist/Klas_GEMM_TensorCore.cu:9-115 (C += A.B).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "klas_internal.h"
#include "ptx_sm100.cuh"

namespace klas {
namespace umma {

constexpr uint32_t BM = 128;  // accumulator rows per CTA (= TMEM lanes)
constexpr uint32_t BN = 256;  // accumulator columns per tile
constexpr uint32_t BK = 64;   // 64 x 2 bytes = one 128-byte swizzle row
constexpr uint32_t UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;
constexpr uint32_t B_CHUNK_BYTES = 64 * BK * 2;  // one 64-column slab of a row-major B tile
constexpr uint32_t ACC_STAGES = 2;
constexpr uint32_t TMEM_COLS = ACC_STAGES * BN;  // 512 = all of tensor memory
constexpr uint32_t NUM_THREADS = 192;
constexpr uint32_t NUM_EPI_WARPS = 4;
#ifndef KLAS_XFORM_WARPS
#define KLAS_XFORM_WARPS 4
#endif
constexpr uint32_t XFORM_WARPS = KLAS_XFORM_WARPS;   // extra warps of the kernels that map A / B in shared memory
constexpr uint32_t XFORM_THREADS = XFORM_WARPS * 32;
constexpr uint32_t XFULL_OFFSET = 192;    // byte offset of the "operands mapped" barriers in the barrier block
constexpr uint32_t BARRIER_BYTES = 256;
constexpr uint32_t MAX_STAGES = 8;        // barrier slots per ring (the 128 x 64 tile runs eight 24 KiB stages)
constexpr uint32_t RING_BYTES = 192 * 1024;            // operand ring of every tile shape
constexpr uint32_t EPI_BLOCK_BYTES = 32 * 128;         // output staging block of one epilogue warp: 32 rows x 128 bytes
constexpr uint32_t DEFAULT_RASTER_GROUP = 8;  // tile columns swept together for L2 reuse
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

#ifndef KLAS_PAIR_STAGES
#define KLAS_PAIR_STAGES 6
#endif
#ifndef KLAS_PAIR_RELEASE
#define KLAS_PAIR_RELEASE 1
#endif

template <bool PAIR>
struct Shape {
    static constexpr uint32_t CTAS = PAIR ? 2 : 1;
    static constexpr uint32_t TILE_M = BM * CTAS;     // rows of one tile of the CTA group
    static constexpr uint32_t B_COLS = BN / CTAS;     // B columns staged by each CTA
    static constexpr uint32_t STAGES = PAIR ? KLAS_PAIR_STAGES : 4;
    // Consecutive stages released by one tcgen05.commit.  A commit costs the issuing thread
    // about as much as two MMAs, so the pair tiles free their stages two at a time.
    static constexpr uint32_t RELEASE_GROUP = PAIR ? KLAS_PAIR_RELEASE : 1;
    static constexpr uint32_t B_STAGE_BYTES = B_COLS * BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static_assert(STAGES * STAGE_BYTES == RING_BYTES && STAGES <= MAX_STAGES, "ring layout");
    static constexpr uint32_t SMEM_BYTES = RING_BYTES + NUM_EPI_WARPS * EPI_BLOCK_BYTES + BARRIER_BYTES + 1024;
};

// First failing wait of the most recent launches on this device (0 = none).
__device__ int g_umma_status;
// Host-visible mirror of the word (a mapped, pinned int; null until the first launch on the
// device): a blocking caller that has just synchronised reads it with a plain load instead of
// paying a device round trip per call.
__device__ int *g_umma_host_flag;


struct Params {
    const void *C;
    void *D;
    uint32_t M, N, K, batch;
    uint64_t ldd, sd;      // C / D: elements between rows, elements between pages
    uint32_t tiles_m, tiles_n, num_tiles, num_kb;
    uint32_t tile_n;       // columns per tile of the single-CTA kernel: 256, or 128 / 64 for small outputs
    uint32_t stages, stage_bytes;   // single-CTA kernel: ring depth and bytes per stage (4 x 48, 6 x 32 or 8 x 24 KiB)
    // K split (single-CTA and pair kernels): a tile's K range is cut into `ksplit` parts of `kb_per`
    // K blocks, one work item each; `num_work` = num_tiles * ksplit.  Part q of page b writes its
    // f32 partial product as page b * ksplit + q of D (a workspace then; a second kernel adds the parts).
    uint32_t ksplit, kb_per, num_work;
    uint32_t tile0;        // first tile of this launch (single-CTA and pair kernels): a launch may cover the tail of the tile list only
    float alpha, beta;
    uint32_t idesc;
    uint32_t b_row_major;  // 1: B is K x N (N contiguous) -> MN-major operand
    uint32_t raster_group; // tile columns swept together before moving down the rows
    uint32_t in_bf16;      // element type of A and B: 1 = bf16, 0 = f16
    uint32_t map_a, map_b; // element-wise maps applied to the staged operands (klas_map)
    uint32_t comb;         // how the accumulator meets the old output value (klas_comb)
    int *status;           // optional caller-visible copy of the status word
};

enum WaitSite : int {
    SITE_PRODUCER_EMPTY = 0x11,
    SITE_MMA_FULL = 0x21,
    SITE_MMA_TMEM_EMPTY = 0x22,
    SITE_EPI_TMEM_FULL = 0x31,
    SITE_XFORM_FULL = 0x41,
};

struct Ctl {
    volatile int *abort_flag;  // shared memory, per CTA
    int *user_status;
};

// Spins on an mbarrier phase for at most WAIT_LIMIT_NS.  On give-up records
// `site` in the status words and returns false; also returns false early when
// another role of this CTA (or another CTA) has already given up.
// `backoff_ns` > 0 marks the roles whose waits are long (epilogue, producer): they poll with a
// suspend-time hint of 32 x that many nanoseconds, so the hardware parks them until the phase
// completes instead of their spinning (or sleeping past the completion) while the tensor pipe works:
// fewer instructions, less power under the board's cap.
// CLUSTER_ACQUIRE: the phase is completed by arrivals from the other CTA of the pair that
// publish shared-memory writes of that CTA.
template <bool CLUSTER_ACQUIRE = false>
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const Ctl &ctl,
                                             int site, uint64_t limit_ns = WAIT_LIMIT_NS,
                                             uint32_t backoff_ns = 0) {
    auto poll = [&] {
        if (CLUSTER_ACQUIRE) return ptx::mbar_try_wait_cluster(bar, parity);
        return backoff_ns ? ptx::mbar_try_wait_hint(bar, parity, backoff_ns * 32u) : ptx::mbar_try_wait(bar, parity);
    };
    if (poll()) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (poll()) return true;
        if ((++spins & 0x3F) == 0) {
            if (*ctl.abort_flag != 0) return false;
            if (*reinterpret_cast<volatile int *>(&g_umma_status) != 0) {
                *ctl.abort_flag = 1;
                return false;
            }
            if (ptx::globaltimer_ns() - t0 > limit_ns) {
                *ctl.abort_flag = 1;
                atomicCAS(&g_umma_status, 0, site);
                if (ctl.user_status) atomicCAS(ctl.user_status, 0, site);
                if (int *hf = g_umma_host_flag) {
                    *reinterpret_cast<volatile int *>(hf) = site;
                    __threadfence_system();
                }
                __threadfence();
                return false;
            }
        }
    }
}

__device__ __forceinline__ void decode_tile(uint32_t t, const Params &p, uint32_t &b, uint32_t &tm,
                                            uint32_t &tn) {
    const uint32_t per_batch = p.tiles_m * p.tiles_n;
    b = t / per_batch;
    const uint32_t r = t - b * per_batch;
    const uint32_t group_tiles = p.raster_group * p.tiles_m;
    const uint32_t g = r / group_tiles;
    const uint32_t first_n = g * p.raster_group;
    const uint32_t width = min(p.raster_group, p.tiles_n - first_n);
    const uint32_t in = r - g * group_tiles;
    tm = in / width;
    tn = first_n + in % width;
}

// One unit of the persistent loops of the single-CTA and pair kernels: a tile, or with a K split
// one part of a tile's K blocks.  The parts of a tile are consecutive work items, so they run
// at the same time on neighbouring CTA groups.
struct WorkItem {
    uint32_t tile, part, kb0, kb1;
    __device__ __forceinline__ WorkItem(uint32_t w, const Params &p) {
        const uint32_t local = p.ksplit > 1 ? w / p.ksplit : w;
        tile = p.tile0 + local;
        part = w - local * p.ksplit;
        kb0 = part * p.kb_per;
        kb1 = min(kb0 + p.kb_per, p.num_kb);
    }
};

template <typename T>
struct OutTraits;
template <>
struct OutTraits<float> {
    static __device__ __forceinline__ float to_f32(float v) { return v; }
    static __device__ __forceinline__ float from_f32(float v) { return v; }
};
template <>
struct OutTraits<__half> {
    static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <>
struct OutTraits<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) {
        return __bfloat162float(v);
    }
    static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) {
        return __float2bfloat16_rn(v);
    }
};

// ---- element-wise hooks ----------------------------------------------------------------------
// Pre-maps of the staged operands and the rule that merges the accumulator into the output:
// the run-time counterparts of the map / combine functions the reference inlines into its
// tensor-core kernels at extraction time (include/kuiper/tensorcores.h:30-59, KPR_LOAD_MAP and
// KPR_STORE_COMB).  A map is evaluated in f32 on the 16-bit element and rounded back once.
// Every map sends 0 to 0, so the zero fill of ragged K edges stays neutral.
template <uint32_t OP>
__device__ __forceinline__ float map_f32(float x) {
    if constexpr (OP == KLAS_MAP_SQRT) {
        float r;
        // <= 1 ulp of f32 before the 16-bit rounding; f32 subnormals (only bf16 inputs below
        // 1.2e-38 convert to those) count as 0
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
        return r;
    } else if constexpr (OP == KLAS_MAP_ABS) {
        return fabsf(x);
    } else if constexpr (OP == KLAS_MAP_SQUARE) {
        return x * x;
    } else if constexpr (OP == KLAS_MAP_RELU) {
        return fmaxf(x, 0.0f);
    } else if constexpr (OP == KLAS_MAP_NEG) {
        return -x;
    } else {
        return x;
    }
}

// Two packed 16-bit elements at a time.  Sign manipulations are bit operations, max and the
// (exactly representable in f32, hence once-rounded) square are native packed instructions;
// only sqrt goes through f32 and the special-function unit.
template <bool BF16, uint32_t OP>
__device__ __forceinline__ uint32_t map_pair(uint32_t w) {
    if constexpr (OP == KLAS_MAP_ABS) {
        return w & 0x7fff7fffu;
    } else if constexpr (OP == KLAS_MAP_NEG) {
        return w ^ 0x80008000u;
    } else if constexpr (BF16) {
        const __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162 *>(&w);
        __nv_bfloat162 r;
        if constexpr (OP == KLAS_MAP_RELU) {
            r = __hmax2(x, __floats2bfloat162_rn(0.0f, 0.0f));
        } else if constexpr (OP == KLAS_MAP_SQUARE) {
            r = __hmul2(x, x);
        } else {
            const float2 f = __bfloat1622float2(x);
            r = __floats2bfloat162_rn(map_f32<OP>(f.x), map_f32<OP>(f.y));
        }
        return *reinterpret_cast<const uint32_t *>(&r);
    } else {
        const __half2 x = *reinterpret_cast<const __half2 *>(&w);
        __half2 r;
        if constexpr (OP == KLAS_MAP_RELU) {
            r = __hmax2(x, __floats2half2_rn(0.0f, 0.0f));
        } else if constexpr (OP == KLAS_MAP_SQUARE) {
            r = __hmul2(x, x);
        } else {
            const float2 f = __half22float2(x);
            r = __floats2half2_rn(map_f32<OP>(f.x), map_f32<OP>(f.y));
        }
        return *reinterpret_cast<const uint32_t *>(&r);
    }
}

// One warp maps `bytes` (a multiple of 4 KiB) of shared memory in place, 16 bytes per lane per
// access, eight accesses in flight.  The operand tiles are swizzled, which an element-wise map
// does not care about.
template <bool BF16, uint32_t OP>
__device__ __forceinline__ void xform_region(uint32_t addr, uint32_t bytes, uint32_t lane) {
    constexpr uint32_t STEP = 32 * 16;
    constexpr uint32_t DEPTH = 8;
    for (uint32_t off = lane * 16; off < bytes; off += DEPTH * STEP) {
        uint32_t w[DEPTH][4];
#pragma unroll
        for (uint32_t u = 0; u < DEPTH; ++u) ptx::lds128(addr + off + u * STEP, w[u]);
#pragma unroll
        for (uint32_t u = 0; u < DEPTH; ++u) {
#pragma unroll
            for (uint32_t j = 0; j < 4; ++j) w[u][j] = map_pair<BF16, OP>(w[u][j]);
            ptx::sts128(addr + off + u * STEP, w[u]);
        }
    }
}

template <bool BF16>
__device__ __forceinline__ void xform_dispatch(uint32_t op, uint32_t addr, uint32_t bytes, uint32_t lane) {
    switch (op) {
        case KLAS_MAP_SQRT: xform_region<BF16, KLAS_MAP_SQRT>(addr, bytes, lane); break;
        case KLAS_MAP_ABS: xform_region<BF16, KLAS_MAP_ABS>(addr, bytes, lane); break;
        case KLAS_MAP_SQUARE: xform_region<BF16, KLAS_MAP_SQUARE>(addr, bytes, lane); break;
        case KLAS_MAP_RELU: xform_region<BF16, KLAS_MAP_RELU>(addr, bytes, lane); break;
        case KLAS_MAP_NEG: xform_region<BF16, KLAS_MAP_NEG>(addr, bytes, lane); break;
        default: break;
    }
}

// One ring stage of a mapping kernel, handled by ONE warp (the mapping warps take the stages in
// turn, so that one stage's wait for its stores to drain overlaps the next stages' work): waits
// (bounded) until the stage's copies have landed, maps the A and / or B bytes in place, makes the
// writes visible to the tensor core's reads and arrives on `xfull_bar` (possibly a barrier of
// the pair's even CTA).
__device__ __forceinline__ bool xform_stage(const Params &p, uint32_t full_bar, uint32_t parity, const Ctl &ctl,
                                            int site, uint32_t a_addr, uint32_t a_bytes, uint32_t b_bytes,
                                            uint32_t xfull_bar_cluster, uint32_t lane) {
    bool ok = lane != 0 || bounded_wait(full_bar, parity, ctl, site, WAIT_LIMIT_NS, 32);
    ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
    if (!ok) return false;
    // Each lane observes the completed phase itself (immediate: the phase cannot advance before
    // this warp's own arrival below), which orders the copies' writes before its reads.
    for (uint32_t i = 0; i < 1024 && !ptx::mbar_try_wait(full_bar, parity); ++i) {
    }
    if (p.in_bf16) {
        xform_dispatch<true>(p.map_a, a_addr, a_bytes, lane);
        xform_dispatch<true>(p.map_b, a_addr + a_bytes, b_bytes, lane);
    } else {
        xform_dispatch<false>(p.map_a, a_addr, a_bytes, lane);
        xform_dispatch<false>(p.map_b, a_addr + a_bytes, b_bytes, lane);
    }
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) ptx::mbar_arrive_cluster(xfull_bar_cluster);
    return true;
}

template <uint32_t COMB>
__device__ __forceinline__ float comb_f32(float old, float acc, float alpha, float beta) {
    if constexpr (COMB == KLAS_COMB_MAX) return fmaxf(old, acc);
    else if constexpr (COMB == KLAS_COMB_MIN) return fminf(old, acc);
    else if constexpr (COMB == KLAS_COMB_MUL) return old * acc;
    else return fmaf(alpha, acc, beta * old);
}

// One 32-row x 128-byte block of the old C as a warp fetches it: four rows per instruction, 8 lanes
// per row, 128 contiguous bytes (`q[i]` is this lane's 16 bytes of row 4 i + lane / 8).
struct OldBlock {
    uint4 q[8];
};

template <typename OutT>
__device__ __forceinline__ void load_old_block(OldBlock &ob, const OutT *C, uint32_t col_blk, uint32_t row0,
                                               uint32_t b, uint32_t lane, const Params &p) {
    const uint32_t gcol = col_blk + (lane & 7u) * (16 / sizeof(OutT));
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t r = i * 4u + (lane >> 3);
        ob.q[i] = make_uint4(0u, 0u, 0u, 0u);
        if (row0 + r < p.M && gcol < p.N)   // plain loads: C may be D (in-place accumulate)
            ob.q[i] = *reinterpret_cast<const uint4 *>(C + size_t(b) * p.sd + size_t(row0 + r) * p.ldd + gcol);
    }
}

// Output path of the accumulators: converts one chunk (32 rows x 32 columns, lane r holding row r)
// and transposes it through shared memory so that global accesses are coalesced.
// Lane r writes 16-byte piece j of its row to piece (j ^ (r & 7)) of a 32-row x 128-byte block
// (conflict-free); once the block's last chunk is staged the warp reads it back four rows per
// instruction -- 8 lanes per row, 128 contiguous bytes -- and stores those.  A warp storing its
// own rows directly touches 32 different lines per instruction: measured on the 128 x 256
// tile at 2048^3, 9100 cycles per tile of a 43000-cycle kernel.  `c` is the chunk's index in
// the tile (it decides the position within the block), `col` its first column, `row0` the
// warp's first row, `buf` the warp's staging block.
// With an old C (alpha / beta, max / min / mul, in-place accumulate) the block of C travels the
// other way first: `ob` holds it (fetched coalesced while the previous block was on its way out),
// it is laid into the staging block in the same swizzle, each lane picks up its own row's pieces
// from there, combines and overwrites them.  `next_col_blk` < `tile_end`: the block to fetch next.
// (Each lane reading and writing its own row of C and D in global memory made the alpha/beta
// product at 8192^3 take 1.00-1.14 ms against 0.74 ms for the plain one, 0.38 against 0.12 ms at K = 1024.)
template <typename OutT>
__device__ __forceinline__ void emit_staged(const uint32_t (&v)[32], uint32_t c, uint32_t col, uint32_t row0,
                                            uint32_t b, uint32_t buf, uint32_t lane, const Params &p,
                                            bool relu, float plain_scale, const OutT *C = nullptr,
                                            OldBlock *ob = nullptr, uint32_t next_col_blk = 0, uint32_t tile_end = 0) {
    constexpr uint32_t COLS_PER_BLOCK = 128 / sizeof(OutT);     // columns of one 128-byte staging row
    constexpr uint32_t CHUNKS_PER_BLOCK = COLS_PER_BLOCK / 32;  // TMEM chunks (32 columns) per block
    constexpr uint32_t PIECES = 32 * sizeof(OutT) / 16;         // 16-byte pieces per chunk per row
    constexpr uint32_t VEC = 16 / sizeof(OutT);
    OutT *const D = static_cast<OutT *>(p.D);
    const uint32_t sub = c % CHUNKS_PER_BLOCK;
    if (C != nullptr && sub == 0) {
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t r = i * 4u + (lane >> 3);
            const uint32_t addr = buf + r * 128u + (((lane & 7u) ^ (r & 7u)) * 16u);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(ob->q[i].x), "r"(ob->q[i].y),
                         "r"(ob->q[i].z), "r"(ob->q[i].w)
                         : "memory");
        }
        __syncwarp();
        if (next_col_blk < tile_end) load_old_block<OutT>(*ob, C, next_col_blk, row0, b, lane, p);
    }
    auto stage_pieces = [&](auto comb_tag) {
        constexpr uint32_t COMB = decltype(comb_tag)::value;
#pragma unroll
        for (uint32_t j = 0; j < PIECES; ++j) {
            union {
                uint4 raw;
                OutT e[VEC];
            } pk, old;
            const uint32_t piece = (sub * PIECES + j) ^ (lane & 7u);
            const uint32_t addr = buf + lane * 128u + piece * 16u;
            if (C != nullptr) {
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(old.raw.x), "=r"(old.raw.y), "=r"(old.raw.z), "=r"(old.raw.w)
                             : "r"(addr)
                             : "memory");
#pragma unroll
                for (uint32_t e = 0; e < VEC; ++e)
                    pk.e[e] = OutTraits<OutT>::from_f32(comb_f32<COMB>(OutTraits<OutT>::to_f32(old.e[e]),
                                                                        __uint_as_float(v[j * VEC + e]), p.alpha, p.beta));
            } else {
#pragma unroll
                for (uint32_t e = 0; e < VEC; ++e) {
                    const float a = __uint_as_float(v[j * VEC + e]) * plain_scale;
                    pk.e[e] = OutTraits<OutT>::from_f32(relu ? fmaxf(a, 0.0f) : a);
                }
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk.raw.x),
                         "r"(pk.raw.y), "r"(pk.raw.z), "r"(pk.raw.w)
                         : "memory");
        }
    };
    if (C == nullptr) {
        stage_pieces(std::integral_constant<uint32_t, KLAS_COMB_AXPBY>{});
    } else {
        switch (p.comb) {
            case KLAS_COMB_MAX: stage_pieces(std::integral_constant<uint32_t, KLAS_COMB_MAX>{}); break;
            case KLAS_COMB_MIN: stage_pieces(std::integral_constant<uint32_t, KLAS_COMB_MIN>{}); break;
            case KLAS_COMB_MUL: stage_pieces(std::integral_constant<uint32_t, KLAS_COMB_MUL>{}); break;
            default: stage_pieces(std::integral_constant<uint32_t, KLAS_COMB_AXPBY>{}); break;
        }
    }
    if (sub == CHUNKS_PER_BLOCK - 1) {
        __syncwarp();
        const uint32_t col_blk = col - sub * 32u;
        const uint32_t piece = lane & 7u;
        const uint32_t gcol = col_blk + piece * VEC;
#pragma unroll
        for (uint32_t i = 0; i < 8; ++i) {
            const uint32_t r = i * 4u + (lane >> 3);
            uint4 val;
            const uint32_t addr = buf + r * 128u + ((piece ^ (r & 7u)) * 16u);
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                         : "r"(addr)
                         : "memory");
            if (row0 + r < p.M && gcol < p.N)
                *reinterpret_cast<uint4 *>(D + size_t(b) * p.sd + size_t(row0 + r) * p.ldd + gcol) = val;
        }
        __syncwarp();   // the buffer may be overwritten by the next block
    }
}

// Second step of a K-split product: adds the f32 partial products (pages b * parts + q of `ws`,
// each rows x cols, dense) in the order of q -- so the result is the same from run to run -- and
// sends the sum through the output rule of the unsplit kernel: alpha / beta / the old C / relu /
// the output type.  One thread per 4 consecutive columns; everything it reads is in L2.
struct ReduceArgs {
    const float *ws;
    const void *C;
    void *D;
    uint32_t rows, cols, parts, batch;
    uint64_t ldd, sd;
    float alpha, beta;
    uint32_t comb;
    // tile0 > 0: only the tiles from tile0 on (in the product kernel's tile order) were split
    uint32_t tile0, tile_m, tile_n, tiles_m, tiles_n, raster_group;
};

template <typename OutT, uint32_t COMB>
__device__ __forceinline__ void reduce_store(const float (&acc)[4], OutT *d, const OutT *c, const ReduceArgs &a) {
    OutT out[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float v;
        if (c != nullptr)
            v = comb_f32<COMB>(OutTraits<OutT>::to_f32(c[j]), acc[j], a.alpha, a.beta);
        else
            v = a.comb == KLAS_COMB_RELU ? fmaxf(acc[j], 0.0f) : (a.comb == KLAS_COMB_SCALED ? acc[j] * a.alpha : acc[j]);
        out[j] = OutTraits<OutT>::from_f32(v);
    }
    if constexpr (sizeof(OutT) == 4)
        *reinterpret_cast<uint4 *>(d) = *reinterpret_cast<const uint4 *>(out);
    else
        *reinterpret_cast<uint2 *>(d) = *reinterpret_cast<const uint2 *>(out);
}

template <typename OutT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const ReduceArgs a) {
    const uint64_t page_elems = uint64_t(a.rows) * a.cols;
    // whole matrix: one item per 4 columns of every row and page; tail only (tile0 > 0, one page):
    // one item per 4 columns of every row of the tiles from tile0 on, found through the tile order
    const uint64_t quads_per_row = a.cols / 4;
    const uint64_t tile_quads = uint64_t(a.tile_m) * (a.tile_n / 4);
    const uint64_t total = a.tile0 > 0 ? uint64_t(a.tiles_m * a.tiles_n - a.tile0) * tile_quads
                                       : uint64_t(a.batch) * a.rows * quads_per_row;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        uint64_t b = 0, r, c4;
        if (a.tile0 > 0) {
            const uint32_t t = a.tile0 + uint32_t(i / tile_quads);
            const uint32_t in_tile = uint32_t(i % tile_quads);
            // decode_tile's order: groups of `raster_group` tile columns, rows fastest within a group
            const uint32_t group_tiles = a.raster_group * a.tiles_m;
            const uint32_t g = t / group_tiles, first_n = g * a.raster_group;
            const uint32_t width = min(a.raster_group, a.tiles_n - first_n);
            const uint32_t in = t - g * group_tiles;
            const uint32_t tm = in / width, tn = first_n + in % width;
            r = uint64_t(tm) * a.tile_m + in_tile / (a.tile_n / 4);
            c4 = uint64_t(tn) * a.tile_n + (in_tile % (a.tile_n / 4)) * 4;
            if (r >= a.rows || c4 >= a.cols) continue;
        } else {
            b = i / (uint64_t(a.rows) * quads_per_row);
            const uint64_t in_page = i - b * a.rows * quads_per_row;
            r = in_page / quads_per_row;
            c4 = (in_page - r * quads_per_row) * 4;
        }
        const float *src = a.ws + (b * a.parts) * page_elems + r * a.cols + c4;
        // all parts' loads go out together (at most 8); the sum is taken in index order
        float4 q[8];
#pragma unroll
        for (uint32_t part = 0; part < 8; ++part)
            if (part < a.parts) q[part] = __ldcg(reinterpret_cast<const float4 *>(src + part * page_elems));
        float acc[4] = {q[0].x, q[0].y, q[0].z, q[0].w};
#pragma unroll
        for (uint32_t part = 1; part < 8; ++part)
            if (part < a.parts) acc[0] += q[part].x, acc[1] += q[part].y, acc[2] += q[part].z, acc[3] += q[part].w;
        const uint64_t off = b * a.sd + r * a.ldd + c4;
        OutT *d = static_cast<OutT *>(a.D) + off;
        const OutT *c = a.C ? static_cast<const OutT *>(a.C) + off : nullptr;
        switch (a.comb) {
            case KLAS_COMB_MAX: reduce_store<OutT, KLAS_COMB_MAX>(acc, d, c, a); break;
            case KLAS_COMB_MIN: reduce_store<OutT, KLAS_COMB_MIN>(acc, d, c, a); break;
            case KLAS_COMB_MUL: reduce_store<OutT, KLAS_COMB_MUL>(acc, d, c, a); break;
            default: reduce_store<OutT, KLAS_COMB_AXPBY>(acc, d, c, a); break;
        }
    }
}

// XFORM adds four warps that map the staged A / B bytes in place between the copy and the MMA
// (single-CTA tiles only).
// OLD_C: the instantiation whose epilogue meets an old C (alpha / beta, max / min / mul, in-place
// accumulate).  Products without one run instantiations that carry none of that path's registers.
template <typename OutT, bool PAIR, bool XFORM = false, bool OLD_C = false>
__global__ void __launch_bounds__(NUM_THREADS + (XFORM ? XFORM_THREADS : 0), 1)
    gemm_umma_kernel(const __grid_constant__ CUtensorMap tm_a,
                     const __grid_constant__ CUtensorMap tm_b, const Params p) {
    static_assert(!(PAIR && XFORM), "operand maps are built for the single-CTA and the wide tiles");
    using S = Shape<PAIR>;
    // The single-CTA tile comes in three widths; a narrower tile has smaller stages and a deeper
    // ring (the same 192 KiB), because what it lacks is bytes in flight, not arithmetic.
    const uint32_t STAGES = PAIR ? S::STAGES : p.stages;
    const uint32_t STAGE_BYTES = PAIR ? S::STAGE_BYTES : p.stage_bytes;

    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzled tiles need 1024-byte aligned bases.  The dynamic shared window
    // starts at the same offset in both CTAs of a pair, so the padding is identical.
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;

    const uint32_t epi_base = smem_base + RING_BYTES;
    uint8_t *bar_region = smem + RING_BYTES + NUM_EPI_WARPS * EPI_BLOCK_BYTES;
    const uint32_t bar_base = epi_base + NUM_EPI_WARPS * EPI_BLOCK_BYTES;
    // layout: full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2], tmem slot, abort flag
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (MAX_STAGES + s); };
    auto tfull_bar = [&](uint32_t a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
    auto tempty_bar = [&](uint32_t a) { return bar_base + 8u * (2 * MAX_STAGES + ACC_STAGES + a); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_region + 8u * (2 * MAX_STAGES + 2 * ACC_STAGES));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    [[maybe_unused]] auto xfull_bar = [&](uint32_t s) { return bar_base + XFULL_OFFSET + 8u * s; };
    static_assert(8u * (2 * MAX_STAGES + 2 * ACC_STAGES) + 8u <= XFULL_OFFSET && XFULL_OFFSET + 8u * MAX_STAGES <= BARRIER_BYTES,
                  "barrier block layout");

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;  // 0 = the CTA that issues MMAs
    const uint32_t group = blockIdx.x / S::CTAS;                    // index of this CTA group
    const uint32_t num_groups = gridDim.x / S::CTAS;
    const Ctl ctl{abort_flag, p.status};

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
            if constexpr (XFORM) ptx::mbar_init(xfull_bar(s), 1);
        }
        for (uint32_t a = 0; a < ACC_STAGES; ++a) {
            ptx::mbar_init(tfull_bar(a), 1);
            ptx::mbar_init(tempty_bar(a), NUM_EPI_WARPS * S::CTAS);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0 && p.num_kb > 0) {
        ptx::prefetch_tensormap(&tm_a);
        ptx::prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        // both CTAs' barriers must exist before either side signals the other's
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        // One thread runs the whole loop: no warp-wide votes or re-convergence per stage.
        // Like the MMA issuer's, this thread's instruction stream is kept short: destination, barrier
        // and K coordinate are running values.
        uint32_t stage = 0, phase = 0;
        bool ok = lane == 0;
        const uint32_t full0 = full_bar(0), empty0 = empty_bar(0);
        [[maybe_unused]] const uint32_t full0_cta0 = PAIR ? ptx::map_to_cta(full0, 0) : full0;
        uint32_t a_dst = smem_base, fullb = full0, emptyb = empty0;
        [[maybe_unused]] uint32_t fullb_cta0 = full0_cta0;
        const uint32_t tile_n = PAIR ? BN : p.tile_n;
        const uint32_t tx_bytes = PAIR ? 2 * STAGE_BYTES : A_STAGE_BYTES + tile_n * BK * 2u;   // the even CTA's barrier counts both CTAs' loads
        const bool b_row_major = p.b_row_major != 0;
        for (uint32_t w = group; ok && w < p.num_work; w += num_groups) {
            const WorkItem wi(w, p);
            uint32_t b, tm, tn;
            decode_tile(wi.tile, p, b, tm, tn);
            const int32_t a_row = int32_t(tm * S::TILE_M + cta_rank * BM);
            const int32_t b_col = int32_t(tn * tile_n + cta_rank * S::B_COLS);
            int32_t k0 = int32_t(wi.kb0 * BK);
            for (uint32_t kb = wi.kb0; kb < wi.kb1; ++kb, k0 += int32_t(BK)) {
                if (stage % S::RELEASE_GROUP == 0) {
                    // stages are handed back in groups; the group's last stage carries the barrier
                    ok = bounded_wait(emptyb + 8u * (S::RELEASE_GROUP - 1), phase ^ 1u, ctl, SITE_PRODUCER_EMPTY, WAIT_LIMIT_NS, 64);
                    if (!ok) break;
                }
                const uint32_t b_dst = a_dst + A_STAGE_BYTES;
                if constexpr (PAIR) {
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(fullb, tx_bytes);
                    ptx::tma_load_3d_pair(a_dst, &tm_a, fullb_cta0, k0, a_row, int32_t(b));
                    if (b_row_major) {
#pragma unroll
                        for (uint32_t j = 0; j < S::B_COLS / 64; ++j)
                            ptx::tma_load_3d_pair(b_dst + j * B_CHUNK_BYTES, &tm_b, fullb_cta0, b_col + int32_t(j * 64), k0, int32_t(b));
                    } else {
                        ptx::tma_load_3d_pair(b_dst, &tm_b, fullb_cta0, k0, b_col, int32_t(b));
                    }
                } else {
                    ptx::mbar_arrive_expect_tx(fullb, tx_bytes);
                    ptx::tma_load_3d(a_dst, &tm_a, fullb, k0, a_row, int32_t(b));
                    if (b_row_major) {
                        for (uint32_t j = 0; j < tile_n / 64; ++j)
                            ptx::tma_load_3d(b_dst + j * B_CHUNK_BYTES, &tm_b, fullb, b_col + int32_t(j * 64), k0, int32_t(b));
                    } else {
                        ptx::tma_load_3d(b_dst, &tm_b, fullb, k0, b_col, int32_t(b));
                    }
                }
                ++stage;
                a_dst += STAGE_BYTES, fullb += 8u, emptyb += 8u, fullb_cta0 += 8u;
                if (stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                    a_dst = smem_base, fullb = full0, emptyb = empty0, fullb_cta0 = full0_cta0;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // K-major operand: 8-row groups 1024 bytes apart; a K step of 16 elements = 32 bytes.
        // MN-major B: 64-column slabs 8192 bytes apart (leading), 8-row K groups 1024 bytes
        // apart (stride); a K step of 16 rows = 2048 bytes.
        // The loop below is one thread's instruction stream, and that stream is what bounds the
        // narrower tiles, so it is kept short: descriptors as 32-bit halves with the low half a running
        // value (start address >> 4; stage and K step add constants), barrier addresses as running values.
        const uint64_t a_desc_base = ptx::umma_desc_base_sw128(16, 1024);
        const uint64_t b_desc_base = p.b_row_major ? ptx::umma_desc_base_sw128(B_CHUNK_BYTES, 1024)
                                                   : ptx::umma_desc_base_sw128(16, 1024);
        const uint32_t a_hi = uint32_t(a_desc_base >> 32), b_hi = uint32_t(b_desc_base >> 32);
        const uint32_t a_lo0 = uint32_t(a_desc_base) | ((smem_base & 0x3FFFFu) >> 4);
        const uint32_t b_lo0 = uint32_t(b_desc_base) | (((smem_base + A_STAGE_BYTES) & 0x3FFFFu) >> 4);
        const uint32_t stage_step = STAGE_BYTES >> 4;
        const uint32_t b_step = (p.b_row_major ? UMMA_K * 128u : UMMA_K * 2u) >> 4;   // one K step of 16
        const uint32_t full0 = XFORM ? xfull_bar(0) : full_bar(0), empty0 = empty_bar(0);
        const uint32_t idesc = p.idesc;
        uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
        uint32_t a_lo = a_lo0, b_lo = b_lo0, fullb = full0, emptyb = empty0;
        bool ok = lane == 0;   // one thread runs the whole loop
        const bool issuer = cta_rank == 0;
        auto mma = [&](uint32_t d, uint32_t kk, uint32_t accumulate) {
            if constexpr (PAIR)
                ptx::umma_f16_ss_pair_halves(d, a_lo + kk * (UMMA_K * 2u >> 4), a_hi, b_lo + kk * b_step, b_hi, idesc, accumulate);
            else
                ptx::umma_f16_ss_halves(d, a_lo + kk * (UMMA_K * 2u >> 4), a_hi, b_lo + kk * b_step, b_hi, idesc, accumulate);
        };
        static_assert(BK / UMMA_K == 4, "the K block is issued as four MMAs");
        for (uint32_t w = group; issuer && ok && p.num_kb > 0 && w < p.num_work; w += num_groups) {
            const WorkItem wi(w, p);
            ok = bounded_wait(tempty_bar(acc), acc_phase ^ 1u, ctl, SITE_MMA_TMEM_EMPTY);
            if (!ok) break;
            ptx::tc_fence_after_sync();   // orders the epilogue's TMEM reads before these MMAs' writes
            const uint32_t d_tmem = tmem_base + acc * BN;
            uint32_t later = 0;   // 0 in the tile's first K block: its first MMA overwrites the accumulator
            for (uint32_t kb = wi.kb0; kb < wi.kb1; ++kb) {
                ok = bounded_wait(fullb, phase, ctl, SITE_MMA_FULL);
                if (!ok) break;
                mma(d_tmem, 0, later);
                mma(d_tmem, 1, 1u);
                mma(d_tmem, 2, 1u);
                mma(d_tmem, 3, 1u);
                later = 1u;
                // free the shared-memory stage (in both CTAs) once these MMAs retire
                if constexpr (PAIR) {
                    if (stage % S::RELEASE_GROUP == S::RELEASE_GROUP - 1) ptx::umma_commit_pair_mask(emptyb, 0x3);
                    if (kb + 1 == wi.kb1) ptx::umma_commit_pair_mask(tfull_bar(acc), 0x3);
                } else {
                    ptx::umma_commit(emptyb);
                    if (kb + 1 == wi.kb1) ptx::umma_commit(tfull_bar(acc));
                }
                ++stage;
                a_lo += stage_step, b_lo += stage_step, fullb += 8u, emptyb += 8u;
                if (stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                    a_lo = a_lo0, b_lo = b_lo0, fullb = full0, emptyb = empty0;
                }
            }
            if (++acc == ACC_STAGES) {
                acc = 0;
                acc_phase ^= 1u;
            }
        }
        __syncwarp();
    } else if (XFORM && warp >= 2 + NUM_EPI_WARPS) {
        // ------------------------------------------------------------ operand maps
        const uint32_t xw = warp - (2 + NUM_EPI_WARPS);
        uint32_t stage = 0, phase = 0, turn = 0;
        bool ok = true;
        for (uint32_t w = group; ok && w < p.num_work; w += num_groups) {
            const WorkItem wi(w, p);
            for (uint32_t kb = wi.kb0; kb < wi.kb1; ++kb) {
                if (turn == xw)
                    ok = xform_stage(p, full_bar(stage), phase, ctl, SITE_XFORM_FULL, smem_base + stage * STAGE_BYTES,
                                     A_STAGE_BYTES, PAIR ? S::B_STAGE_BYTES : p.tile_n * BK * 2u, xfull_bar(stage), lane);
                if (!ok) break;
                if (++turn == XFORM_WARPS) turn = 0;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t quad = warp & 3u;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
        const OutT *const C = OLD_C ? static_cast<const OutT *>(p.C) : nullptr;
        uint32_t acc = 0, acc_phase = 0;
        bool ok = true;
        for (uint32_t w = group; ok && w < p.num_work; w += num_groups) {
            const WorkItem wi(w, p);
            uint32_t b, tm, tn;
            decode_tile(wi.tile, p, b, tm, tn);
            const uint32_t row0 = tm * S::TILE_M + cta_rank * BM + quad * 32u;
            const uint32_t tile_n = PAIR ? BN : p.tile_n;
            const uint32_t col0 = tn * tile_n;
            const uint32_t page = b * p.ksplit + wi.part;   // = b unless K is split (a split launch has no old C)
            constexpr uint32_t COLS_PER_BLOCK = 128 / sizeof(OutT);
            // the first block of the old C is on its way while the accumulator is still being computed
            OldBlock old_c;
            if (C != nullptr) load_old_block<OutT>(old_c, C, col0, row0, page, lane, p);
            if (p.num_kb > 0) {
                ok = lane != 0 || bounded_wait(tfull_bar(acc), acc_phase, ctl, SITE_EPI_TMEM_FULL, WAIT_LIMIT_NS, 128);
                ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;   // lane 0 polls, the warp follows
                if (!ok) break;
                ptx::tc_fence_after_sync();
            }
            const uint32_t buf = epi_base + (warp - 2) * EPI_BLOCK_BYTES;
            const uint32_t taddr0 = tmem_base + ((quad * 32u) << 16) + acc * BN;
            const bool relu = p.comb == KLAS_COMB_RELU;
            const float plain_scale = p.comb == KLAS_COMB_SCALED ? p.alpha : 1.0f;   // x * 1.0f is exact
            const bool have_acc = p.num_kb > 0;
            const uint32_t nchunk = tile_n / 32;   // 2, 4 or 8
            {
                // Chunks leave through the staging block (with an old C: after meeting it there), the
                // next chunk's tcgen05.ld in flight while the current one is converted and stored.
                uint32_t va[32], vb[32];
                if (have_acc) {
                    ptx::tmem_ld_32x32b_x32(taddr0, va);
                } else {
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) va[j] = vb[j] = 0u;
                }
                auto emit = [&](const uint32_t (&v)[32], uint32_t c) {
                    const uint32_t col = col0 + c * 32u;
                    const uint32_t next_blk = col - (c % (COLS_PER_BLOCK / 32)) * 32u + COLS_PER_BLOCK;
                    emit_staged<OutT>(v, c, col, row0, page, buf, lane, p, relu, plain_scale, C, &old_c, next_blk, col0 + tile_n);
                };
#pragma unroll 1
                for (uint32_t c = 0; c < nchunk; c += 2) {
                    if (have_acc) {
                        ptx::tmem_ld_wait();
                        ptx::tmem_ld_32x32b_x32(taddr0 + (c + 1) * 32u, vb);
                    }
                    emit(va, c);
                    if (have_acc) {
                        ptx::tmem_ld_wait();
                        if (c + 2 < nchunk) ptx::tmem_ld_32x32b_x32(taddr0 + (c + 2) * 32u, va);
                    }
                    emit(vb, c + 1);
                }
            }
            if (p.num_kb > 0) {
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    // the accumulator stage is free when both CTAs' epilogues have drained it
                    if constexpr (PAIR)
                        ptx::mbar_arrive_cluster(ptx::map_to_cta(tempty_bar(acc), 0));
                    else
                        ptx::mbar_arrive(tempty_bar(acc));
                }
                if (++acc == ACC_STAGES) {
                    acc = 0;
                    acc_phase ^= 1u;
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (PAIR) {
        // neither CTA may leave while its partner can still touch its barriers or operands
        ptx::cluster_arrive();
        ptx::cluster_wait();
    }
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if (*abort_flag != 0) {
            // A role gave up: let copies and MMAs already in flight land before the
            // tensor memory and this CTA's shared memory are handed back.
            for (int i = 0; i < 256; ++i) __nanosleep(1000);
        }
        if constexpr (PAIR)
            ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else
            ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// "Wide" instantiation for problems that fill the machine: a cluster of two CTAs owns a
// 512 x 256 tile; each CTA holds 256 rows of A (two M=128 halves) and 128 columns of B,
// 4 stages of 48 KiB.  Per K step the even CTA issues two M=256 pair-MMAs (one per half),
// so a barrier round covers 8 MMAs and the B slab staged by a CTA feeds 512 output rows:
// the L2 -> SM bytes per flop are half those of the single-CTA tile.  Both accumulator
// halves (2 x 256 columns) fill tensor memory, so the epilogue drains TMEM before the next
// tile's MMAs start; it is kept short by eight epilogue warps (one group of four per half)
// that transpose 32 x 128-byte blocks through swizzled shared memory into coalesced global
// stores, and the producer keeps loading during it.
// ---------------------------------------------------------------------------
namespace wide {
constexpr uint32_t STAGES = 4;
constexpr uint32_t A_ROWS = 256;                       // rows of A staged by each CTA
constexpr uint32_t B_COLS = 128;                       // columns of B staged by each CTA
constexpr uint32_t A_BYTES = A_ROWS * BK * 2;
constexpr uint32_t B_BYTES = B_COLS * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;    // 48 KiB
constexpr uint32_t TILE_M = 2 * A_ROWS;                // rows of a cluster tile
constexpr uint32_t EPI_BUF_BYTES = 32 * 128;           // one staging block: 32 rows x 128 bytes
constexpr uint32_t EPI_WARPS = 8;                     // two groups of four, one per accumulator half
constexpr uint32_t THREADS = (2 + EPI_WARPS) * 32;
constexpr uint32_t EPI_BYTES = EPI_WARPS * EPI_BUF_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BARRIER_BYTES + 1024;
}  // namespace wide

enum : int { SITE_WIDE = 0x100 };

// XFORM adds four warps per CTA that map the staged A / B bytes in place, taking the ring's
// stages in turn.  Each CTA then counts its own copies on its own barrier, the stage's mapping
// warp waits there, and the two warps of the pair (one per CTA) report to a barrier of the even
// CTA that the MMA thread waits on.
template <typename OutT, bool XFORM = false, bool OLD_C = false>
__global__ void __launch_bounds__(wide::THREADS + (XFORM ? XFORM_THREADS : 0), 1)
    gemm_umma_wide_kernel(const __grid_constant__ CUtensorMap tm_a,
                          const __grid_constant__ CUtensorMap tm_b, const Params p) {
    using namespace wide;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    const uint32_t epi_base = smem_base + STAGES * STAGE_BYTES;
    uint8_t *bar_region = smem + STAGES * STAGE_BYTES + EPI_BYTES;
    const uint32_t bar_base = epi_base + EPI_BYTES;
    // layout: full[STAGES], empty[STAGES], tmem_full, tmem_empty, tmem slot, abort flag
    auto full_bar = [&](uint32_t s) { return bar_base + 8u * s; };
    auto empty_bar = [&](uint32_t s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
    const uint32_t tempty_bar = bar_base + 8u * (2 * STAGES + 1);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_region + 8u * (2 * STAGES + 2));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    [[maybe_unused]] auto xfull_bar = [&](uint32_t s) { return bar_base + XFULL_OFFSET + 8u * s; };
    static_assert(8u * (2 * STAGES + 2) + 8u <= XFULL_OFFSET && XFULL_OFFSET + 8u * STAGES <= BARRIER_BYTES,
                  "barrier block layout");

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = ptx::cluster_ctarank();
    const uint32_t group = blockIdx.x / 2;
    const uint32_t num_groups = gridDim.x / 2;
    const Ctl ctl{abort_flag, p.status};

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
            if constexpr (XFORM) ptx::mbar_init(xfull_bar(s), 2);
        }
        ptx::mbar_init(tfull_bar, 1);
        ptx::mbar_init(tempty_bar, EPI_WARPS * 2);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0 && p.num_kb > 0) {
        ptx::prefetch_tensormap(&tm_a);
        ptx::prefetch_tensormap(&tm_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        uint32_t stage = 0, phase = 0;
        bool ok = lane == 0;
        [[maybe_unused]] const uint32_t full_bars_cta0 = ptx::map_to_cta(full_bar(0), 0);
        for (uint32_t t = group; ok && t < p.num_tiles; t += num_groups) {
            uint32_t b, tm, tn;
            decode_tile(t, p, b, tm, tn);
            const int32_t a_row = int32_t(tm * TILE_M + cta_rank * A_ROWS);
            const int32_t b_col = int32_t(tn * BN + cta_rank * B_COLS);
            for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                ok = bounded_wait(empty_bar(stage), phase ^ 1u, ctl, SITE_WIDE | SITE_PRODUCER_EMPTY, WAIT_LIMIT_NS, 64);
                if (!ok) break;
                const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
                const uint32_t b_dst = a_dst + A_BYTES;
                const int32_t k0 = int32_t(kb * BK);
                if constexpr (XFORM) {
                    // each CTA counts its own copies: its mapping warps wait on this barrier
                    ptx::mbar_arrive_expect_tx(full_bar(stage), STAGE_BYTES);
                    ptx::tma_load_3d(a_dst, &tm_a, full_bar(stage), k0, a_row, int32_t(b));
                    if (p.b_row_major) {
#pragma unroll
                        for (uint32_t j = 0; j < B_COLS / 64; ++j)
                            ptx::tma_load_3d(b_dst + j * B_CHUNK_BYTES, &tm_b, full_bar(stage),
                                             b_col + int32_t(j * 64), k0, int32_t(b));
                    } else {
                        ptx::tma_load_3d(b_dst, &tm_b, full_bar(stage), k0, b_col, int32_t(b));
                    }
                } else {
                    // the even CTA's barrier counts the bytes of both CTAs' loads
                    if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_bar(stage), 2 * STAGE_BYTES);
                    const uint32_t bar = full_bars_cta0 + 8u * stage;
                    ptx::tma_load_3d_pair(a_dst, &tm_a, bar, k0, a_row, int32_t(b));
                    if (p.b_row_major) {
#pragma unroll
                        for (uint32_t j = 0; j < B_COLS / 64; ++j)
                            ptx::tma_load_3d_pair(b_dst + j * B_CHUNK_BYTES, &tm_b, bar,
                                                  b_col + int32_t(j * 64), k0, int32_t(b));
                    } else {
                        ptx::tma_load_3d_pair(b_dst, &tm_b, bar, k0, b_col, int32_t(b));
                    }
                }
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (one thread, even CTA)
        const uint64_t a_desc_base = ptx::umma_desc_base_sw128(16, 1024);
        const uint64_t b_desc_base = p.b_row_major ? ptx::umma_desc_base_sw128(B_CHUNK_BYTES, 1024)
                                                   : ptx::umma_desc_base_sw128(16, 1024);
        const uint32_t b_kstep = p.b_row_major ? UMMA_K * 128u : UMMA_K * 2u;
        uint32_t stage = 0, phase = 0, tile_phase = 0;
        bool ok = lane == 0 && cta_rank == 0;
        for (uint32_t t = group; ok && p.num_kb > 0 && t < p.num_tiles; t += num_groups) {
            // both CTAs' epilogues must have drained the previous tile's accumulators
            {
                ok = bounded_wait(tempty_bar, tile_phase ^ 1u, ctl, SITE_WIDE | SITE_MMA_TMEM_EMPTY);
            }
            if (!ok) break;
            ptx::tc_fence_after_sync();
            for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                {
                    if constexpr (XFORM)
                        ok = bounded_wait<true>(xfull_bar(stage), phase, ctl, SITE_WIDE | SITE_MMA_FULL);
                    else
                        ok = bounded_wait(full_bar(stage), phase, ctl, SITE_WIDE | SITE_MMA_FULL);
                }
                if (!ok) break;
                const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (uint32_t kk = 0; kk < BK / UMMA_K; ++kk) {
                    const uint64_t b_desc = ptx::umma_desc_at(b_desc_base, b_addr + kk * b_kstep);
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h) {
                        // half h: rows [128 h, 128 h + 128) of each CTA's A tile -> accumulator columns [256 h, ...)
                        const uint64_t a_desc = ptx::umma_desc_at(
                            a_desc_base, a_addr + h * (BM * BK * 2) + kk * UMMA_K * 2u);
                        ptx::umma_f16_ss_pair(tmem_base + h * BN, a_desc, b_desc, p.idesc,
                                              (kb | kk) != 0 ? 1u : 0u);
                    }
                }
                ptx::umma_commit_pair_mask(empty_bar(stage), 0x3);
                if (kb + 1 == p.num_kb) ptx::umma_commit_pair_mask(tfull_bar, 0x3);
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
            tile_phase ^= 1u;
        }
        __syncwarp();
    } else if (XFORM && warp >= 2 + EPI_WARPS) {
        // ------------------------------------------------------------ operand maps (4 warps per CTA)
        const uint32_t xw = warp - (2 + EPI_WARPS);
        const uint32_t xfull_cta0 = ptx::map_to_cta(xfull_bar(0), 0);
        uint32_t stage = 0, phase = 0, turn = 0;
        bool ok = true;
        for (uint32_t t = group; ok && t < p.num_tiles; t += num_groups) {
            for (uint32_t kb = 0; kb < p.num_kb; ++kb) {
                if (turn == xw)
                    ok = xform_stage(p, full_bar(stage), phase, ctl, SITE_WIDE | SITE_XFORM_FULL,
                                     smem_base + stage * STAGE_BYTES, A_BYTES, B_BYTES, xfull_cta0 + 8u * stage, lane);
                if (!ok) break;
                if (++turn == XFORM_WARPS) turn = 0;
                if (++stage == STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (8 warps)
        // Warps 2-5 drain accumulator half 0, warps 6-9 half 1; within a group warp w owns the
        // TMEM lanes of quadrant w & 3.  Each warp walks its 8 chunks of 32 columns with the
        // next tcgen05.ld in flight while the current chunk is converted and staged, and hands
        // the accumulator back as soon as its last chunk is in registers.
        const uint32_t quad = warp & 3u;
        const uint32_t h = (warp - 2) >> 2;
        const OutT *const C = OLD_C ? static_cast<const OutT *>(p.C) : nullptr;
        constexpr uint32_t NCHUNK = BN / 32;
        const uint32_t buf = epi_base + (warp - 2) * EPI_BUF_BYTES;
        const uint32_t tempty_cta0 = ptx::map_to_cta(tempty_bar, 0);
        const uint32_t taddr0 = tmem_base + ((quad * 32u) << 16) + h * BN;
        const bool relu = p.comb == KLAS_COMB_RELU;
        const float plain_scale = p.comb == KLAS_COMB_SCALED ? p.alpha : 1.0f;   // x * 1.0f is exact
        uint32_t tile_phase = 0;
        bool ok = true;
        for (uint32_t t = group; ok && t < p.num_tiles; t += num_groups) {
            uint32_t b, tm, tn;
            decode_tile(t, p, b, tm, tn);
            const bool have_acc = p.num_kb > 0;
            const uint32_t row0 = tm * TILE_M + cta_rank * A_ROWS + h * BM + quad * 32u;
            constexpr uint32_t COLS_PER_BLOCK = 128 / sizeof(OutT);
            // the first block of the old C is on its way while the accumulator is still being computed
            OldBlock old_c;
            if (C != nullptr) load_old_block<OutT>(old_c, C, tn * BN, row0, b, lane, p);
            if (have_acc) {
                ok = lane != 0 || bounded_wait(tfull_bar, tile_phase, ctl, SITE_WIDE | SITE_EPI_TMEM_FULL, WAIT_LIMIT_NS, 128);
                ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;   // lane 0 polls, the warp follows
                if (!ok) break;
                ptx::tc_fence_after_sync();
            }

            // Every chunk goes through the warp's staging block (emit_staged), where it meets the old C if there is one.
            auto emit = [&](const uint32_t (&v)[32], uint32_t c) {
                const uint32_t col = tn * BN + c * 32u;
                const uint32_t next_blk = col - (c % (COLS_PER_BLOCK / 32)) * 32u + COLS_PER_BLOCK;
                emit_staged<OutT>(v, c, col, row0, b, buf, lane, p, relu, plain_scale, C, &old_c, next_blk, (tn + 1) * BN);
            };

            uint32_t va[32], vb[32];
            if (have_acc) {
                ptx::tmem_ld_32x32b_x32(taddr0, va);
            } else {
#pragma unroll
                for (uint32_t j = 0; j < 32; ++j) va[j] = vb[j] = 0u;
            }
#pragma unroll
            for (uint32_t c = 0; c < NCHUNK; c += 2) {
                if (have_acc) {
                    ptx::tmem_ld_wait();
                    ptx::tmem_ld_32x32b_x32(taddr0 + (c + 1) * 32u, vb);
                }
                emit(va, c);
                if (have_acc) {
                    ptx::tmem_ld_wait();
                    if (c + 2 < NCHUNK) {
                        ptx::tmem_ld_32x32b_x32(taddr0 + (c + 2) * 32u, va);
                    } else {
                        // last chunk is in registers: this warp no longer needs the accumulator
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(tempty_cta0);
                    }
                }
                emit(vb, c + 1);
            }
            if (have_acc) tile_phase ^= 1u;
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if (*abort_flag != 0) {
            for (int i = 0; i < 256; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// Diagnostic kernel: one warp waits, with the pipeline's bounded wait, on a barrier that
// nothing will ever signal.  After `limit_ns` the wait gives up, records SITE_PROBE in the
// status word and the kernel returns normally -- the path a stalled pipeline would take.
enum : int { SITE_PROBE = 0x7F };
__global__ void wait_probe_kernel(uint64_t limit_ns, int *user_status, int *gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    const Ctl ctl{&abort_flag, user_status};
    const bool ok = bounded_wait(ptx::smem_u32(&bar), 0, ctl, SITE_PROBE, limit_ns);
    if (threadIdx.x == 0 && gave_up) *gave_up = ok ? 0 : 1;
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) !=
                cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return static_cast<EncodeTiledFn>(nullptr);
        return reinterpret_cast<EncodeTiledFn>(sym);
    }();
    return fn;
}

// 3-D map over `batch` row-major pages of `outer` x `inner` elements of `elt` bytes,
// box = box_inner x box_outer x 1, 128-byte swizzle, zero fill outside (loads) / clipping (stores).
// `row_stride` / `page_stride` (elements; 0 = contiguous) place rows and pages further apart.
static int make_map(CUtensorMap *map, int dtype, const void *base, uint64_t inner, uint64_t outer,
                    uint64_t batch, uint32_t box_inner, uint32_t box_outer, uint64_t row_stride = 0,
                    uint64_t page_stride = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(KLAS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const uint64_t elt = dtype_size(dtype);
    if (row_stride == 0) row_stride = inner;
    if (page_stride == 0) page_stride = row_stride * outer;
    const cuuint64_t dims[3] = {inner, outer, batch};
    const cuuint64_t strides[2] = {row_stride * elt, page_stride * elt};
    const cuuint32_t box[3] = {box_inner, box_outer, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapDataType dt = dtype == KLAS_BF16   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                   : dtype == KLAS_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                       : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult rc = fn(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS)
        return fail(KLAS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (inner=%llu outer=%llu batch=%llu)",
                    int(rc), (unsigned long long)inner, (unsigned long long)outer,
                    (unsigned long long)batch);
    return KLAS_OK;
}

template <typename OutT, bool XFORM, bool OLD_C>
static int launch_wide_typed_c(const CUtensorMap &ta, const CUtensorMap &tb, const Params &p, int grid,
                               cudaStream_t stream) {
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        KLAS_TRY_CUDA(cudaFuncSetAttribute(gemm_umma_wide_kernel<OutT, XFORM, OLD_C>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, wide::SMEM_BYTES));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid), 1, 1);
    cfg.blockDim = dim3(wide::THREADS + (XFORM ? XFORM_THREADS : 0), 1, 1);
    cfg.dynamicSmemBytes = wide::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_umma_wide_kernel<OutT, XFORM, OLD_C>, ta, tb, p),
                      "gemm_umma_wide_kernel launch");
}

template <typename OutT, bool XFORM>
static int launch_wide_typed(const CUtensorMap &ta, const CUtensorMap &tb, const Params &p, int grid,
                             cudaStream_t stream) {
    return p.C != nullptr ? launch_wide_typed_c<OutT, XFORM, true>(ta, tb, p, grid, stream)
                          : launch_wide_typed_c<OutT, XFORM, false>(ta, tb, p, grid, stream);
}

template <typename OutT, bool PAIR, bool XFORM, bool OLD_C>
static int launch_typed_c(const CUtensorMap &ta, const CUtensorMap &tb, const Params &p, int grid,
                          cudaStream_t stream) {
    constexpr uint32_t SMEM = Shape<PAIR>::SMEM_BYTES;
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        KLAS_TRY_CUDA(cudaFuncSetAttribute(gemm_umma_kernel<OutT, PAIR, XFORM, OLD_C>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(grid), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS + (XFORM ? XFORM_THREADS : 0), 1, 1);
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR ? 2 : 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return check_cuda(cudaLaunchKernelEx(&cfg, gemm_umma_kernel<OutT, PAIR, XFORM, OLD_C>, ta, tb, p),
                      "gemm_umma_kernel launch");
}

template <typename OutT, bool PAIR, bool XFORM>
static int launch_typed(const CUtensorMap &ta, const CUtensorMap &tb, const Params &p, int grid,
                        cudaStream_t stream) {
    return p.C != nullptr ? launch_typed_c<OutT, PAIR, XFORM, true>(ta, tb, p, grid, stream)
                          : launch_typed_c<OutT, PAIR, XFORM, false>(ta, tb, p, grid, stream);
}

template <bool PAIR, bool XFORM>
static int launch_mode(int out_dtype, const CUtensorMap &ta, const CUtensorMap &tb, const Params &p,
                       int grid, cudaStream_t stream) {
    switch (out_dtype) {
        case KLAS_F32: return launch_typed<float, PAIR, XFORM>(ta, tb, p, grid, stream);
        case KLAS_F16: return launch_typed<__half, PAIR, XFORM>(ta, tb, p, grid, stream);
        default: return launch_typed<__nv_bfloat16, PAIR, XFORM>(ta, tb, p, grid, stream);
    }
}

template <bool XFORM>
static int launch_wide_mode(int out_dtype, const CUtensorMap &ta, const CUtensorMap &tb, const Params &p,
                            int grid, cudaStream_t stream) {
    switch (out_dtype) {
        case KLAS_F32: return launch_wide_typed<float, XFORM>(ta, tb, p, grid, stream);
        case KLAS_F16: return launch_wide_typed<__half, XFORM>(ta, tb, p, grid, stream);
        default: return launch_wide_typed<__nv_bfloat16, XFORM>(ta, tb, p, grid, stream);
    }
}

}  // namespace umma


int umma_ensure_host_flag();

// Workspace of the K-split launches: the partial products.  One buffer per (device, stream) that
// has run a split launch, because launches on different streams may overlap; launches on one
// stream follow one another and share theirs.
namespace {
constexpr int SPLIT_POOL = 8;                        // streams per device with a buffer of their own
struct SplitBuffer {
    cudaStream_t stream = nullptr;
    void *ptr = nullptr;
    size_t cap = 0;
    bool used = false;
};
std::mutex g_split_mutex;
SplitBuffer g_split[64][SPLIT_POOL];
}  // namespace

// Finds or makes the buffer of `stream` with room for `bytes` of partial sums.  Returns KLAS_OK with
// *out = nullptr when none can be had without disturbing the caller (the stream is recording a
// graph and memory would have to be allocated, or the pool is full): the launch then runs unsplit.
static int split_workspace(cudaStream_t stream, size_t bytes, void **out) {
    *out = nullptr;
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return KLAS_OK;
    std::lock_guard<std::mutex> lock(g_split_mutex);
    SplitBuffer *slot = nullptr;
    for (SplitBuffer &b : g_split[dev])
        if (b.used && b.stream == stream) slot = &b;
    if (!slot)
        for (SplitBuffer &b : g_split[dev])
            if (!b.used && !slot) slot = &b;
    if (!slot) return KLAS_OK;
    const size_t want = bytes;
    if (slot->cap < want) {
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (int rc = check_cuda(cudaStreamIsCapturing(stream, &capturing), "cudaStreamIsCapturing")) return rc;
        if (capturing != cudaStreamCaptureStatusNone) return KLAS_OK;
        if (slot->ptr)
            if (int rc = check_cuda(cudaFree(slot->ptr), "cudaFree")) return rc;   // waits for the device
        *slot = SplitBuffer{};
        void *fresh = nullptr;
        if (int rc = check_cuda(cudaMalloc(&fresh, want), "cudaMalloc (K-split workspace)")) return rc;
        slot->ptr = fresh;
        slot->cap = want;
        slot->stream = stream;
        slot->used = true;
    }
    *out = slot->ptr;
    return KLAS_OK;
}

int umma_release_split_workspace() {
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return KLAS_OK;
    std::lock_guard<std::mutex> lock(g_split_mutex);
    for (SplitBuffer &b : g_split[dev]) {
        if (b.ptr)
            if (int rc = check_cuda(cudaFree(b.ptr), "cudaFree")) return rc;
        b = SplitBuffer{};
    }
    return KLAS_OK;
}

int umma_wait_probe(uint32_t limit_ms, int *gave_up, cudaStream_t stream) {
    if (int rc = umma_ensure_host_flag()) return rc;
    umma::wait_probe_kernel<<<1, 32, 0, stream>>>(uint64_t(limit_ms) * 1000000ull, nullptr, gave_up);
    return check_cuda(cudaGetLastError(), "wait_probe_kernel launch");
}

// Device address of the status word, for other kernels of the library that use bounded waits.
int umma_status_address(int **out) {
    void *ptr = nullptr;
    KLAS_TRY_CUDA(cudaGetSymbolAddress(&ptr, umma::g_umma_status));
    *out = static_cast<int *>(ptr);
    return KLAS_OK;
}

// 3-D tiled tensor map with 128-byte swizzle (see umma::make_map), for the attention kernel.
int make_tensor_map_3d(CUtensorMap *map, int dtype, const void *base, uint64_t inner, uint64_t outer, uint64_t batch,
                       uint32_t box_inner, uint32_t box_outer) {
    return umma::make_map(map, dtype, base, inner, outer, batch, box_inner, box_outer);
}

// The host-visible mirror of the status word: one mapped int per device, created before the first
// launch on that device and kept for the life of the process.
static std::mutex g_flag_mutex;
static volatile int *g_host_flags[64] = {};

int umma_ensure_host_flag() {
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return KLAS_OK;   // no mirror: callers fall back to the device word
    std::lock_guard<std::mutex> lock(g_flag_mutex);
    if (g_host_flags[dev]) return KLAS_OK;
    int *h = nullptr, *d = nullptr;
    KLAS_TRY_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&h), sizeof(int), cudaHostAllocMapped));
    *h = 0;
    KLAS_TRY_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&d), h, 0));
    KLAS_TRY_CUDA(cudaMemcpyToSymbol(umma::g_umma_host_flag, &d, sizeof(d)));
    g_host_flags[dev] = h;
    return KLAS_OK;
}

// 0 when no bounded wait has given up on this device since the last clear, else its site code.
// Exact only after the launches of interest have been synchronised with.
int umma_peek_status() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    volatile int *h = g_host_flags[dev];
    return h ? *h : 0;
}

int umma_read_status(int *value) {
    return check_cuda(cudaMemcpyFromSymbol(value, umma::g_umma_status, sizeof(int)),
                      "cudaMemcpyFromSymbol(status)");
}

int umma_clear_status() {
    const int zero = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_host_flags[dev]) *g_host_flags[dev] = 0;
    return check_cuda(cudaMemcpyToSymbol(umma::g_umma_status, &zero, sizeof(int)),
                      "cudaMemcpyToSymbol(status)");
}

int launch_gemm_umma(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                     uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                     void *D, float alpha, float beta, int *status_word, cudaStream_t stream) {
    return launch_gemm_umma_fused(in_dtype, out_dtype, b_major, batch, rows, shared, cols, A, B, C, D, alpha, beta,
                                  KLAS_MAP_ID, KLAS_MAP_ID, C ? KLAS_COMB_AXPBY : KLAS_COMB_NEW, status_word, stream);
}

int launch_gemm_umma_fused(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                           uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                           void *D, float alpha, float beta, int map_a, int map_b, int comb,
                           int *status_word, cudaStream_t stream) {
    TcStrides st{};   // all zero: contiguous
    return launch_gemm_umma_strided(in_dtype, out_dtype, b_major, batch, rows, shared, cols, A, B, C, D, st, alpha, beta,
                                    map_a, map_b, comb, status_word, stream);
}

// What a launch of the given shape will run: kernel, tile width, K parts, whether the last round is cut.
// Pure host arithmetic on the shape, the SM count and the tuning knobs (klas_b200_gemm_tc_plan
// exposes it, so the choice can be tested without a GPU).
struct TilePlan {
    bool use_wide, pair, tail_split;
    uint32_t single_tile_n;
    uint64_t auto_parts;
};

static TilePlan plan_tiles(uint64_t rows, uint64_t cols, uint64_t shared, uint32_t batch, bool xform, int sm_count) {
    using namespace umma;
    // Tile shape: single CTAs with 128 x 256 tiles, CTA pairs with 256 x 256 tiles, or "wide" CTA
    // pairs with 512 x 256 tiles, whichever a wave count x tile cost estimate makes fastest.  The
    // kernels are persistent with a static round-robin of tiles, so a launch takes
    // ceil(tiles / slots) rounds; per round a wide tile costs twice a 256 x 256 one, less what it
    // saves by sharing operands.  The relative rates are the 8192^3 row of the tuning run
    // `python -m kuiper_b200.tune_tc` (TFLOP/s of each tile shape where all of them fill the
    // machine); re-run it and update the three constants when a kernel changes.
    // Examples the estimate gets right where "wide once it fills the machine"
    // did not: 3072^3 (72 wide tiles, one round: 1388 against 1267 TFLOP/s for two rounds of single tiles),
    // 3584 x 3072 (84 wide tiles would take two rounds; pairs: 1167 against 959), 2048^2 (one
    // round of 128 single tiles: 896 against 600 for 32 wide tiles on 74 pairs).
    // The KLAS_KNOB_TC_MODE knob overrides the choice.
    constexpr double RATE_SINGLE = 1336.0, RATE_PAIR = 1433.0, RATE_WIDE = 1539.0, WIDE_DRAIN_KB = 6.0, PAIR_TILE_KB = 1.3, NARROW_COST = 0.75, SLIM_COST = 0.65;
    constexpr uint32_t SPLIT_MIN_SAVED_KB = 22;   // K blocks (of 64) a split must take off a tile to pay for its second kernel
    constexpr double TAIL_OVERHEAD_KB = 45.0;     // what the extra launch and the adding kernel of a cut last round cost, in K blocks
    const uint64_t single_tiles = ((rows + BM - 1) / BM) * ((cols + BN - 1) / BN) * batch;
    const uint64_t pair_tiles = ((rows + 2 * BM - 1) / (2 * BM)) * ((cols + BN - 1) / BN) * batch;
    const uint64_t wide_tiles = ((rows + wide::TILE_M - 1) / wide::TILE_M) * ((cols + BN - 1) / BN) * batch;
    const bool can_pair = sm_count >= 2;
    const uint64_t sms = uint64_t(sm_count), pairs = uint64_t(sm_count / 2);
    const double cost_single = double((single_tiles + sms - 1) / sms);
    const bool pair_ok = can_pair && rows > BM && single_tiles >= sms && !xform;   // the pair tile has no mapped form
    const double num_kb_d = double((shared + BK - 1) / BK);
    // A pair tile's fixed cost (cluster hand-shakes per tile) weighs more the shorter K is: at
    // 8192 x 8192 x 512 single tiles measured 801 against 749 TFLOP/s, at K = 8192 1336 against 1433.
    const double pair_short_k = num_kb_d > 0 ? (1.0 + PAIR_TILE_KB / num_kb_d) / (1.0 + PAIR_TILE_KB / 128.0) : 1.0;
    const double pair_rate = (RATE_SINGLE / RATE_PAIR) * pair_short_k;
    const double cost_pair = pair_ok ? double((pair_tiles + pairs - 1) / pairs) * pair_rate : 1e30;
    // The wide tile's epilogue is not hidden behind the next tile's MMAs (both accumulator halves
    // belong to one tile): about six K blocks' worth per tile, which the rate measured at K = 8192
    // contains once per 128 K blocks.  8192 x 8192 x 512: single tiles 791, wide 708 TFLOP/s.
    const double wide_drain = num_kb_d > 0 ? (1.0 + WIDE_DRAIN_KB / num_kb_d) / (1.0 + WIDE_DRAIN_KB / 128.0) : 1.0;
    const double cost_wide = can_pair ? double((wide_tiles + pairs - 1) / pairs) * 2.0 * (RATE_SINGLE / RATE_WIDE) * wide_drain : 1e30;
    // A part-filled last round of single or pair tiles can be cut along K so that it fills the machine
    // too (second launch + the kernel that adds the parts: about TAIL_OVERHEAD_KB K blocks' worth).
    const uint64_t num_kb_all = (shared + BK - 1) / BK;
    auto with_tail_cut = [&](uint64_t tiles, uint64_t slots) -> double {   // rounds, or 1e30 where it does not apply
        const uint64_t rem = tiles % slots, full = tiles / slots;
        if (batch != 1 || rem == 0 || full == 0 || num_kb_all == 0) return 1e30;
        uint64_t parts = slots / rem;
        if (parts > 8) parts = 8;
        if (parts < 2) return 1e30;
        const uint64_t kb_per = (num_kb_all + parts - 1) / parts;
        if (num_kb_all < kb_per + SPLIT_MIN_SAVED_KB) return 1e30;
        return double(full) + double(kb_per) / double(num_kb_all) + TAIL_OVERHEAD_KB / double(num_kb_all);
    };
    const double cost_single_tail = with_tail_cut(single_tiles, sms);
    const double cost_pair_tail = pair_ok ? with_tail_cut(pair_tiles, pairs) * pair_rate : 1e30;
    const double best_single = cost_single_tail < cost_single ? cost_single_tail : cost_single;
    const double best_pair = cost_pair_tail < cost_pair ? cost_pair_tail : cost_pair;
    bool use_wide = can_pair && cost_wide < best_single && cost_wide <= best_pair;
    bool pair = pair_ok && !use_wide && best_pair <= best_single;
    bool tail_split = !use_wide && (pair ? cost_pair_tail < cost_pair : cost_single_tail < cost_single);
    // Small outputs: the single-CTA kernel with 128-column tiles puts twice as many CTAs to work
    // (1024^2: 64 tiles instead of 32 on 148 SMs).  A CTA takes the same time per K block whatever
    // the tile's width (about 660 cycles: the copy-issue and MMA-issue threads, not the arithmetic,
    // set it), so a narrower tile only pays through its shorter prologue and epilogue when the
    // round count stays the same (2048^2, K = 2048: one round of 128 x 256 tiles 19.4 us, two
    // rounds of 128 x 128 29.2 us, four of 128 x 64 50.0 us).
    // Smaller still (1024^2: 128 tiles of 128 x 64) when even the 128-column tiles leave SMs idle.
    const uint64_t narrow_tiles = ((rows + BM - 1) / BM) * ((cols + 127) / 128) * batch;
    const uint64_t slim_tiles = ((rows + BM - 1) / BM) * ((cols + 63) / 64) * batch;
    const double cost_narrow = double((narrow_tiles + sms - 1) / sms) * NARROW_COST;
    const double cost_slim = double((slim_tiles + sms - 1) / sms) * SLIM_COST;
    uint32_t single_tile_n = BN;
    if (!use_wide && !pair) {
        double best = best_single;
        if (cost_narrow < best) best = cost_narrow, single_tile_n = 128, tail_split = false;
        if (cost_slim < best) best = cost_slim, single_tile_n = 64, tail_split = false;
    }
    // Long K over few tiles: cut each 128 x 256 tile's K range into parts that fill the SMs
    // (1024 x 1024 x 4096: 32 tiles x 4 parts, 17.3 us against 27.4 us for 128 tiles of 128 x 64).
    // A split costs a second kernel that adds the parts (4-6 us for a 1024^2 output), a K block 0.34 us.
    uint64_t auto_parts = 1;
    if (!use_wide && !pair && single_tiles * 2 <= sms && debug_knob(KLAS_KNOB_TC_MODE) == 0) {
        uint64_t parts = sms / single_tiles;
        if (parts > 8) parts = 8;
        const uint64_t kb_per = (num_kb_all + parts - 1) / parts;
        if (num_kb_all >= kb_per + SPLIT_MIN_SAVED_KB) {
            auto_parts = parts;
            single_tile_n = BN;
        }
    }
    if (debug_knob(KLAS_KNOB_TC_MODE) != 0) tail_split = false;   // forced shapes run one launch unless KLAS_KNOB_TC_TAIL asks
    switch (debug_knob(KLAS_KNOB_TC_MODE)) {   // a test or tuning run forcing one tile shape
        case 1: pair = use_wide = false; single_tile_n = BN; break;
        case 2: pair = use_wide = false; single_tile_n = 128; break;
        case 3: pair = can_pair && !xform; use_wide = false; break;
        case 4: use_wide = can_pair; break;
        case 5: pair = use_wide = false; single_tile_n = 64; break;
        default: break;
    }
    return TilePlan{use_wide, pair, tail_split, single_tile_n, auto_parts};
}

int umma_plan(uint64_t rows, uint64_t shared, uint64_t cols, uint32_t batch, int sm_count, int *kind, int *tile_cols,
              int *k_parts, int *tail_cut) {
    if (sm_count < 1 || batch == 0) return fail(KLAS_ERR_INVALID, "gemm_tc_plan: sm_count and batch must be positive");
    const TilePlan pl = plan_tiles(rows, cols, shared, batch, false, sm_count);
    const uint64_t sms = uint64_t(sm_count), pairs = uint64_t(sm_count / 2);
    if (kind) *kind = pl.use_wide ? 2 : (pl.pair ? 1 : 0);
    if (tile_cols) *tile_cols = (pl.use_wide || pl.pair) ? int(umma::BN) : int(pl.single_tile_n);
    int parts = 1, tail = 0;
    if (!pl.use_wide) {
        const int knob = debug_knob(KLAS_KNOB_TC_KSPLIT);
        uint64_t want = knob >= 2 ? uint64_t(knob) : (knob == 0 ? pl.auto_parts : 1);
        const uint64_t num_kb = (shared + umma::BK - 1) / umma::BK;
        if (want > 8) want = 8;
        if (want > num_kb) want = num_kb;
        if (want >= 2) {
            const uint64_t kb_per = (num_kb + want - 1) / want;
            want = (num_kb + kb_per - 1) / kb_per;
        }
        parts = want >= 2 ? int(want) : 1;
        const uint64_t tile_m = pl.pair ? 2 * umma::BM : umma::BM, tile_n = pl.pair ? umma::BN : pl.single_tile_n;
        const uint64_t tiles = ((rows + tile_m - 1) / tile_m) * ((cols + tile_n - 1) / tile_n) * batch;
        const uint64_t slots = pl.pair ? pairs : sms;
        const int tknob = debug_knob(KLAS_KNOB_TC_TAIL);
        const uint64_t rem = slots ? tiles % slots : 0;
        if (parts == 1 && batch == 1 && rem > 0 && tiles > rem && slots / rem >= 2 && num_kb >= 2 &&
            (tknob == 2 || (tknob == 0 && pl.tail_split)))
            tail = 1;
    }
    if (k_parts) *k_parts = parts;
    if (tail_cut) *tail_cut = tail;
    return KLAS_OK;
}

int launch_gemm_umma_strided(int in_dtype, int out_dtype, int b_major, uint32_t batch, uint64_t rows,
                             uint64_t shared, uint64_t cols, const void *A, const void *B, const void *C,
                             void *D, const TcStrides &st, float alpha, float beta, int map_a, int map_b, int comb,
                             int *status_word, cudaStream_t stream) {
    using namespace umma;
    // rows of A are `shared` long; rows of B `cols` (row-major) or `shared` (column-major) long
    const uint64_t b_inner = b_major == KLAS_B_ROW_MAJOR ? cols : shared, b_outer = b_major == KLAS_B_ROW_MAJOR ? shared : cols;
    const uint64_t lda = st.lda ? st.lda : shared, ldb = st.ldb ? st.ldb : b_inner, ldd = st.ldd ? st.ldd : cols;
    const uint64_t sa = st.stride_a ? st.stride_a : lda * rows, sb = st.stride_b ? st.stride_b : ldb * b_outer,
                   sd = st.stride_d ? st.stride_d : ldd * rows;
    if (lda < shared || ldb < b_inner || ldd < cols) return fail(KLAS_ERR_INVALID, "gemm_tc: a row stride is shorter than the row");
    if ((lda | ldb | ldd | sa | sb | sd) % 8 != 0)
        return fail(KLAS_ERR_UNSUPPORTED, "gemm_tc: row and page strides must be multiples of 8 elements");
    if (batch > 1 && sd < (rows - 1) * ldd + cols) return fail(KLAS_ERR_INVALID, "gemm_tc: pages of D overlap");
    if (map_a < KLAS_MAP_ID || map_a > KLAS_MAP_NEG || map_b < KLAS_MAP_ID || map_b > KLAS_MAP_NEG)
        return fail(KLAS_ERR_INVALID, "gemm_tc: unknown operand map (%d, %d)", map_a, map_b);
    if (comb < KLAS_COMB_NEW || comb > KLAS_COMB_SCALED) return fail(KLAS_ERR_INVALID, "gemm_tc: unknown combine rule %d", comb);
    const bool reads_c = comb != KLAS_COMB_NEW && comb != KLAS_COMB_RELU && comb != KLAS_COMB_SCALED;
    if (reads_c && !C && rows && cols && batch) return fail(KLAS_ERR_INVALID, "gemm_tc: this combine rule needs C");
    if (!reads_c) C = nullptr;
    const bool xform = (map_a != KLAS_MAP_ID || map_b != KLAS_MAP_ID) && shared > 0;
    if (in_dtype != KLAS_BF16 && in_dtype != KLAS_F16)
        return fail(KLAS_ERR_INVALID, "gemm_tc: in_dtype must be KLAS_BF16 or KLAS_F16");
    if (out_dtype != KLAS_F32 && out_dtype != KLAS_F16 && out_dtype != KLAS_BF16)
        return fail(KLAS_ERR_INVALID, "gemm_tc: out_dtype must be KLAS_F32, KLAS_F16 or KLAS_BF16");
    if (b_major != KLAS_B_ROW_MAJOR && b_major != KLAS_B_COL_MAJOR)
        return fail(KLAS_ERR_INVALID, "gemm_tc: bad b_major");
    if (rows == 0 || cols == 0 || batch == 0) return KLAS_OK;
    if (!D || (shared > 0 && (!A || !B)))
        return fail(KLAS_ERR_INVALID, "gemm_tc: null matrix pointer");
    if (int rc = umma_ensure_host_flag()) return rc;
    if (shared % 8 != 0 || cols % 8 != 0)
        return fail(KLAS_ERR_UNSUPPORTED,
                    "gemm_tc: shared (%llu) and cols (%llu) must be multiples of 8",
                    (unsigned long long)shared, (unsigned long long)cols);
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
         reinterpret_cast<uintptr_t>(C) | reinterpret_cast<uintptr_t>(D)) & 15u)
        return fail(KLAS_ERR_INVALID, "gemm_tc: A, B, C, D must be 16-byte aligned");
    if (rows > 0x7fffffffull || cols > 0x7fffffffull || shared > 0x7fffffffull)
        return fail(KLAS_ERR_TOO_LARGE, "gemm_tc: dimension beyond 2^31-1");

    DeviceInfo info;
    if (int rc = device_info(&info)) return rc;
    if (info.cc_major != 10)
        return fail(KLAS_ERR_UNSUPPORTED, "gemm_tc needs an sm_100 device (found sm_%d%d)",
                    info.cc_major, info.cc_minor);

    const TilePlan plan = plan_tiles(rows, cols, shared, batch, xform, info.sm_count);
    const bool use_wide = plan.use_wide, pair = plan.pair, tail_split = plan.tail_split;
    const uint32_t single_tile_n = plan.single_tile_n;
    const uint64_t auto_parts = plan.auto_parts;
    const uint64_t sms = uint64_t(info.sm_count), pairs = uint64_t(info.sm_count / 2);
    const uint64_t wide_tiles = ((rows + wide::TILE_M - 1) / wide::TILE_M) * ((cols + BN - 1) / BN) * batch;
    if (use_wide) {
        Params p{};
        p.C = C;
        p.D = D;
        p.M = uint32_t(rows);
        p.N = uint32_t(cols);
        p.K = uint32_t(shared);
        p.batch = batch;
        p.tiles_m = uint32_t((rows + wide::TILE_M - 1) / wide::TILE_M);
        p.tiles_n = uint32_t((cols + BN - 1) / BN);
        if (wide_tiles > 0xffffffffull) return fail(KLAS_ERR_TOO_LARGE, "gemm_tc: too many tiles");
        p.num_tiles = uint32_t(wide_tiles);
        p.num_kb = uint32_t((shared + BK - 1) / BK);
        p.ldd = ldd;
        p.sd = sd;
        p.alpha = alpha;
        p.beta = beta;
        p.b_row_major = (b_major == KLAS_B_ROW_MAJOR) ? 1u : 0u;
        p.idesc = ptx::umma_idesc_f16(in_dtype == KLAS_BF16, false, p.b_row_major != 0, 256, BN);
        p.status = status_word;
        p.in_bf16 = in_dtype == KLAS_BF16 ? 1u : 0u;
        p.map_a = uint32_t(map_a);
        p.map_b = uint32_t(map_b);
        p.comb = uint32_t(comb);
        p.raster_group = DEFAULT_RASTER_GROUP;
        if (const int v = debug_knob(KLAS_KNOB_TC_RASTER); v >= 1) p.raster_group = uint32_t(v);
        CUtensorMap ta{}, tb{};
        if (shared > 0) {
            if (int rc = make_map(&ta, in_dtype, A, shared, rows, batch, BK, wide::A_ROWS, lda, sa)) return rc;
            if (p.b_row_major) {
                if (int rc = make_map(&tb, in_dtype, B, cols, shared, batch, 64, BK, ldb, sb)) return rc;
            } else {
                if (int rc = make_map(&tb, in_dtype, B, shared, cols, batch, BK, wide::B_COLS, ldb, sb)) return rc;
            }
        }
        const uint64_t groups = wide_tiles < uint64_t(info.sm_count / 2) ? wide_tiles : uint64_t(info.sm_count / 2);
        return xform ? launch_wide_mode<true>(out_dtype, ta, tb, p, int(groups * 2), stream)
                     : launch_wide_mode<false>(out_dtype, ta, tb, p, int(groups * 2), stream);
    }
    const uint32_t tile_m = pair ? Shape<true>::TILE_M : Shape<false>::TILE_M;

    Params p{};
    p.C = C;
    p.D = D;
    p.M = uint32_t(rows);
    p.N = uint32_t(cols);
    p.K = uint32_t(shared);
    p.batch = batch;
    p.tile_n = pair ? BN : single_tile_n;
    p.stage_bytes = A_STAGE_BYTES + p.tile_n * BK * 2u;
    p.stages = RING_BYTES / p.stage_bytes;   // 4 x 48, 6 x 32 or 8 x 24 KiB
    p.tiles_m = uint32_t((rows + tile_m - 1) / tile_m);
    p.tiles_n = uint32_t((cols + p.tile_n - 1) / p.tile_n);
    const uint64_t num_tiles = uint64_t(p.tiles_m) * p.tiles_n * batch;
    if (num_tiles > 0xffffffffull) return fail(KLAS_ERR_TOO_LARGE, "gemm_tc: too many tiles");
    p.num_tiles = uint32_t(num_tiles);
    p.num_kb = uint32_t((shared + BK - 1) / BK);
    p.ldd = ldd;
    p.sd = sd;
    p.alpha = alpha;
    p.beta = beta;
    p.b_row_major = (b_major == KLAS_B_ROW_MAJOR) ? 1u : 0u;
    p.idesc = ptx::umma_idesc_f16(in_dtype == KLAS_BF16, false, p.b_row_major != 0, tile_m, p.tile_n);
    p.status = status_word;
    p.in_bf16 = in_dtype == KLAS_BF16 ? 1u : 0u;
    p.map_a = uint32_t(map_a);
    p.map_b = uint32_t(map_b);
    p.comb = uint32_t(comb);
    p.raster_group = DEFAULT_RASTER_GROUP;
    if (const int v = debug_knob(KLAS_KNOB_TC_RASTER); v >= 1) p.raster_group = uint32_t(v);

    // One launch covers a range of the tile list, whole or with each tile's K range cut into parts.
    // Cut tiles write f32 partial products into a workspace and a second kernel adds them in index
    // order and applies the output rule (alpha, beta, the old C, the output type), so the result is
    // the same from run to run.  Two plans use that:
    //  * every tile cut (few tiles, long K: chosen above, or forced by KLAS_KNOB_TC_KSPLIT);
    //  * only the tiles of a part-filled last round cut, so that they fill the machine too, after a
    //    first launch for the full rounds (2560 x 2048 x 4096 in pair tiles: 74 tiles whole, then
    //    6 tiles x 8 parts, instead of two rounds).
    struct Pass {
        uint32_t tile0, tiles, parts, kb_per;
    };
    const uint64_t slots = pair ? pairs : sms;
    Pass first{0, uint32_t(num_tiles), 1, p.num_kb}, tail{0, 0, 1, p.num_kb};
    float *split_ws = nullptr;
    auto parts_for = [&](uint64_t want, Pass &pass) {   // settles parts and K blocks per part; false: stay whole
        if (want > 8) want = 8;
        if (want > p.num_kb) want = p.num_kb;
        if (want < 2) return false;
        const uint32_t kb_per = uint32_t((p.num_kb + want - 1) / want);
        want = (p.num_kb + kb_per - 1) / kb_per;   // no empty part
        if (want < 2) return false;
        pass.parts = uint32_t(want);
        pass.kb_per = kb_per;
        return true;
    };
    {
        const int knob = debug_knob(KLAS_KNOB_TC_KSPLIT);
        const uint64_t want = knob >= 2 ? uint64_t(knob) : (knob == 0 ? auto_parts : 1);
        Pass cut = first;
        if (want >= 2 && parts_for(want, cut)) {
            void *ws = nullptr;
            if (int rc = split_workspace(stream, size_t(batch) * cut.parts * rows * cols * sizeof(float), &ws)) return rc;
            if (ws != nullptr) {
                first = cut;
                split_ws = static_cast<float *>(ws);
            }
        }
    }
    if (first.parts == 1 && batch == 1 && num_tiles > 0) {
        const int knob = debug_knob(KLAS_KNOB_TC_TAIL);
        const uint64_t rem = num_tiles % slots, full = num_tiles - rem;
        const bool wanted = knob == 2 || (knob == 0 && tail_split);
        Pass cut{uint32_t(full), uint32_t(rem), 1, p.num_kb};
        if (wanted && rem > 0 && full > 0 && parts_for(slots / rem, cut)) {
            const size_t bytes = size_t(cut.parts) * rows * cols * sizeof(float);
            void *ws = nullptr;
            if (bytes <= (size_t(1) << 30))
                if (int rc = split_workspace(stream, bytes, &ws)) return rc;
            if (ws != nullptr) {
                first.tiles = uint32_t(full);
                tail = cut;
                split_ws = static_cast<float *>(ws);
            }
        }
    }

    const uint32_t b_cols = pair ? Shape<true>::B_COLS : p.tile_n;
    CUtensorMap ta{}, tb{};
    if (shared > 0) {
        if (int rc = make_map(&ta, in_dtype, A, shared, rows, batch, BK, BM, lda, sa)) return rc;
        if (p.b_row_major) {
            if (int rc = make_map(&tb, in_dtype, B, cols, shared, batch, 64, BK, ldb, sb)) return rc;
        } else {
            if (int rc = make_map(&tb, in_dtype, B, shared, cols, batch, BK, b_cols, ldb, sb)) return rc;
        }
    }
    auto run = [&](const Pass &pass) -> int {
        Params q = p;
        q.tile0 = pass.tile0;
        q.num_tiles = pass.tiles;
        q.ksplit = pass.parts;
        q.kb_per = pass.parts > 1 ? pass.kb_per : p.num_kb;
        const uint64_t num_work = uint64_t(pass.tiles) * pass.parts;
        q.num_work = uint32_t(num_work);
        int kernel_out_dtype = out_dtype;
        if (pass.parts > 1) {
            // the product kernel writes plain f32 parts; the output rule moves to the second kernel
            q.C = nullptr;
            q.D = split_ws;
            q.ldd = cols;
            q.sd = rows * cols;
            q.comb = KLAS_COMB_NEW;
            q.alpha = 1.0f;
            q.beta = 0.0f;
            kernel_out_dtype = KLAS_F32;
        }
        int rc;
        if (pair) {
            const uint64_t groups = num_work < pairs ? num_work : pairs;
            rc = launch_mode<true, false>(kernel_out_dtype, ta, tb, q, int(groups * 2), stream);
        } else {
            const int grid = int(num_work < sms ? num_work : sms);
            rc = xform ? launch_mode<false, true>(kernel_out_dtype, ta, tb, q, grid, stream)
                       : launch_mode<false, false>(kernel_out_dtype, ta, tb, q, grid, stream);
        }
        if (rc != KLAS_OK || pass.parts == 1) return rc;
        ReduceArgs ra{split_ws, C, D, uint32_t(rows), uint32_t(cols), pass.parts, batch, ldd, sd, alpha, beta, uint32_t(comb),
                      pass.tile0, tile_m, p.tile_n, p.tiles_m, p.tiles_n, p.raster_group};
        const uint64_t threads = pass.tile0 > 0 ? uint64_t(pass.tiles) * tile_m * (p.tile_n / 4) : uint64_t(batch) * rows * (cols / 4);
        uint64_t blocks = (threads + 255) / 256;
        if (blocks > sms * 8) blocks = sms * 8;
        if (blocks == 0) blocks = 1;
        switch (out_dtype) {
            case KLAS_F32: splitk_reduce_kernel<float><<<unsigned(blocks), 256, 0, stream>>>(ra); break;
            case KLAS_F16: splitk_reduce_kernel<__half><<<unsigned(blocks), 256, 0, stream>>>(ra); break;
            default: splitk_reduce_kernel<__nv_bfloat16><<<unsigned(blocks), 256, 0, stream>>>(ra); break;
        }
        return check_cuda(cudaGetLastError(), "splitk_reduce_kernel launch");
    };
    if (int rc = run(first)) return rc;
    if (tail.tiles > 0) return run(tail);
    return KLAS_OK;
}

}  // namespace klas
