// Fused scaled-dot-product attention for sm_100a:  O = softmax(scale * Q.K^T) . V  per head,
// without ever writing the score matrix to global memory.
//
// One CTA owns 128 query rows of one head and walks the keys 128 at a time:
//   warp 0      TMA producer: Q once, then K and V tiles through a two-stage ring;
//   warp 1      owns tensor memory; one thread issues S_j = Q.K_j^T into one of two 128-column score
//               buffers (so S_(j+1) is being multiplied while the softmax warps work on S_j);
//   warp 2      one thread issues O += P_j.V_j into a third region of tensor memory;
//   warps 3-10  two threads per query row (= TMEM lane), one for keys 0-63 of the tile and columns
//               0 .. E/2 of O, one for the other halves: read their part of the row of S_j twice
//               (maximum, then exponentials), exchange the partial maxima through shared memory,
//               keep a reference point m and a partial sum l, write P_j = exp(S_j - m) as a 16-bit,
//               128-byte-swizzled A operand into shared memory.  O accumulates in tensor memory across
//               the tiles; m follows the running maximum only in steps of 2^8 or more, and only then
//               are O (tcgen05.ld / st) and l rescaled.
// Where a tile's time goes (cycle counters of one softmax warp, in a scratch build): of ~2950 cycles
// per 128 x 128 tile at E = 128, 1340 are the exponentials -- the special-function unit's rate for
// the two warps of a scheduler, 2 x 64 x 8 cycles -- and the rest is the serial chain around them
// (wait for S and load it 540, maximum 200, exchange 300, wait for the previous P.V 275, store and
// publish P 290); the tensor core needs 1024.  One thread per row took 3950 cycles, four per row
// gained nothing over two, and issuing the two products from one thread or from two made no
// difference.  Also tried and measured no better: two independent streams of tiles per CTA (even /
// odd tiles, each with its own scores, P, O, producer and issuing thread, combined at the end, the
// second started half a period late), and a single optimistic pass per tile with the inherited
// reference point.  The warps are bound by instruction issue, not by the special-function unit:
// every instruction per score costs the two warps of a scheduler two cycles per key, so the next
// step is fewer instructions per score, not more overlap.  (One try at that, also measured: for f16,
// rounding the exponent's argument to f16 and taking two exponentials per special-function operation,
// with the row sum added pairwise in f16 first -- 5.75 instead of 7 instructions per pair of scores
// -- ran 5 % slower, 666 against 700 TFLOP/s at 256 heads of 2048 x 128; not kept.)
// K is a K-major B operand (its rows are the columns of K^T), V an MN-major one, P a K-major A
// operand: the three layouts the GEMM kernel uses, with the same descriptors.
// Exponentials are ex2 of a pre-scaled argument (scale * log2 e folded into one multiply).
// All hand-offs are mbarriers with bounded waits; a wait that gives up raises the library's
// tensor-core status word and every role drains.
//
// Takes over the work of the reference's attention kernels, which exist in its F* sources only:
// src/lib/kernel/Kuiper.Kernel.SDPA.Naive.fst:390-470 (GEMM, row softmax, GEMM through global
// memory) and src/lib/kernel/Kuiper.Kernel.FlashAttention.fst (one thread block per query tile,
// running maximum and sum per row).
#include <atomic>

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "klas_internal.h"
#include "ptx_sm100.cuh"

namespace klas {
namespace fa {

constexpr uint32_t BM = 128;          // query rows per CTA (= TMEM lanes)
constexpr uint32_t BN = 128;          // keys per step
constexpr uint32_t SOFTMAX_WARPS = 8;
constexpr uint32_t FIRST_SOFTMAX_WARP = 3;    // warp 0 producer, warp 1 Q.K^T issuer, warp 2 P.V issuer
constexpr uint32_t THREADS = (FIRST_SOFTMAX_WARP + SOFTMAX_WARPS) * 32;
constexpr uint32_t STAGES = 2;
constexpr uint32_t ATOM_BYTES = 128 * 128;   // 128 rows x one 128-byte swizzle row
constexpr uint32_t TMEM_COLS = 512;          // S0 at 0, S1 at 128, O at 256
constexpr uint64_t WAIT_LIMIT_NS = 1000ull * 1000ull * 1000ull;

enum : int { SITE_FA = 0x200 };


template <uint32_t E>
struct Cfg {
    static constexpr uint32_t ATOMS = E / 64;             // swizzle atoms along the head dimension
    static constexpr uint32_t TILE_BYTES = ATOMS * ATOM_BYTES;   // a 128 x E tile of Q, K or V
    static constexpr uint32_t P_BYTES = 2 * ATOM_BYTES;   // 128 x 128 probabilities
    // (value, tag) words the two threads of a row exchange: partial maxima [tile parity][key half][row],
    // then the partial sums [key half][row]
    static constexpr uint32_t XCHG_BYTES = (2 * 2 * BM + 2 * BM) * 8;
    static constexpr uint32_t SMEM = TILE_BYTES * (1 + 2 * STAGES) + P_BYTES + XCHG_BYTES + 256 + 1024;
};

struct Params {
    void *out;
    uint32_t L, S, pages, num_kv;
    float scale_log2;      // scale * log2(e)
    uint32_t idesc_qk, idesc_pv;
    uint32_t bf16;
    int *status;           // the library's tensor-core status word
};

struct Ctl {
    volatile int *abort_flag;
    int *status;
};

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, const Ctl &ctl, int site, uint32_t backoff_ns = 0) {
    // `backoff_ns` > 0: a role whose wait may be long polls with a suspend-time hint (the hardware parks
    // the thread and wakes it when the phase completes) instead of spinning
    auto poll = [&] { return backoff_ns ? ptx::mbar_try_wait_hint(bar, parity, backoff_ns * 32u) : ptx::mbar_try_wait(bar, parity); };
    if (poll()) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (poll()) return true;
        if ((++spins & 0x3F) == 0) {
            if (*ctl.abort_flag != 0) return false;
            if (ptx::globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                *ctl.abort_flag = 1;
                if (ctl.status) atomicCAS(ctl.status, 0, SITE_FA | site);
                __threadfence();
                return false;
            }
        }
    }
}

__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ uint32_t pack16(float lo, float hi, bool bf16) {
    if (bf16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t *>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t *>(&v);
}

template <uint32_t E>
__global__ void __launch_bounds__(THREADS, 1)
    sdpa_fused_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
    using C = Cfg<E>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t *smem = smem_raw + pad;
    const uint32_t smem_base = raw_addr + pad;
    const uint32_t q_base = smem_base;
    auto k_base = [&](uint32_t s) { return smem_base + C::TILE_BYTES * (1 + s); };
    auto v_base = [&](uint32_t s) { return smem_base + C::TILE_BYTES * (1 + STAGES + s); };
    const uint32_t p_base = smem_base + C::TILE_BYTES * (1 + 2 * STAGES);
    volatile unsigned long long *xchg =
        reinterpret_cast<volatile unsigned long long *>(smem + C::TILE_BYTES * (1 + 2 * STAGES) + C::P_BYTES);
    for (uint32_t i = threadIdx.x; i < C::XCHG_BYTES / 8; i += THREADS) xchg[i] = 0ull;   // tag 0 = nothing yet
    const uint32_t bar_base = p_base + C::P_BYTES + C::XCHG_BYTES;
    uint8_t *bar_region = smem + C::TILE_BYTES * (1 + 2 * STAGES) + C::P_BYTES + C::XCHG_BYTES;
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_free[2], p_full, o_full
    const uint32_t q_full = bar_base;
    auto k_full = [&](uint32_t s) { return bar_base + 8u * (1 + s); };
    auto k_empty = [&](uint32_t s) { return bar_base + 8u * (3 + s); };
    auto v_full = [&](uint32_t s) { return bar_base + 8u * (5 + s); };
    auto v_empty = [&](uint32_t s) { return bar_base + 8u * (7 + s); };
    auto s_full = [&](uint32_t b) { return bar_base + 8u * (9 + b); };
    auto s_free = [&](uint32_t b) { return bar_base + 8u * (11 + b); };
    const uint32_t p_full = bar_base + 8u * 13;
    const uint32_t o_full = bar_base + 8u * 14;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_region + 8u * 15);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles_q = (p.L + BM - 1) / BM;
    const uint32_t page = blockIdx.x / tiles_q;
    const uint32_t q0 = (blockIdx.x % tiles_q) * BM;
    const Ctl ctl{abort_flag, p.status};

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (uint32_t s = 0; s < STAGES; ++s) {
            ptx::mbar_init(k_full(s), 1);
            ptx::mbar_init(k_empty(s), 1);
            ptx::mbar_init(v_full(s), 1);
            ptx::mbar_init(v_empty(s), 1);
            ptx::mbar_init(s_full(s), 1);
            ptx::mbar_init(s_free(s), SOFTMAX_WARPS);   // one arrival per softmax warp
        }
        ptx::mbar_init(p_full, SOFTMAX_WARPS);
        ptx::mbar_init(o_full, 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tm_q);
        ptx::prefetch_tensormap(&tm_k);
        ptx::prefetch_tensormap(&tm_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (one thread)
        if (lane == 0) {
            ptx::mbar_arrive_expect_tx(q_full, C::TILE_BYTES);
            for (uint32_t a = 0; a < C::ATOMS; ++a)
                ptx::tma_load_3d(q_base + a * ATOM_BYTES, &tm_q, q_full, int32_t(a * 64), int32_t(q0), int32_t(page));
            bool ok = true;
            for (uint32_t j = 0; ok && j < p.num_kv; ++j) {
                const uint32_t st = j % STAGES, ph = (j / STAGES) & 1u;
                ok = bounded_wait(k_empty(st), ph ^ 1u, ctl, 0x11, 64);
                if (!ok) break;
                ptx::mbar_arrive_expect_tx(k_full(st), C::TILE_BYTES);
                for (uint32_t a = 0; a < C::ATOMS; ++a)
                    ptx::tma_load_3d(k_base(st) + a * ATOM_BYTES, &tm_k, k_full(st), int32_t(a * 64), int32_t(j * BN), int32_t(page));
                ok = bounded_wait(v_empty(st), ph ^ 1u, ctl, 0x12, 64);
                if (!ok) break;
                ptx::mbar_arrive_expect_tx(v_full(st), C::TILE_BYTES);
                for (uint32_t a = 0; a < C::ATOMS; ++a)
                    ptx::tma_load_3d(v_base(st) + a * ATOM_BYTES, &tm_v, v_full(st), int32_t(a * 64), int32_t(j * BN), int32_t(page));
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ Q.K^T issuer (one thread)
        // The two products are issued by two threads: one thread spends ~60 cycles per MMA and ~150 per
        // commit, and sixteen N = 128 MMAs plus four commits per tile cost more than the MMAs take.
        if (lane == 0) {
            const uint64_t kmajor = ptx::umma_desc_base_sw128(16, 1024);
            bool ok = bounded_wait(q_full, 0, ctl, 0x21);
            for (uint32_t j = 0; ok && j < p.num_kv; ++j) {
                const uint32_t st = j % STAGES;
                if (j >= 2) {   // this score buffer was last used by tile j - 2
                    ok = bounded_wait(s_free(j & 1u), ((j - 2) / 2) & 1u, ctl, 0x23);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                }
                ok = bounded_wait(k_full(st), (j / STAGES) & 1u, ctl, 0x24);
                if (!ok) break;
                // S_j = Q.K_j^T: E / 16 steps; step kk reads 16 head-dimension elements (32 bytes) of atom kk / 4
#pragma unroll
                for (uint32_t kk = 0; kk < E / 16; ++kk) {
                    const uint32_t off = (kk / 4) * ATOM_BYTES + (kk % 4) * 32u;
                    ptx::umma_f16_ss(tmem_base + (j & 1u) * BN, ptx::umma_desc_at(kmajor, q_base + off),
                                     ptx::umma_desc_at(kmajor, k_base(st) + off), p.idesc_qk, kk != 0 ? 1u : 0u);
                }
                ptx::umma_commit(k_empty(st));
                ptx::umma_commit(s_full(j & 1u));
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        // ------------------------------------------------------------ P.V issuer (one thread)
        if (lane == 0) {
            const uint64_t kmajor = ptx::umma_desc_base_sw128(16, 1024);
            const uint64_t mnmajor = ptx::umma_desc_base_sw128(ATOM_BYTES, 1024);   // next 64 columns: one slab further
            bool ok = true;
            for (uint32_t j = 0; ok && j < p.num_kv; ++j) {
                const uint32_t st = j % STAGES;
                ok = bounded_wait(p_full, j & 1u, ctl, 0x25);
                if (!ok) break;
                ok = bounded_wait(v_full(st), (j / STAGES) & 1u, ctl, 0x26);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                // O += P_j.V_j: 8 steps of 16 keys; P is K-major (two atoms of 64 keys), V MN-major (16 key rows = 2048 bytes)
#pragma unroll
                for (uint32_t kk = 0; kk < BN / 16; ++kk) {
                    const uint32_t p_off = (kk / 4) * ATOM_BYTES + (kk % 4) * 32u;
                    ptx::umma_f16_ss(tmem_base + 2 * BN, ptx::umma_desc_at(kmajor, p_base + p_off),
                                     ptx::umma_desc_at(mnmajor, v_base(st) + kk * 2048u), p.idesc_pv, (j | kk) != 0 ? 1u : 0u);
                }
                ptx::umma_commit(v_empty(st));
                ptx::umma_commit(o_full);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ softmax, two threads per query row
        const uint32_t quad = warp & 3u;
        const uint32_t half = (warp - FIRST_SOFTMAX_WARP) >> 2;   // 0: keys 0-63, O columns [0, E/2); 1: the rest
        const uint32_t r = quad * 32u + lane;                     // row of the tile = TMEM lane
        const uint32_t lane_addr = (quad * 32u) << 16;
        const bool bf16 = p.bf16 != 0;
        constexpr uint32_t EH = E / 2;                            // O columns per thread
        const uint32_t o_addr = tmem_base + lane_addr + 2 * BN + half * EH;
        float m = -INFINITY, l = 0.0f;
        bool ok = true;
        // The two threads of a row trade a float through shared memory: each publishes (value, tag)
        // in its slot and polls the partner's slot for the same tag -- a bounded wait like all the
        // others (a hardware barrier between the two warps could not be left if the partner gave up).
        auto trade = [&](volatile unsigned long long *mine, volatile unsigned long long *theirs, float value, uint32_t tag,
                         float &got) -> bool {
            *mine = (static_cast<unsigned long long>(tag) << 32) | __float_as_uint(value);
            for (uint32_t spins = 0;; ++spins) {
                const unsigned long long w = *theirs;
                if (uint32_t(w >> 32) == tag) {
                    got = __uint_as_float(uint32_t(w));
                    return true;
                }
                if ((spins & 0x3F) == 0x3F) {
                    if (*ctl.abort_flag != 0) return false;
                    if (spins > (1u << 24)) {
                        *ctl.abort_flag = 1;
                        if (ctl.status) atomicCAS(ctl.status, 0, SITE_FA | 0x34);
                        return false;
                    }
                }
            }
        };
        // waits (once per tile) until P.V of tile `tile` has completed: O is up to date, P may be rewritten
        auto wait_pv = [&](uint32_t tile, int site) -> bool {
            bool w = lane != 0 || bounded_wait(o_full, tile & 1u, ctl, site, 32);
            w = __shfl_sync(0xffffffffu, int(w), 0) != 0;
            if (w) ptx::tc_fence_after_sync();
            return w;
        };
        for (uint32_t j = 0; ok && j < p.num_kv; ++j) {
            const uint32_t sb = j & 1u;
            ok = lane != 0 || bounded_wait(s_full(sb), (j / 2) & 1u, ctl, 0x31, 32);
            ok = __shfl_sync(0xffffffffu, int(ok), 0) != 0;
            if (!ok) break;
            ptx::tc_fence_after_sync();
            const uint32_t s_addr = tmem_base + lane_addr + sb * BN + half * 64u;
            const uint32_t left = p.S - j * BN;                                   // keys that exist from this tile on
            const uint32_t valid = left > half * 64u ? left - half * 64u : 0u;   // ... among this thread's 64
            // This thread's 64 scores, read once (both loads in flight together) and kept in registers.
            uint32_t sv[2][32];
            ptx::tmem_ld_32x32b_x32(s_addr, sv[0]);
            ptx::tmem_ld_32x32b_x32(s_addr + 32u, sv[1]);
            ptx::tmem_ld_wait();
            if (valid < 64u) {
#pragma unroll
                for (uint32_t c = 0; c < 2; ++c)
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i)
                        if (c * 32 + i >= valid) sv[c][i] = 0xff800000u;   // -inf: exp gives 0, max ignores it
            }
            // the score buffer may be multiplied into again
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(s_free(sb));
            // maximum of the raw scores (the scale is positive, so it commutes with max); four chains
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (uint32_t c = 0; c < 2; ++c)
#pragma unroll
                for (uint32_t i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            float other_mx;
            ok = trade(xchg + (sb * 2 + half) * BM + r, xchg + (sb * 2 + (half ^ 1u)) * BM + r, mx, j + 1, other_mx);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float m_cand = fmaxf(m, fmaxf(mx, other_mx) * p.scale_log2);
            // The reference point m only has to keep exp2(x - m) in range, so it is moved (and the sums
            // so far rescaled) only when the maximum has grown by more than 2^8; until then P.V simply
            // keeps accumulating into the same O in tensor memory and nobody has to touch it.
            const bool move = m_cand - m > 8.0f;                  // true on the first tile (m = -inf)
            bool pv_done = j == 0;
            if (__any_sync(0xffffffffu, move)) {
                const float alpha = move ? ex2(m - m_cand) : 1.0f;
                if (move) m = m_cand;
                l *= alpha;
                if (j > 0) {
                    ok = wait_pv(j - 1, 0x32);
                    if (!ok) break;
                    pv_done = true;
#pragma unroll
                    for (uint32_t c = 0; c < EH / 32; ++c) {
                        uint32_t v[32];
                        ptx::tmem_ld_32x32b_x32(o_addr + c * 32u, v);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
                        ptx::tmem_st_32x32b_x32(o_addr + c * 32u, v);
                    }
                    ptx::tmem_st_wait();
                    ptx::tc_fence_before_sync();
                }
            }
            // exponentials and row sum (four chains); P packed to 16 bits in registers
            uint32_t pw[8][4];
            float l4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (uint32_t c = 0; c < 2; ++c) {
                float e[32];
#pragma unroll
                for (uint32_t i = 0; i < 32; ++i) {
                    e[i] = ex2(fmaf(__uint_as_float(sv[c][i]), p.scale_log2, -m));
                    l4[i & 3] += e[i];
                }
#pragma unroll
                for (uint32_t q = 0; q < 4; ++q)
#pragma unroll
                    for (uint32_t h = 0; h < 4; ++h) pw[c * 4 + q][h] = pack16(e[q * 8 + 2 * h], e[q * 8 + 2 * h + 1], bf16);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            // P of the previous tile must have been consumed before it is overwritten
            if (!pv_done) {
                ok = wait_pv(j - 1, 0x35);
                if (!ok) break;
            }
#pragma unroll
            for (uint32_t piece = 0; piece < 8; ++piece)          // eight 16-byte pieces of 8 keys, swizzled A operand
                ptx::sts128(p_base + half * ATOM_BYTES + r * 128u + ((piece ^ (r & 7u)) * 16u), pw[piece]);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(p_full);
        }
        if (ok && p.num_kv > 0) ok = wait_pv(p.num_kv - 1, 0x33);
        if (ok) {
            // the row sum is the sum of the two partial sums (both relative to the same m)
            float other_l;
            ok = trade(xchg + (4 + half) * BM + r, xchg + (4 + (half ^ 1u)) * BM + r, l, 1u, other_l);
            l += other_l;
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            const float inv = p.num_kv > 0 ? 1.0f / l : 0.0f;
            uint8_t *dst = static_cast<uint8_t *>(p.out) + ((size_t(page) * p.L + q0 + r) * E + half * EH) * 2;
#pragma unroll
            for (uint32_t c = 0; c < EH / 32; ++c) {
                uint32_t v[32];
                ptx::tmem_ld_32x32b_x32(o_addr + c * 32u, v);
                ptx::tmem_ld_wait();
                if (q0 + r < p.L) {
#pragma unroll
                    for (uint32_t i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack16(__uint_as_float(v[8 * i + 0]) * inv, __uint_as_float(v[8 * i + 1]) * inv, bf16);
                        w.y = pack16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv, bf16);
                        w.z = pack16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv, bf16);
                        w.w = pack16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv, bf16);
                        reinterpret_cast<uint4 *>(dst + c * 64)[i] = w;
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        if (*abort_flag != 0) {
            for (int i = 0; i < 256; ++i) __nanosleep(1000);   // let copies and MMAs in flight land
        }
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace fa


int umma_status_address(int **out);
int make_tensor_map_3d(CUtensorMap *map, int dtype, const void *base, uint64_t inner, uint64_t outer, uint64_t batch,
                       uint32_t box_inner, uint32_t box_outer);

template <uint32_t E>
static int launch_sdpa_e(const CUtensorMap &tq, const CUtensorMap &tk, const CUtensorMap &tv, const fa::Params &p,
                         unsigned grid, cudaStream_t stream) {
    static std::atomic<bool> configured[64] = {};
    int dev = 0;
    KLAS_TRY_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        KLAS_TRY_CUDA(cudaFuncSetAttribute(fa::sdpa_fused_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           int(fa::Cfg<E>::SMEM)));
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    fa::sdpa_fused_kernel<E><<<grid, fa::THREADS, fa::Cfg<E>::SMEM, stream>>>(tq, tk, tv, p);
    return check_cuda(cudaGetLastError(), "sdpa_fused_kernel launch");
}

int launch_sdpa_fused(int dtype, uint32_t pages, uint64_t l, uint64_t s, uint64_t e, const void *Q, const void *K,
                      const void *V, void *out, float scale, cudaStream_t stream) {
    if (dtype != KLAS_F16 && dtype != KLAS_BF16) return fail(KLAS_ERR_INVALID, "sdpa_fused: dtype must be KLAS_F16 or KLAS_BF16");
    if (e != 64 && e != 128) return fail(KLAS_ERR_UNSUPPORTED, "sdpa_fused: head dimension %llu (64 and 128 are built)", (unsigned long long)e);
    if (pages == 0 || l == 0) return KLAS_OK;
    if (s == 0) return fail(KLAS_ERR_INVALID, "sdpa_fused: no keys (s == 0)");
    if (!(scale > 0.0f) || !(scale < 3.0e38f)) return fail(KLAS_ERR_INVALID, "sdpa_fused: scale must be positive and finite");
    if (!Q || !K || !V || !out) return fail(KLAS_ERR_INVALID, "sdpa_fused: null pointer");
    if ((reinterpret_cast<uintptr_t>(Q) | reinterpret_cast<uintptr_t>(K) | reinterpret_cast<uintptr_t>(V) |
         reinterpret_cast<uintptr_t>(out)) & 15u)
        return fail(KLAS_ERR_INVALID, "sdpa_fused: Q, K, V and out must be 16-byte aligned");
    if (l > 0x7fffffffull || s > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "sdpa_fused: dimension beyond 2^31-1");
    DeviceInfo info;
    if (int rc = device_info(&info)) return rc;
    if (info.cc_major != 10) return fail(KLAS_ERR_UNSUPPORTED, "sdpa_fused needs an sm_100 device");
    const uint64_t tiles_q = (l + fa::BM - 1) / fa::BM;
    if (tiles_q * pages > 0x7fffffffull) return fail(KLAS_ERR_TOO_LARGE, "sdpa_fused: too many query tiles for one grid");
    fa::Params p{};
    p.out = out;
    p.L = uint32_t(l);
    p.S = uint32_t(s);
    p.pages = pages;
    p.num_kv = uint32_t((s + fa::BN - 1) / fa::BN);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.bf16 = dtype == KLAS_BF16 ? 1u : 0u;
    p.idesc_qk = ptx::umma_idesc_f16(dtype == KLAS_BF16, false, false, fa::BM, fa::BN);
    p.idesc_pv = ptx::umma_idesc_f16(dtype == KLAS_BF16, false, true, fa::BM, uint32_t(e));
    if (int rc = umma_status_address(&p.status)) return rc;
    CUtensorMap tq{}, tk{}, tv{};
    if (int rc = make_tensor_map_3d(&tq, dtype, Q, e, l, pages, 64, fa::BM)) return rc;
    if (int rc = make_tensor_map_3d(&tk, dtype, K, e, s, pages, 64, fa::BN)) return rc;
    if (int rc = make_tensor_map_3d(&tv, dtype, V, e, s, pages, 64, fa::BN)) return rc;
    const unsigned grid = unsigned(tiles_q * pages);
    return e == 64 ? launch_sdpa_e<64>(tq, tk, tv, p, grid, stream) : launch_sdpa_e<128>(tq, tk, tv, p, grid, stream);
}

}  // namespace klas
