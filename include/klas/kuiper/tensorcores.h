/*
 * kuiper/tensorcores.h of the runtime shim: the fragment helpers that code extracted from
 * Kuiper.Kernel.GEMM.TensorCore* is written against (FStarLang/kuiper
 * include/kuiper/tensorcores.h:9-59), over the warp-level nvcuda::wmma API.  This library's own
 * tensor-core kernels do not use them (they issue tcgen05 instructions); the header exists so
 * that extracted code which includes <kuiper.h> still compiles against this include directory.
 *
 * The element-wise hooks are macros because the generated code passes them an EXPRESSION written
 * in terms of fixed local names: `_kpr_i` (register index), `_kpr_in_v` (loaded value),
 * `_kpr_old_v` / `_kpr_new_v` (resident value / accumulator value).
 */
#ifndef KUIPER_TENSORCORES_H
#define KUIPER_TENSORCORES_H 1

#include <stdint.h>
#include <mma.h>
using namespace nvcuda;

#define kpr_fragment(...) wmma::fragment<__VA_ARGS__>
#define KPR_INIT(ty) (ty){0}
#define KPR_INIT_ARR(ty, size) (ty[size]){0}

#define KPR_NELEM(fr) ((fr).num_elements)
#define KPR_FRAG_GET(fr, i) ((fr).x[(i)])
#define KPR_FRAG_SET(fr, i, v) ((fr).x[(i)] = (v))

/* load a fragment, then replace every register by `mapped` (an expression over _kpr_in_v) */
#define KPR_LOAD_MAP(gm, fr, ldm, mapped)                                    \
    do {                                                                     \
        wmma::load_matrix_sync((fr), (gm), (ldm));                           \
        const uint32_t _kpr_n = KPR_NELEM(fr);                               \
        for (uint32_t _kpr_i = 0; _kpr_i < _kpr_n; ++_kpr_i) {               \
            [[maybe_unused]] const auto _kpr_in_v = KPR_FRAG_GET(fr, _kpr_i); \
            KPR_FRAG_SET(fr, _kpr_i, (mapped));                              \
        }                                                                    \
    } while (0)

/* read the resident tile, combine it register by register with the accumulator `fr` through
 * `combined` (an expression over _kpr_old_v and _kpr_new_v), store the result */
#define KPR_STORE_COMB(gm, fr, ldm, combined)                                       \
    do {                                                                            \
        auto _kpr_old = (fr);                                                       \
        wmma::load_matrix_sync(_kpr_old, (gm), (ldm), wmma::mem_row_major);         \
        const uint32_t _kpr_n = KPR_NELEM(fr);                                      \
        for (uint32_t _kpr_i = 0; _kpr_i < _kpr_n; ++_kpr_i) {                      \
            [[maybe_unused]] const auto _kpr_old_v = KPR_FRAG_GET(_kpr_old, _kpr_i); \
            [[maybe_unused]] const auto _kpr_new_v = KPR_FRAG_GET(fr, _kpr_i);      \
            KPR_FRAG_SET(fr, _kpr_i, (combined));                                   \
        }                                                                           \
        wmma::store_matrix_sync((gm), (fr), (ldm), wmma::mem_row_major);            \
    } while (0)

#endif /* KUIPER_TENSORCORES_H */
