// Comparison copy of the reference's SpMM unit (FStarLang/kuiper dist/Klas_SPMM.cu, included from
// where it lies) with its size guards compiled out.  The reference's wrappers refuse rows, shared
// or cols >= 10000 (dist/Klas_SPMM.cu:196-198; the FIXME in
// src/lib/sparse/Kuiper.Sparse.SPMM.fst:2164-2169), which rules out the benchmark's 131072^2
// matrix; the kernels themselves index with 32-bit products that stay below 2^32 there
// (131072 * 256 = 2^25 elements of C, 8.4 M nonzeros), so only the guard stands in the way of
// timing them.  Used for the "reference kernel on the same GPU" comparison row only.
// Compile with: -I <kuiper>/include -I <kuiper>/dist
#include <kuiper.h>
#undef KPR_GUARD
#define KPR_GUARD(b) ((void)0)
#include "Klas_SPMM.cu"
