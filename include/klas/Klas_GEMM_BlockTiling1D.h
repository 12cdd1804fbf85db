/* Klas_GEMM_BlockTiling1D.h -- prototypes of the reference's Klas_GEMM_BlockTiling1D entry points (FStarLang/kuiper dist/Klas_GEMM_BlockTiling1D.h),
 * served by libklas_b200.so through the Klas_GEMM_BlockTiling1D compatibility object.  C++ linkage, as in the reference. */
#ifndef Klas_GEMM_BlockTiling1D_H
#define Klas_GEMM_BlockTiling1D_H

#include <kuiper.h>
#include "klas_signatures.h"

#define KLAS_ENTRY(name, params, ...) void name params;
KLAS_NUM_TYPES(KLAS_BT1D_ENTRIES, BlockTiling1D)
#undef KLAS_ENTRY

#define Klas_GEMM_BlockTiling1D_H_DEFINED
#endif /* Klas_GEMM_BlockTiling1D_H */
